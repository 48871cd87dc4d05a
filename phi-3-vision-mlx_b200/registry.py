"""Model registry: which class serves a checkpoint is decided by its config.json, as load() has always done for the two Phi-3
checkpoints (`architectures`: Phi3ForCausalLM / Phi3VForCausalLM). Designs register a config parser and a model class under the
name their config.json carries in `architectures[0]` or `architecture`.

    entry.config(dict) -> config object        entry.build(cfg, weights, device=..., dtype=..., **kw) -> model
    entry.engine: 'batch' (rectangular batches through api._generate) or 'paged' (engine.Engine / engine.Scheduler)
"""
import json
import os
from types import SimpleNamespace

_REGISTRY = {}


def register(name, config, build, engine):
    _REGISTRY[name] = SimpleNamespace(name=name, config=config, build=build, engine=engine)


def names():
    return sorted(_REGISTRY)


def arch_of(cfg_dict):
    a = cfg_dict.get('architectures')
    if a:
        return a[0]
    return cfg_dict.get('architecture')


def entry_for(cfg_dict):
    name = arch_of(cfg_dict)
    if name not in _REGISTRY:
        raise KeyError(f'no model registered for architecture {name!r} (known: {names()})')
    return _REGISTRY[name]


def read_config(path):
    with open(os.path.join(path, 'config.json')) as f:
        return json.load(f)


def read_weights(path):
    """every *.safetensors file of a checkpoint folder as one name -> tensor dict"""
    import glob
    from safetensors.torch import load_file
    w = {}
    for f in sorted(glob.glob(os.path.join(path, '*.safetensors'))):
        w.update(load_file(f))
    if not w:
        raise FileNotFoundError(f'no *.safetensors under {path}')
    return w


def load_model(path, device='cuda', dtype=None, **kw):
    """checkpoint folder -> model object of the registered class"""
    d = read_config(path)
    ent = entry_for(d)
    if ent.engine == 'batch':
        from . import api
        return api.load(model_path=path, device=device, **kw)[0]
    import torch
    return ent.build(ent.config(d), read_weights(path), device=device, dtype=dtype or torch.bfloat16, **kw)


def _phi3_config(d):
    d = dict(d)
    d.setdefault('use_quantized_cache', False)
    d.setdefault('num_key_value_heads', d.get('num_attention_heads'))
    return SimpleNamespace(**d)


def _phi3_build(cfg, weights, device='cuda', dtype=None, **kw):
    from .model import Phi3B200
    return Phi3B200(cfg, weights, device=device, **kw)


def _tagenex_config(d):
    from .configs import TagenexConfig
    return TagenexConfig(d)


def _tagenex_build(cfg, weights, device='cuda', dtype=None, **kw):
    import torch
    from .tagenex import TagenexB200
    return TagenexB200(cfg, weights, device=device, dtype=dtype or torch.bfloat16)


def _tapalix_config(d):
    from .configs import TapalixConfig
    return TapalixConfig(d)


def _tapalix_build(cfg, weights, device='cuda', dtype=None, **kw):
    import torch
    from .tapalix import TapalixB200
    return TapalixB200(cfg, weights, device=device, dtype=dtype or torch.bfloat16)


def _dugalix_config(d):
    from .configs import DugalixConfig
    return DugalixConfig(d)


def _dugalix_build(cfg, weights, device='cuda', dtype=None, **kw):
    import torch
    from .dugalix import DugalixB200
    return DugalixB200(cfg, weights, device=device, dtype=dtype or torch.bfloat16)


def _danalorn_config(d):
    from .configs import DanalornConfig
    return DanalornConfig(d)


def _danalorn_build(cfg, weights, device='cuda', dtype=None, **kw):
    import torch
    from .danalorn import DanalornB200
    return DanalornB200(cfg, weights, device=device, dtype=dtype or torch.bfloat16)


register('Phi3ForCausalLM', _phi3_config, _phi3_build, 'batch')
register('Phi3VForCausalLM', _phi3_config, _phi3_build, 'batch')
register('Tagenex', _tagenex_config, _tagenex_build, 'paged')
register('Tapalix', _tapalix_config, _tapalix_build, 'paged')
register('Dugalix', _dugalix_config, _dugalix_build, 'paged')
register('Danalorn', _danalorn_config, _danalorn_build, 'paged')
