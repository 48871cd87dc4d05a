"""Seeded random-init checkpoints with the reference's parameter names.

Names follow the module tree of /root/reference/phi.py (Phi3ForCausalLM phi:599-617,
Phi3ImageEmbedding phi:374-391, ClipModel phi:208-221), i.e. the HF safetensors keys the
reference loads at /root/reference/phi_3_vision_mlx.py:265,371-374 (patch_embedding weight
already in the reference's post-transpose [O,kh,kw,I] layout).
All tensors are bf16 (HF checkpoints are bf16); the CPU oracle and the CUDA path are fed
the same dict. There is no network in this environment, so benchmarks and parity tests
use these instead of the published checkpoints (stated in bench.py's `data` field).
"""
import torch
from .configs import CLIP_VIT_L14_336


def _names(cfg, clip_cfg, vision):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    hd = H // cfg.num_attention_heads
    qkv = cfg.num_attention_heads * hd + 2 * cfg.num_key_value_heads * hd
    out = [('model.embed_tokens.weight', (V, H), 'emb')]
    for i in range(cfg.num_hidden_layers):
        p = f'model.layers.{i}.'
        out += [(p + 'input_layernorm.weight', (H,), 'norm'), (p + 'self_attn.qkv_proj.weight', (qkv, H), 'lin'),
                (p + 'self_attn.o_proj.weight', (H, cfg.num_attention_heads * hd), 'res'),
                (p + 'post_attention_layernorm.weight', (H,), 'norm'),
                (p + 'mlp.gate_up_proj.weight', (2 * I, H), 'lin'), (p + 'mlp.down_proj.weight', (H, I), 'res')]
    out += [('model.norm.weight', (H,), 'norm'), ('lm_head.weight', (V, H), 'lin')]
    if vision:
        c = clip_cfg
        D, F = c.hidden_size, c.intermediate_size
        P = 'model.vision_embed_tokens.img_processor.vision_model.'
        npos = (c.image_size // c.patch_size) ** 2 + 1
        out += [(P + 'embeddings.class_embedding', (D,), 'b'),
                (P + 'embeddings.patch_embedding.weight', (D, c.patch_size, c.patch_size, c.num_channels), 'lin'),
                (P + 'embeddings.position_embedding.weight', (npos, D), 'b'),
                (P + 'pre_layrnorm.weight', (D,), 'norm'), (P + 'pre_layrnorm.bias', (D,), 'b')]
        for j in range(c.num_hidden_layers):
            L = P + f'encoder.layers.{j}.'
            for n in ('q_proj', 'k_proj', 'v_proj', 'out_proj'):
                out += [(L + f'self_attn.{n}.weight', (D, D), 'cres' if n == 'out_proj' else 'lin'),
                        (L + f'self_attn.{n}.bias', (D,), 'b')]
            out += [(L + 'layer_norm1.weight', (D,), 'norm'), (L + 'layer_norm1.bias', (D,), 'b'),
                    (L + 'layer_norm2.weight', (D,), 'norm'), (L + 'layer_norm2.bias', (D,), 'b'),
                    (L + 'mlp.fc1.weight', (F, D), 'lin'), (L + 'mlp.fc1.bias', (F,), 'b'),
                    (L + 'mlp.fc2.weight', (D, F), 'cres'), (L + 'mlp.fc2.bias', (D,), 'b')]
        out += [(P + 'post_layernorm.weight', (D,), 'norm'), (P + 'post_layernorm.bias', (D,), 'b')]
        E = cfg.img_processor['image_dim_out'] * 4
        Vp = 'model.vision_embed_tokens.'
        out += [(Vp + 'glb_GN', (1, 1, E), 'gn'), (Vp + 'sub_GN', (1, 1, 1, E), 'gn'),
                (Vp + 'img_projection.0.weight', (H, E), 'lin'), (Vp + 'img_projection.0.bias', (H,), 'b'),
                (Vp + 'img_projection.2.weight', (H, H), 'lin'), (Vp + 'img_projection.2.bias', (H,), 'b')]
    return out


PEAK_ALPHA = 0.01


def random_weights(cfg, seed=0, device='cpu', clip_cfg=None, vision=None, init='gpt2'):
    """N(0,sigma) bf16 tensors, GPT-2-style: linear 0.02, residual-writing projections (o_proj,
    down_proj, CLIP out_proj/fc2) 0.02/sqrt(2*n_layers), embedding 1.0, norm gains 1+0.1*N,
    biases/pos 0.1*N, GN separators N(0,1). With the residual scaling the residual stream stays
    O(1) over 32 layers and the random network is not chaotic (a plain 0.02 init amplifies a 1e-3
    perturbation ~25x by layer 32, which says nothing about kernel accuracy); logits have O(1)
    spread (SURVEY.md §7 hard part 1).

    init='peaked' (the parity checkpoint): identical tensors, except that lm_head is TIED to the embedding through a
    fixed seeded permutation, lm_head[t] = PEAK_ALPHA * embed[perm[t]]. The residual stream of this init keeps a cosine
    of ~0.68 with the input embedding through all 32 layers, so every position has ONE logit of ~20 over a N(0, 0.6)
    background: the top-1 / top-2 margin (~17) is far above the bf16 noise of any correct implementation (~2e-2 of the
    peak), which makes "greedy ids agree on >= 99 % of positions" a property of the kernels instead of a coin flip at
    the noise floor. Greedy generation walks the permutation (x -> perm^-1(x)), so the rollout is not a repeated
    token. The flat 'gpt2' init (median margin 0.18) stays available to measure the noise floor itself."""
    assert init in ('gpt2', 'peaked')
    if vision is None:
        vision = 'V' in cfg.architectures[0]
    clip_cfg = clip_cfg or CLIP_VIT_L14_336
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape, kind in _names(cfg, clip_cfg, vision):
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        if kind == 'lin':
            t.mul_(0.02)
        elif kind == 'res':
            t.mul_(0.02 / (2 * cfg.num_hidden_layers) ** 0.5)
        elif kind == 'cres':
            t.mul_(0.02 / (2 * clip_cfg.num_hidden_layers) ** 0.5)
        elif kind == 'norm':
            t.mul_(0.1).add_(1.0)
        elif kind == 'b':
            t.mul_(0.1)
        w[name] = t.to(torch.bfloat16)
    if init == 'peaked':
        perm = torch.randperm(cfg.vocab_size, generator=torch.Generator().manual_seed(seed + 12345))
        emb = w['model.embed_tokens.weight'].to(torch.float32)
        w['lm_head.weight'] = (PEAK_ALPHA * emb[perm.to(emb.device)]).to(torch.bfloat16)
    return w


def tagenex_tensor_shapes(cfg):
    """name -> shape of every tensor of a Tagenex checkpoint; cfg = the config.json dict"""
    W, V = cfg['width'], cfg['vocab']
    out = {'embed': (V, W)}
    for i, lc in enumerate(cfg['layers']):
        p, m = f'l{i}.', lc['mixer']
        H, G, d = m['heads'], m.get('kv_heads', m['heads']), m['dim']
        dv = m.get('vdim', d)
        out.update({p + 'norm1': (W,), p + 'mix.q': (H * d, W), p + 'mix.k': (G * d, W), p + 'mix.v': (G * dv, W),
                    p + 'mix.q.norm': (d,), p + 'mix.k.norm': (d,), p + 'mix.vmix': (), p + 'mix.r1': (H,), p + 'mix.r2': (H,),
                    p + 'mix.sink': (H,), p + 'mix.g': (H, W), p + 'mix.o': (W, H * dv)})
        f = lc.get('mlp')
        if f is None:
            continue
        out[p + 'norm2'] = (W,)
        if f['kind'] == 'dense':
            F = f['ff']
            out.update({p + 'mlp.gate': (F, W), p + 'mlp.gate.b': (F,), p + 'mlp.up': (F, W), p + 'mlp.up.b': (F,),
                        p + 'mlp.down': (W, F), p + 'mlp.down.b': (W,)})
        else:
            F, E = f['expert']['ff'], f['router']['experts']
            for e in range(E):
                out.update({f'{p}mlp.e{e}.gate': (F, W), f'{p}mlp.e{e}.up': (F, W), f'{p}mlp.e{e}.down': (W, F)})
            out.update({p + 'mlp.router': (E, W), p + 'mlp.router.b': (E,)})
    out.update({'final.norm': (W,), 'head': (V, W)})
    return out


def random_tagenex_weights(cfg, seed=0, device='cpu'):
    """Seeded bf16 tensors for a Tagenex config dict: matrices N(0, 1/fan_in), embedding N(0,1), norm gains 1 + 0.1 N (sublayer
    norms 0.5 + 0.1 N so the residual grows slowly), biases 0.3 N, router logits of unit spread, penalties r1 in [0.2, 1.2],
    r2 in [0.05, 1], sinks N(0,1), mixing weight in [0.2, 0.8]."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda s: torch.randn(s, generator=g, device=device, dtype=torch.float32)
    ru = lambda s, lo, hi: torch.rand(s, generator=g, device=device, dtype=torch.float32) * (hi - lo) + lo
    w = {}
    for name, shape in tagenex_tensor_shapes(cfg).items():
        leaf = name.split('.', 1)[1] if name.startswith('l') and '.' in name else name
        if name == 'embed':
            t = rn(shape)
        elif leaf in ('norm1', 'norm2'):
            t = 0.5 + 0.1 * rn(shape)
        elif leaf.endswith('norm'):
            t = 1.0 + 0.1 * rn(shape)
        elif leaf == 'mix.vmix':
            t = ru(shape, 0.2, 0.8)
        elif leaf == 'mix.r1':
            t = ru(shape, 0.2, 1.2)
        elif leaf == 'mix.r2':
            t = ru(shape, 0.05, 1.0)
        elif leaf == 'mix.sink':
            t = rn(shape)
        elif leaf.endswith('.b'):
            t = 0.3 * rn(shape)
        elif leaf == 'mlp.router':
            t = rn(shape) * (3.0 / shape[1] ** 0.5)
        else:
            t = rn(shape) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def tapalix_tensor_shapes(cfg):
    """name -> shape of every tensor of a Tapalix checkpoint; cfg = the config.json dict"""
    W, V = cfg['width'], cfg['vocab']
    out = {'embed': (V, W)}
    if cfg.get('loop'):
        out['loop.in'] = (W, 2 * W)
    for i, lc in enumerate(cfg['layers']):
        p, m = f'l{i}.', lc['mixer']
        H, d, R = m['heads'], m['dim'], m['kv_rank']
        dv = m.get('vdim', d)
        dr = m.get('rot_dim', 0) if lc['type'] == 'latent_attention' else 0
        out.update({p + 'norm1': (W,), p + 'norm1.b': (W,), p + 'mix.q': (H * (d + dr), W), p + 'mix.dkv': (R + dr, W),
                    p + 'mix.dkv.norm': (R,), p + 'mix.uk': (H * d, R), p + 'mix.uv': (H * dv, R)})
        if lc['type'] == 'latent_attention_2':
            out[p + 'mix.g'] = (H * dv, W)
        out[p + 'mix.o'] = (W, H * dv)
        f = lc.get('mlp')
        if f is None:
            continue
        F, E = f['expert']['ff'], f['router']['experts']
        for e in range(E):
            out.update({f'{p}mlp.e{e}.gate': (F, W), f'{p}mlp.e{e}.up': (F, W), f'{p}mlp.e{e}.down': (W, F)})
        out.update({p + 'mlp.router': (E, W), p + 'mlp.correction': (E,)})
        if f.get('shared'):
            S = f['shared']['ff']
            out.update({p + 'mlp.shared.gate': (S, W), p + 'mlp.shared.up': (S, W), p + 'mlp.shared.down': (W, S)})
    out.update({'final.norm': (W,), 'final.norm.b': (W,), 'head': (V, W)})
    return out


def random_tapalix_weights(cfg, seed=0, device='cpu'):
    """Seeded bf16 tensors for a Tapalix config dict: matrices N(0, 1/fan_in) (the embedding N(0, 1/width), since the design
    scales it up again; sublayer output matrices at half that spread so the residual grows slowly), norm gains 1 + 0.1 N, norm
    biases 0.1 N, router logits of unit spread, choice corrections 0.3 N (large enough to change which experts win)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda s: torch.randn(s, generator=g, device=device, dtype=torch.float32)
    w = {}
    for name, shape in tapalix_tensor_shapes(cfg).items():
        leaf = name.split('.', 1)[1] if name.startswith('l') and name[1].isdigit() else name
        if leaf.endswith('.b'):
            t = 0.1 * rn(shape)
        elif leaf.endswith('norm') or leaf.endswith('norm1'):
            t = 1.0 + 0.1 * rn(shape)
        elif leaf == 'mlp.correction':
            t = 0.3 * rn(shape)
        elif leaf == 'mlp.router':
            t = rn(shape) * (3.0 / shape[1] ** 0.5)
        elif leaf == 'mix.o' or leaf.endswith('.down'):
            t = 0.5 * rn(shape) / shape[-1] ** 0.5
        else:
            t = rn(shape) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def dugalix_tensor_shapes(cfg):
    """name -> shape of every tensor of a Dugalix checkpoint; cfg = the config.json dict"""
    W, V = cfg['width'], cfg['vocab']
    out = {'embed': (V, W)}

    def attention(p, m, biased, values):
        H, G, d = m['heads'], m.get('kv_heads', m['heads']), m['dim']
        dv = m.get('vdim', d)
        out.update({p + 'q': (H * d, W), p + 'k': (G * d, W)})
        if values:
            out[p + 'v'] = (G * dv, W)
        out[p + 'o'] = (W, H * dv)
        if biased:
            out.update({p + 'q.b': (H * d,), p + 'k.b': (G * d,), p + 'v.b': (G * dv,), p + 'o.b': (W,)})
        else:
            out[p + 'pb'] = (H,)

    for i, lc in enumerate(cfg['layers']):
        p, m = f'l{i}.', lc['mixer']
        out.update({p + 'norm1': (W,), p + 'norm1b': (W,), p + 'shift': (W,)})
        if lc['type'] == 'parallel':
            attention(p + 'mix.left.', m['left'], True, True)
            r = m['right']
            H, d = r['heads'], r['dim']
            dv = r.get('vdim', d)
            q = p + 'mix.right.'
            out.update({q + 'q': (H * d, W), q + 'k': (H * d, W), q + 'v': (H * dv, W), q + 'g': (H * dv, W), q + 'o': (W, H * dv),
                        q + 'norm': (H * dv,), q + 'i': (H, W), q + 'i.b': (H,), q + 'f': (H, W), q + 'f.b': (H,)})
        else:
            attention(p + 'mix.', m, False, False)
        f = lc.get('mlp')
        if f is None:
            continue
        out.update({p + 'norm2': (W,), p + 'norm2b': (W,)})
        if f['kind'] == 'dense':
            out.update({p + 'mlp.up': (f['ff'], W), p + 'mlp.down': (W, f['ff'])})
            continue
        F, E = f['expert']['ff'], f['router']['experts']
        n_out = E + int(f['router'].get('identity') or 0)
        for e in range(E):
            out.update({f'{p}mlp.e{e}.up': (F, W), f'{p}mlp.e{e}.down': (W, F)})
        out.update({p + 'mlp.router': (n_out, W), p + 'mlp.correction': (n_out,)})
        if f.get('shared'):
            S = f['shared']['ff']
            out.update({p + 'mlp.shared.up': (S, W), p + 'mlp.shared.down': (W, S), p + 'mlp.shared.sg': (1, W)})
    out.update({'final.norm': (W,), 'head': (V, W)})
    return out


def random_dugalix_weights(cfg, seed=0, device='cpu'):
    """Seeded bf16 tensors for a Dugalix config dict: matrices N(0, 1/fan_in), the embedding of unit spread, norm gains (stored
    around zero) 0.1 N, biases 0.1 N except the gate biases of the matrix memory (input gates around -1, forget gates around 3 so
    that the memory reaches back over tens of tokens), per-head score biases around -2 (sigmoid weights add up over the window),
    shift factors uniform in [0, 1], router rows of a spread that gives peaked probabilities and choice corrections of 0.1 N
    (comparable to the probabilities, so that they change which experts win)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda s: torch.randn(s, generator=g, device=device, dtype=torch.float32)
    w = {}
    for name, shape in dugalix_tensor_shapes(cfg).items():
        leaf = name.split('.', 1)[1] if name.startswith('l') and name[1].isdigit() else name
        if leaf.endswith('right.i.b'):
            t = -1.0 + 0.5 * rn(shape)
        elif leaf.endswith('right.f.b'):
            t = 3.0 + rn(shape)
        elif leaf.endswith('.pb'):
            t = -2.0 + 0.5 * rn(shape)
        elif leaf.endswith('.b'):
            t = 0.1 * rn(shape)
        elif leaf == 'shift':
            t = torch.rand(shape, generator=g, device=device, dtype=torch.float32)
        elif leaf == 'embed':
            t = rn(shape)
        elif 'norm' in leaf.rsplit('.', 1)[-1]:
            t = 0.1 * rn(shape)
        elif leaf == 'mlp.correction':
            t = 0.1 * rn(shape)
        elif leaf == 'mlp.router':
            t = rn(shape) * (2.0 / shape[1] ** 0.5)
        else:
            t = rn(shape) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def danalorn_tensor_shapes(cfg):
    """name -> shape of every tensor of a Danalorn checkpoint; cfg = the config.json dict"""
    W, V = cfg['width'], cfg['vocab']
    out = {'embed': (V, W)}
    bg = (cfg.get('embedding') or {}).get('bigram')
    if bg:
        out['bigram'] = (bg['buckets'] + 1, W)
    for i, lc in enumerate(cfg['layers']):
        p, m = f'l{i}.', lc['mixer']
        a = p + 'mix.'
        out.update({p + 'norm1': (W,), p + 'norm1b': (W,)})
        if lc['type'] == 'latent_attention':
            H, d, dr, R, Q = m['heads'], m['dim'], m.get('rot_dim', 0), m['kv_rank'], m['q_rank']
            dv = m.get('vdim', d)
            out.update({a + 'dq': (Q, W), a + 'dq.norm': (Q,), a + 'uq': (H * (d + dr), Q)})
            if m.get('kv_from') is None:
                out.update({a + 'dkv': (R + dr, W), a + 'dkv.norm': (R,)})
            out.update({a + 'uk': (H * d, R), a + 'uv': (H * dv, R), a + 'sink': (H,), a + 'o': (W, H * dv)})
        elif lc['type'] == 'attention':
            H, G, d = m['heads'], m.get('kv_heads', m['heads']), m['dim']
            dv = m.get('vdim', d)
            out.update({a + 'q': (H * d, W), a + 'q.b': (H * d,), a + 'k': (G * d, W), a + 'k.b': (G * d,), a + 'v': (G * dv, W),
                        a + 'v.b': (G * dv,), a + 'q.norm': (d,), a + 'k.norm': (d,), a + 'g': (H * dv, W), a + 'o': (W, H * dv)})
        elif lc['type'] == 'gla':
            H, d = m['heads'], m['dim']
            dv = m.get('vdim', d)
            r = m.get('decay_rank', 16)          # checkpoints fix this by the shape of a1; random ones take 16 unless told otherwise
            out.update({a + 'q': (H * d, W), a + 'k': (H * d, W), a + 'v': (H * dv, W), a + 'g': (H * dv, W), a + 'o': (W, H * dv),
                        a + 'norm': (dv,), a + 'a1': (r, W), a + 'a2': (H * d, r), a + 'a2.b': (H * d,)})
        else:
            raise NotImplementedError(lc['type'])
        f = lc.get('mlp')
        if f is not None:
            out.update({p + 'norm2': (W,), p + 'norm2b': (W,), p + 'mlp.up': (f['ff'], W), p + 'mlp.down': (W, f['ff'])})
    out.update({'final.norm': (W,), 'head': (V, W)})
    return out


def random_danalorn_weights(cfg, seed=0, device='cpu'):
    """Seeded bf16 tensors for a Danalorn config dict: matrices N(0, 1/fan_in), embedding and pair table of unit spread (the pair
    table weighs as much as a scaled token row would not: it has to show beside it, so its spread is that of the scaled rows),
    norm gains around one, biases 0.1 N except the decay biases of the recurrence (around 3 +- 2: decays from a few tokens to
    hundreds), sinks N(0, 1)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda s: torch.randn(s, generator=g, device=device, dtype=torch.float32)
    scale = float((cfg.get('embedding') or {}).get('scale', 1.0))
    w = {}
    for name, shape in danalorn_tensor_shapes(cfg).items():
        leaf = name.split('.', 1)[1] if name.startswith('l') and name[1].isdigit() else name
        if leaf == 'mix.a2.b':
            t = 3.0 + 2.0 * rn(shape)
        elif leaf == 'mix.a2':
            t = 2.0 * rn(shape) / shape[-1] ** 0.5
        elif leaf.endswith('.b'):
            t = 0.1 * rn(shape)
        elif leaf == 'embed':
            t = rn(shape)
        elif leaf == 'bigram':
            t = rn(shape) * scale
        elif leaf == 'mix.sink':
            t = rn(shape)
        elif 'norm' in leaf.rsplit('.', 1)[-1]:
            t = 1.0 + 0.1 * rn(shape)
        else:
            t = rn(shape) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w
