"""Frozen hyper-parameters for the two checkpoints the reference serves.

The reference reads these at run time from the downloaded HF ``config.json``
(/root/reference/phi_3_vision_mlx.py:258,359-363); none is in its tree, so the
public Phi-3.5-mini-instruct / Phi-3.5-vision-instruct values are frozen here.
LongRoPE factor vectors: /root/reference/assets/su_rope_explained.ipynb:309-310.
CLIP constants: /root/reference/phi.py:375-384.
"""
from types import SimpleNamespace
import copy

SHORT_FACTOR = [1.05, 1.05, 1.05, 1.1, 1.1, 1.1, 1.2500000000000002, 1.2500000000000002, 1.4000000000000004,
                1.4500000000000004, 1.5500000000000005, 1.8500000000000008, 1.9000000000000008, 2.000000000000001,
                2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001,
                2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001,
                2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001, 2.000000000000001,
                2.000000000000001, 2.000000000000001, 2.000000000000001, 2.1000000000000005, 2.1000000000000005, 2.2,
                2.3499999999999996, 2.3499999999999996, 2.3499999999999996, 2.3499999999999996, 2.3999999999999995,
                2.3999999999999995, 2.6499999999999986, 2.6999999999999984, 2.8999999999999977, 2.9499999999999975,
                3.049999999999997, 3.049999999999997, 3.049999999999997]
LONG_FACTOR = [1.0299999713897705, 1.0499999523162842, 1.0499999523162842, 1.0799999237060547, 1.2299998998641968,
               1.2299998998641968, 1.2999999523162842, 1.4499999284744263, 1.5999999046325684, 1.6499998569488525,
               1.8999998569488525, 2.859999895095825, 3.68999981880188, 5.419999599456787, 5.489999771118164,
               5.489999771118164, 9.09000015258789, 11.579999923706055, 15.65999984741211, 15.769999504089355,
               15.789999961853027, 18.360000610351562, 21.989999771118164, 23.079999923706055, 30.009998321533203,
               32.35000228881836, 32.590003967285156, 35.56000518798828, 39.95000457763672, 53.840003967285156,
               56.20000457763672, 57.95000457763672, 59.29000473022461, 59.77000427246094, 59.920005798339844,
               61.190006256103516, 61.96000671386719, 62.50000762939453, 63.3700065612793, 63.48000717163086,
               63.48000717163086, 63.66000747680664, 63.850006103515625, 64.08000946044922, 64.760009765625,
               64.80001068115234, 64.81001281738281, 64.81001281738281]

ID_EOS = 32007   # /root/reference/phi_3_vision_mlx.py:42
ID_ASS = 32001   # /root/reference/phi_3_vision_mlx.py:43

CLIP_VIT_L14_336 = SimpleNamespace(hidden_size=1024, image_size=336, intermediate_size=4096, layer_norm_eps=1e-5,
                                   num_attention_heads=16, num_channels=3, num_hidden_layers=24, patch_size=14)

PHI35_MINI = SimpleNamespace(
    architectures=["Phi3ForCausalLM"], hidden_size=3072, num_hidden_layers=32, num_attention_heads=32,
    num_key_value_heads=32, intermediate_size=8192, vocab_size=32064, rms_norm_eps=1e-5, rope_theta=10000.0,
    max_position_embeddings=131072, original_max_position_embeddings=4096,
    rope_scaling={"type": "su", "short_factor": SHORT_FACTOR, "long_factor": LONG_FACTOR},
    use_quantized_cache=False)

PHI35_VISION = copy.deepcopy(PHI35_MINI)
PHI35_VISION.architectures = ["Phi3VForCausalLM"]
PHI35_VISION.img_processor = {"image_dim_out": 1024, "num_img_tokens": 144}


def tiny(vision=False, layers=2, **kw):
    """Small same-shaped-head config (head_dim stays 96) for quick parity runs."""
    c = copy.deepcopy(PHI35_VISION if vision else PHI35_MINI)
    c.hidden_size, c.num_attention_heads, c.num_key_value_heads = 384, 4, 4
    c.intermediate_size, c.num_hidden_layers, c.vocab_size = 1024, layers, 32064
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def tiny_clip(layers=3):
    c = copy.deepcopy(CLIP_VIT_L14_336)
    c.num_hidden_layers = layers
    return c


def with_overrides(cfg, **kw):
    c = copy.deepcopy(cfg)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


# ------------------------------------------------------------------------------------------------ Tagenex
class TagenexConfig:
    """config.json of a Tagenex checkpoint: {"architecture": "Tagenex", "vocab", "width", "norm": {"eps"}, "layers": [...]}.
    Every layer entry has "type" (the mixer kind; "attention"), "mixer" (heads, kv_heads, dim, vdim, scale, v_mix,
    mask: {size} or absent = no window) and "mlp": null | {"kind": "dense", ff, limit} | {"kind": "moe", expert: {ff, limit},
    router: {experts, top}}. Nothing is assumed equal between layers except the value shape of the layers that mix values."""
    GLU_ALPHA = 1.702          # slope of the sigmoid in the gated activation: fixed by the design

    def __init__(self, d):
        self.raw = d
        self.architecture = d.get('architecture', 'Tagenex')
        self.architectures = [self.architecture]
        self.vocab_size, self.width = int(d['vocab']), int(d['width'])
        self.eps = float(d['norm']['eps'])
        self.layers = []
        first_mix = None
        for i, lc in enumerate(d['layers']):
            if lc.get('type', 'attention') != 'attention':
                raise NotImplementedError(f"layer {i}: mixer type {lc.get('type')!r} is not part of this design")
            m = lc['mixer']
            mixer = SimpleNamespace(kind='attention', heads=int(m['heads']), kv_heads=int(m.get('kv_heads', m['heads'])),
                                    dim=int(m['dim']), vdim=int(m.get('vdim', m['dim'])), scale=float(m['scale']),
                                    window=int((m.get('mask') or {}).get('size') or 0), v_mix=bool(m.get('v_mix', False)),
                                    v_role='none')
            if mixer.heads % mixer.kv_heads:
                raise ValueError(f'layer {i}: heads must be a multiple of kv_heads')
            if mixer.v_mix:
                if first_mix is None:
                    first_mix, mixer.v_role = mixer, 'source'
                else:
                    if (mixer.kv_heads, mixer.vdim) != (first_mix.kv_heads, first_mix.vdim):
                        raise ValueError(f'layer {i}: value mixing needs the value shape of the first mixing layer')
                    mixer.v_role = 'mix'
            f = lc.get('mlp')
            if f is None:
                ff = None
            elif f['kind'] == 'dense':
                ff = SimpleNamespace(kind='dense', ff=int(f['ff']), limit=float(f['limit']))
            elif f['kind'] == 'moe':
                ff = SimpleNamespace(kind='moe', ff=int(f['expert']['ff']), limit=float(f['expert']['limit']),
                                     experts=int(f['router']['experts']), top=int(f['router']['top']))
                if not 1 <= ff.top <= ff.experts:
                    raise ValueError(f'layer {i}: top must be in [1, experts]')
            else:
                raise NotImplementedError(f"layer {i}: feed-forward kind {f['kind']!r}")
            self.layers.append(SimpleNamespace(mixer=mixer, ff=ff))
        self.num_hidden_layers = len(self.layers)

    def kv_layout(self):
        """per layer (kv heads, key size, value size): what the page pool allocates"""
        return [(l.mixer.kv_heads, l.mixer.dim, l.mixer.vdim) for l in self.layers]


def tiny_tagenex(width=96, vocab=300, layers=None, eps=1e-5):
    """A small Tagenex config dict for tests (sizes deliberately unequal: dim != vdim, heads != kv_heads, windows that differ
    between layers, one layer without a window, one without a feed-forward, one that does not mix values)."""
    att = lambda heads, kv, dim, vdim, win, mix, scale=None: {
        'type': 'attention',
        'mixer': dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale or dim ** -0.5, v_mix=mix,
                      **({'mask': {'size': win}} if win else {}))}
    dense = lambda ff, lim=2.0: {'kind': 'dense', 'ff': ff, 'limit': lim}
    moe = lambda ff, e, top, lim=2.0: {'kind': 'moe', 'expert': {'ff': ff, 'limit': lim}, 'router': {'experts': e, 'top': top}}
    if layers is None:
        layers = [dict(att(6, 3, 40, 24, 50, True), mlp=dense(136)),
                  dict(att(4, 1, 48, 24, 0, False), mlp=moe(56, 5, 2)),
                  dict(att(6, 3, 24, 24, 33, True), mlp=None),
                  dict(att(3, 3, 32, 24, 100, True), mlp=moe(40, 3, 3))]
    return {'architecture': 'Tagenex', 'vocab': vocab, 'width': width, 'norm': {'eps': eps}, 'layers': layers}


# ------------------------------------------------------------------------------------------------ Tapalix
class TapalixConfig:
    """config.json of a Tapalix checkpoint: {"architecture": "Tapalix", "vocab", "width", "norm": {"eps"}, "embedding": {"scale"},
    "layers": [...], "loop": {"start", "stop", "times"} or absent, "logit_scale", "logit_softcap"}.
    A layer entry has "type" ("latent_attention": per head `dim` plain and `rot_dim` turning query/key numbers with the rotation
    constants under "rot"; "latent_attention_2": no positions, a sigmoid output gate), "mixer" (heads, dim, vdim, kv_rank, scale,
    rot_dim, rot: {base, dims, scaling: {factor, original, fast, slow} or absent}) and "mlp": null | {"kind": "moe", expert: {ff},
    router: {experts, top, scale, groups: {count, keep} or absent}, shared: {ff} or absent}. Nothing is assumed equal between
    layers. `runs` lists the layer runs in order (a looped layer once per pass): every run has a cache of its own."""

    def __init__(self, d):
        self.raw = d
        self.architecture = d.get('architecture', 'Tapalix')
        self.architectures = [self.architecture]
        self.vocab_size, self.width = int(d['vocab']), int(d['width'])
        self.eps = float(d['norm']['eps'])
        self.embed_scale = float((d.get('embedding') or {}).get('scale', 1.0))
        self.logit_scale = float(d.get('logit_scale') or 1.0)
        self.logit_softcap = float(d.get('logit_softcap') or 0.0)
        self.layers = []
        for i, lc in enumerate(d['layers']):
            kind = lc.get('type')
            if kind not in ('latent_attention', 'latent_attention_2'):
                raise NotImplementedError(f'layer {i}: mixer type {kind!r} is not part of this design')
            m = lc['mixer']
            rotary = kind == 'latent_attention'
            mixer = SimpleNamespace(kind=kind, rotary=rotary, gated=not rotary, heads=int(m['heads']), dim=int(m['dim']),
                                    vdim=int(m.get('vdim', m['dim'])), kv_rank=int(m['kv_rank']), scale=float(m['scale']),
                                    rot_dim=int(m.get('rot_dim', 0)) if rotary else 0, rot=None)
            if rotary and mixer.rot_dim > 0:
                r = m['rot']
                sc = r.get('scaling')
                mixer.rot = SimpleNamespace(base=float(r['base']), dims=int(r.get('dims', mixer.rot_dim)),
                                            scaling=None if not sc else SimpleNamespace(
                                                factor=float(sc['factor']), original=float(sc['original']),
                                                fast=float(sc['fast']), slow=float(sc['slow'])))
                if mixer.rot.dims % 2 or not 0 < mixer.rot.dims <= mixer.rot_dim:
                    raise ValueError(f'layer {i}: rot.dims must be even and at most rot_dim')
            f = lc.get('mlp')
            if f is None:
                ff = None
            elif f['kind'] == 'moe':
                r = f['router']
                g = r.get('groups') or {}
                sh = f.get('shared') or {}
                ff = SimpleNamespace(kind='moe', ff=int(f['expert']['ff']), experts=int(r['experts']), top=int(r['top']),
                                     scale=float(r.get('scale', 1.0)), groups=int(g.get('count', 1)), keep=int(g.get('keep', 1)),
                                     shared_ff=int(sh.get('ff', 0)))
                if not 1 <= ff.top <= ff.experts:
                    raise ValueError(f'layer {i}: top must be in [1, experts]')
                if ff.groups > 1 and (ff.experts % ff.groups or not 1 <= ff.keep <= ff.groups
                                      or ff.keep * (ff.experts // ff.groups) < ff.top):
                    raise ValueError(f'layer {i}: expert groups must divide the experts and the kept ones must hold `top` experts')
            else:
                raise NotImplementedError(f"layer {i}: feed-forward kind {f['kind']!r}")
            self.layers.append(SimpleNamespace(mixer=mixer, ff=ff))
        self.num_hidden_layers = n = len(self.layers)
        lp = d.get('loop')
        if lp:
            lo, hi, times = int(lp['start']), int(lp['stop']), int(lp['times'])
            if not (0 <= lo < hi <= n and times >= 1):
                raise ValueError('loop: need 0 <= start < stop <= layers and times >= 1')
            self.loop = SimpleNamespace(start=lo, stop=hi, times=times)
            order = list(range(lo)) + list(range(lo, hi)) * times + list(range(hi, n))
        else:
            self.loop, lo, order = None, -1, list(range(n))
        # (layer index, does a pass of the loop start with this run)
        self.runs = [(i, i == lo) for i in order]

    def kv_layout(self):
        """per layer RUN (one shared head, latent + turning key numbers, no separate values): what the page pool allocates"""
        return [(1, self.layers[i].mixer.kv_rank + self.layers[i].mixer.rot_dim, 0) for i, _ in self.runs]


def yarn_frequencies(rot):
    """angular frequency of every rotated pair and the factor on cos / sin. Pair i turns by base^(-2i/dims) per position. With
    scaling, pairs that complete fewer than `slow` turns over the `original` context are slowed by `factor`, pairs with more than
    `fast` turns are left alone, and the pairs between are blended linearly in the pair index; cos and sin grow by
    0.1 ln(factor) + 1."""
    import math
    n = rot.dims // 2
    f = [rot.base ** (-2.0 * i / rot.dims) for i in range(n)]
    sc = rot.scaling
    if sc is None:
        return f, 1.0
    index_of = lambda turns: rot.dims * math.log(sc.original / (2 * math.pi * turns)) / (2 * math.log(rot.base))
    lo = max(math.floor(index_of(sc.fast)), 0)
    hi = min(math.ceil(index_of(sc.slow)), rot.dims - 1)
    out = []
    for i in range(n):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / sc.factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(sc.factor) + 1.0


def tiny_tapalix(width=96, vocab=300, layers=None, loop=(1, 3, 2), eps=1e-5):
    """A small Tapalix config dict for tests: sizes deliberately unequal between layers (dim != vdim != kv_rank; head counts,
    ranks and group shapes differ), one layer without a feed-forward, one without expert groups and without a shared expert;
    layers 1 and 2 run twice."""
    rot = lambda dims, factor=4.0: {'base': 10000.0, 'dims': dims,
                                    'scaling': {'factor': factor, 'original': 64, 'fast': 16.0, 'slow': 2.0}}
    la = lambda heads, dim, rd, vdim, rank, scale=None: {
        'type': 'latent_attention',
        'mixer': dict(heads=heads, dim=dim, rot_dim=rd, vdim=vdim, kv_rank=rank, scale=scale or (dim + rd) ** -0.5, rot=rot(rd))}
    la2 = lambda heads, dim, vdim, rank, scale=None: {
        'type': 'latent_attention_2', 'mixer': dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale or dim ** -0.5)}
    moe = lambda ff, e, top, groups=None, shared=None, scale=1.5: {
        'kind': 'moe', 'expert': {'ff': ff},
        'router': dict(experts=e, top=top, scale=scale, **({'groups': {'count': groups[0], 'keep': groups[1]}} if groups else {})),
        **({'shared': {'ff': shared}} if shared else {})}
    if layers is None:
        layers = [dict(la2(3, 24, 40, 56), mlp=moe(40, 6, 2, (3, 2), 72)),
                  dict(la(5, 16, 8, 24, 40), mlp=moe(24, 8, 3, (4, 2), 48)),
                  dict(la2(2, 48, 16, 72), mlp=None),
                  dict(la(4, 24, 24, 32, 48), mlp=moe(32, 5, 2, None, None))]
    d = {'architecture': 'Tapalix', 'vocab': vocab, 'width': width, 'norm': {'eps': eps}, 'embedding': {'scale': width ** 0.5},
         'layers': layers, 'logit_scale': 1.5, 'logit_softcap': 20.0}
    if loop:
        d['loop'] = {'start': loop[0], 'stop': loop[1], 'times': loop[2]}
    return d


# ------------------------------------------------------------------------------------------------ Dugalix
class DugalixConfig:
    """config.json of a Dugalix checkpoint: {"architecture": "Dugalix", "vocab", "width", "norm": {"eps"}, "residual_mult",
    "layers": [...]}. A layer entry has "type", "mixer" and "mlp":
      type "attention": mixer = {heads, kv_heads, dim, vdim, scale, mask: {size}, rot: {base, dims}}: the values are the keys before
                        their rotation (vdim == dim) and a visible key weighs sigmoid(score + per-head bias);
      type "parallel":  mixer = {left: {heads, kv_heads, dim, vdim, scale, mask: {size, keep_first}, rot: {base, dims, scaling:
                        {factor}}}, right: {heads, dim, vdim, gate_cap}, left_scale, right_scale}: softmax attention with biases
                        beside a matrix-memory recurrence;
      mlp: null | {"kind": "dense", ff} | {"kind": "moe", expert: {ff}, router: {experts, identity, top, groups: {count, keep}},
                        shared: {ff}}: `identity` further router outputs stand for experts that return their input.
    Absent optional keys mean: no window, no kept first tokens, no rotation, no slowing factor, no groups, no identity experts, no
    shared unit. Nothing is assumed equal between layers."""
    @staticmethod
    def _attention(i, m, kind):
        mask, r = m.get('mask') or {}, m.get('rot')
        a = SimpleNamespace(kind=kind, heads=int(m['heads']), kv_heads=int(m.get('kv_heads', m['heads'])), dim=int(m['dim']),
                            vdim=int(m.get('vdim', m['dim'])), scale=float(m['scale']), window=int(mask.get('size') or 0),
                            keep_first=int(mask.get('keep_first') or 0), rot=None)
        if a.heads % a.kv_heads:
            raise ValueError(f'layer {i}: heads must be a multiple of kv_heads')
        if r and int(r.get('dims', a.dim)) > 0:
            a.rot = SimpleNamespace(base=float(r['base']), dims=int(r.get('dims', a.dim)),
                                    factor=float((r.get('scaling') or {}).get('factor', 1.0)))
            if a.rot.dims % 2 or a.rot.dims > a.dim:
                raise ValueError(f'layer {i}: rot.dims must be even and at most dim')
        if kind == 'sigmoid' and a.vdim != a.dim:
            raise ValueError(f'layer {i}: keys that double as values need vdim == dim')
        return a

    def __init__(self, d):
        self.raw = d
        self.architecture = d.get('architecture', 'Dugalix')
        self.architectures = [self.architecture]
        self.vocab_size, self.width = int(d['vocab']), int(d['width'])
        self.eps = float(d['norm']['eps'])
        self.residual_mult = float(d.get('residual_mult', 1.0))
        self.layers = []
        for i, lc in enumerate(d['layers']):
            kind, m = lc.get('type'), lc['mixer']
            if kind == 'attention':
                mixer = SimpleNamespace(kind=kind, att=self._attention(i, m, 'sigmoid'), mem=None, att_scale=1.0, mem_scale=0.0)
            elif kind == 'parallel':
                r = m['right']
                mem = SimpleNamespace(heads=int(r['heads']), dim=int(r['dim']), vdim=int(r.get('vdim', r['dim'])),
                                      gate_cap=float(r['gate_cap']))
                if not 1 <= mem.dim <= 512:
                    raise NotImplementedError(f'layer {i}: matrix-memory key size {mem.dim}; the kernels take 1 .. 512')
                mixer = SimpleNamespace(kind=kind, att=self._attention(i, m['left'], 'softmax'), mem=mem,
                                        att_scale=float(m.get('left_scale', 1.0)), mem_scale=float(m.get('right_scale', 1.0)))
            else:
                raise NotImplementedError(f'layer {i}: mixer type {kind!r} is not part of this design')
            f = lc.get('mlp')
            if f is None:
                ff = None
            elif f['kind'] == 'dense':
                ff = SimpleNamespace(kind='dense', ff=int(f['ff']))
            elif f['kind'] == 'moe':
                r = f['router']
                g = r.get('groups') or {}
                ff = SimpleNamespace(kind='moe', ff=int(f['expert']['ff']), experts=int(r['experts']), identity=int(r.get('identity') or 0),
                                     top=int(r['top']), groups=int(g.get('count', 1)), keep=int(g.get('keep', 1)),
                                     shared_ff=int((f.get('shared') or {}).get('ff', 0)))
                ff.outputs = ff.experts + ff.identity          # what the router scores
                if not 1 <= ff.top <= ff.outputs:
                    raise ValueError(f'layer {i}: top must be in [1, experts + identity]')
                if ff.groups > 1 and (ff.outputs % ff.groups or not 1 <= ff.keep <= ff.groups
                                      or ff.keep * (ff.outputs // ff.groups) < ff.top):
                    raise ValueError(f'layer {i}: expert groups must divide experts + identity and the kept ones must hold `top`')
            else:
                raise NotImplementedError(f"layer {i}: feed-forward kind {f['kind']!r}")
            self.layers.append(SimpleNamespace(mixer=mixer, ff=ff))
        self.num_hidden_layers = len(self.layers)

    def kv_layout(self):
        """per layer (kv heads, key size, value size): what the page pool allocates (every layer has an attention)"""
        return [(l.mixer.att.kv_heads, l.mixer.att.dim, l.mixer.att.vdim) for l in self.layers]


def rot_frequencies(rot):
    """angular frequency of every turning pair: base^(-2i/dims), divided by the slowing factor"""
    return [rot.base ** (-2.0 * i / rot.dims) / rot.factor for i in range(rot.dims // 2)]


def tiny_dugalix(width=96, vocab=300, layers=None, eps=1e-5, residual_mult=0.7):
    """A small Dugalix config dict for tests: sizes deliberately unequal between layers and between the halves of a parallel mixer
    (dim != vdim, heads != kv_heads, partly rotated heads, windows and kept prefixes that differ), one layer without a
    feed-forward, a mixture without groups / identity experts / shared unit beside one with all three."""
    rot = lambda dims, factor=None: {'base': 10000.0, 'dims': dims, **({'scaling': {'factor': factor}} if factor else {})}
    sig = lambda heads, kv, dim, win, rd, scale=None: {
        'type': 'attention', 'mixer': dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale or dim ** -0.5,
                                           mask={'size': win}, rot=rot(rd))}
    par = lambda lh, lkv, ld, lv, win, keep, rd, rh, rdim, rv, ls=0.8, rs=1.1, factor=4.0, cap=15.0: {
        'type': 'parallel',
        'mixer': {'left': dict(heads=lh, kv_heads=lkv, dim=ld, vdim=lv, scale=ld ** -0.5, mask={'size': win, 'keep_first': keep},
                               rot=rot(rd, factor)),
                  'right': dict(heads=rh, dim=rdim, vdim=rv, gate_cap=cap), 'left_scale': ls, 'right_scale': rs}}
    dense = lambda ff: {'kind': 'dense', 'ff': ff}
    moe = lambda ff, e, ident, top, groups=None, shared=None: {
        'kind': 'moe', 'expert': {'ff': ff},
        'router': dict(experts=e, identity=ident, top=top, **({'groups': {'count': groups[0], 'keep': groups[1]}} if groups else {})),
        **({'shared': {'ff': shared}} if shared else {})}
    if layers is None:
        layers = [dict(par(6, 3, 24, 40, 37, 5, 16, 3, 24, 40), mlp=moe(40, 5, 3, 3, (4, 3), 72)),
                  dict(sig(4, 2, 40, 33, 24), mlp=dense(136)),
                  dict(par(4, 1, 32, 16, 70, 66, 32, 2, 40, 72, factor=None), mlp=None),
                  dict(sig(3, 3, 24, 90, 8), mlp=moe(32, 4, 0, 2))]
    return {'architecture': 'Dugalix', 'vocab': vocab, 'width': width, 'norm': {'eps': eps}, 'residual_mult': residual_mult,
            'layers': layers}


# ------------------------------------------------------------------------------------------------ Danalorn
class DanalornConfig:
    """config.json of a Danalorn checkpoint: {"architecture": "Danalorn", "vocab", "width", "norm": {"eps"}, "embedding": {"scale",
    "bigram": {"buckets", "mul_prev", "mul_cur"} or absent}, "layers": [...]}. A layer entry has "type", "mixer" and "mlp":
      type "latent_attention": mixer = {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask: {size}, rot: {base, dims}, kv_from}:
                        per head `dim` plain and `rot_dim` turning query/key numbers, queries through a normed vector of q_rank
                        numbers, a sliding window and a learned per-head sink; with kv_from = j the layer has no latent projection
                        and reads the cache of layer j (same kv_rank, rot_dim and rotation);
      type "attention": mixer = {heads, kv_heads, dim, vdim, scale, q_temp: {coef, every}}: biased projections, per-head query/key
                        norm, no rotation, a linear distance bias with the fixed slopes 2^(-8 (h + 1) / heads), one added to the
                        softmax denominator, an element-wise sigmoid output gate; causal without a window;
      type "gla":       mixer = {heads, dim, vdim, tau}: gated linear attention, decay = sigmoid(z)^(1/tau) per key channel;
      mlp: null | {"kind": "dense", ff}: a relu^2 unit.
    Absent optional keys mean: no pair table, no window, no query temperature. Nothing is assumed equal between layers."""
    SLOPE_OCTAVES = 8.0          # the distance-bias slopes of an attention mixer span 2^-8 .. 1: fixed by the design

    def __init__(self, d):
        self.raw = d
        self.architecture = d.get('architecture', 'Danalorn')
        self.architectures = [self.architecture]
        self.vocab_size, self.width = int(d['vocab']), int(d['width'])
        self.eps = float(d['norm']['eps'])
        emb = d.get('embedding') or {}
        self.embed_scale = float(emb.get('scale', 1.0))
        bg = emb.get('bigram')
        self.bigram = None if not bg else SimpleNamespace(buckets=int(bg['buckets']), mul_prev=int(bg['mul_prev']),
                                                          mul_cur=int(bg['mul_cur']))
        if self.bigram is not None and self.bigram.buckets < 1:
            raise ValueError('embedding.bigram.buckets must be at least 1')
        self.layers = []
        for i, lc in enumerate(d['layers']):
            kind, m = lc.get('type'), lc['mixer']
            if kind == 'latent_attention':
                r = m.get('rot') or {}
                mixer = SimpleNamespace(kind=kind, heads=int(m['heads']), dim=int(m['dim']), rot_dim=int(m.get('rot_dim', 0)),
                                        vdim=int(m.get('vdim', m['dim'])), kv_rank=int(m['kv_rank']), q_rank=int(m['q_rank']),
                                        scale=float(m['scale']), window=int((m.get('mask') or {}).get('size') or 0),
                                        kv_from=None if m.get('kv_from') is None else int(m['kv_from']), rot=None)
                if mixer.rot_dim > 0:
                    mixer.rot = SimpleNamespace(base=float(r['base']), dims=int(r.get('dims', mixer.rot_dim)))
                    if mixer.rot.dims % 2 or not 0 < mixer.rot.dims <= mixer.rot_dim:
                        raise ValueError(f'layer {i}: rot.dims must be even and at most rot_dim')
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    src = self.layers[j].mixer if 0 <= j < i else None
                    if src is None or src.kind != kind or src.kv_from is not None:
                        raise ValueError(f'layer {i}: kv_from must name an earlier latent_attention layer with a latent projection of its own')
                    if (src.kv_rank, src.rot_dim) != (mixer.kv_rank, mixer.rot_dim) or \
                            (src.rot and (src.rot.base, src.rot.dims)) != (mixer.rot and (mixer.rot.base, mixer.rot.dims)):
                        raise ValueError(f'layer {i}: kv_rank, rot_dim and rotation must equal those of layer {j}')
            elif kind == 'attention':
                qt = m.get('q_temp') or {}
                mixer = SimpleNamespace(kind=kind, heads=int(m['heads']), kv_heads=int(m.get('kv_heads', m['heads'])), dim=int(m['dim']),
                                        vdim=int(m.get('vdim', m['dim'])), scale=float(m['scale']),
                                        q_temp_coef=float(qt.get('coef', 0.0)), q_temp_every=int(qt.get('every', 0)))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f'layer {i}: heads must be a multiple of kv_heads')
                if mixer.dim > 256 or mixer.vdim > 256:
                    raise NotImplementedError(f'layer {i}: head sizes above 256; the query/key norm kernel takes up to 256')
            elif kind == 'gla':
                mixer = SimpleNamespace(kind=kind, heads=int(m['heads']), dim=int(m['dim']), vdim=int(m.get('vdim', m['dim'])),
                                        tau=float(m['tau']))
                if not 1 <= mixer.dim <= 512:
                    raise NotImplementedError(f'layer {i}: key size {mixer.dim} of the recurrence; the kernels take 1 .. 512')
                if mixer.tau <= 0:
                    raise ValueError(f'layer {i}: tau must be positive')
            else:
                raise NotImplementedError(f'layer {i}: mixer type {kind!r} is not part of this design')
            f = lc.get('mlp')
            if f is None:
                ff = None
            elif f['kind'] == 'dense':
                ff = SimpleNamespace(kind='dense', ff=int(f['ff']))
            else:
                raise NotImplementedError(f"layer {i}: feed-forward kind {f['kind']!r}")
            self.layers.append(SimpleNamespace(mixer=mixer, ff=ff))
        self.num_hidden_layers = len(self.layers)

    def kv_layout(self):
        """per layer (kv heads, key size, value size): what the page pool allocates. A latent layer caches one row (latent vector |
        turning key part) per token as one shared head; a layer that reads another layer's cache, and a recurrent layer, nothing."""
        out = []
        for l in self.layers:
            m = l.mixer
            if m.kind == 'attention':
                out.append((m.kv_heads, m.dim, m.vdim))
            elif m.kind == 'latent_attention' and m.kv_from is None:
                out.append((1, m.kv_rank + m.rot_dim, 0))
            else:
                out.append((0, 0, 0))
        return out

    def slopes(self, heads):
        """slope of the linear distance bias of head h = 0 .. heads - 1"""
        return [2.0 ** (-self.SLOPE_OCTAVES * (h + 1) / heads) for h in range(heads)]


def tiny_danalorn(width=96, vocab=300, layers=None, eps=1e-5, bigram=(257, 29, 5), embed_scale=1.5):
    """A small Danalorn config dict for tests: sizes deliberately unequal between layers (dim != vdim != rot_dim, heads != kv_heads,
    partly rotated turning parts, windows that differ), a latent layer that reads an earlier layer's cache, one layer without a
    feed-forward, an attention layer without a query temperature. The embedding's scale is small, so that the layers' outputs and
    not the first rows of the residual stream decide the logits."""
    la = lambda heads, dim, rd, vdim, rank, qrank, win, rdims=None, base=10000.0, kv_from=None: {
        'type': 'latent_attention',
        'mixer': dict(heads=heads, dim=dim, rot_dim=rd, vdim=vdim, kv_rank=rank, q_rank=qrank, scale=(dim + rd) ** -0.5,
                      rot={'base': base, 'dims': rdims or rd}, **({'mask': {'size': win}} if win else {}),
                      **({'kv_from': kv_from} if kv_from is not None else {}))}
    att = lambda heads, kv, dim, vdim, qt=None: {
        'type': 'attention', 'mixer': dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=dim ** -0.5,
                                           **({'q_temp': {'coef': qt[0], 'every': qt[1]}} if qt else {}))}
    gla = lambda heads, dim, vdim, tau: {'type': 'gla', 'mixer': dict(heads=heads, dim=dim, vdim=vdim, tau=tau)}
    dense = lambda ff: {'kind': 'dense', 'ff': ff}
    if layers is None:
        layers = [dict(gla(3, 24, 40, 8.0), mlp=dense(136)),
                  dict(la(5, 16, 8, 24, 40, 56, 37), mlp=dense(72)),
                  dict(att(6, 3, 24, 40, (0.4, 7)), mlp=None),
                  dict(la(3, 24, 8, 16, 40, 32, 70, kv_from=1), mlp=dense(40)),
                  dict(att(4, 1, 40, 24), mlp=dense(88)),
                  dict(la(4, 8, 24, 32, 48, 40, 0, rdims=16, base=500.0), mlp=dense(56)),
                  dict(gla(2, 40, 72, 3.0), mlp=dense(64))]
    d = {'architecture': 'Danalorn', 'vocab': vocab, 'width': width, 'norm': {'eps': eps}, 'embedding': {'scale': embed_scale},
         'layers': layers}
    if bigram:
        d['embedding']['bigram'] = {'buckets': bigram[0], 'mul_prev': bigram[1], 'mul_cur': bigram[2]}
    return d
