"""Host-side parts of the Danalorn integration that need no GPU: config parsing, the registry, checkpoint shapes, what the page
pool allocates for layers without a cache of their own, and the oracle's own mechanisms on hand-made inputs."""
import math

import pytest
import torch

import phi3_b200  # noqa: F401
from phi3_b200 import configs, registry, weights
from phi3_b200.paged import PagePool, PAGE
from oracle import danalorn_oracle as O

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    d = configs.tiny_danalorn()
    c = configs.DanalornConfig(d)
    assert c.vocab_size == 300 and c.width == 96 and c.eps == 1e-5 and c.embed_scale == 1.5 and len(c.layers) == 7
    assert (c.bigram.buckets, c.bigram.mul_prev, c.bigram.mul_cur) == (257, 29, 5)
    assert [l.mixer.kind for l in c.layers] == ['gla', 'latent_attention', 'attention', 'latent_attention', 'attention',
                                                'latent_attention', 'gla']
    g0, l1, a2, l3, a4, l5 = (c.layers[i].mixer for i in range(6))
    assert (g0.heads, g0.dim, g0.vdim, g0.tau) == (3, 24, 40, 8.0)
    assert (l1.heads, l1.dim, l1.rot_dim, l1.vdim, l1.kv_rank, l1.q_rank, l1.window, l1.kv_from) == (5, 16, 8, 24, 40, 56, 37, None)
    assert (l1.rot.base, l1.rot.dims) == (10000.0, 8) and l1.scale == 24 ** -0.5
    assert (a2.heads, a2.kv_heads, a2.dim, a2.vdim, a2.q_temp_coef, a2.q_temp_every) == (6, 3, 24, 40, 0.4, 7)
    assert (l3.kv_from, l3.heads, l3.dim, l3.vdim, l3.window) == (1, 3, 24, 16, 70) and (a4.q_temp_every, a4.kv_heads) == (0, 1)
    assert (l5.window, l5.rot.dims, l5.rot_dim, l5.rot.base) == (0, 16, 24, 500.0)
    assert c.layers[2].ff is None and c.layers[0].ff.ff == 136
    # a latent layer caches one shared row per token; a layer that borrows a cache, and a recurrent layer, nothing
    assert c.kv_layout() == [(0, 0, 0), (1, 48, 0), (3, 24, 40), (0, 0, 0), (1, 40, 24), (1, 72, 0), (0, 0, 0)]
    assert c.slopes(4) == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8] and c.slopes(3)[0] == 2.0 ** (-8 / 3)
    plain = configs.DanalornConfig(configs.tiny_danalorn(bigram=None))
    assert plain.bigram is None
    bare = configs.tiny_danalorn()
    del bare['embedding']
    assert configs.DanalornConfig(bare).embed_scale == 1.0 and configs.DanalornConfig(bare).bigram is None
    for key, val, err in ((('layers', 0, 'type'), 'recurrent', NotImplementedError), (('layers', 0, 'mlp', 'kind'), 'glu', NotImplementedError),
                          (('layers', 1, 'mixer', 'rot', 'dims'), 7, ValueError), (('layers', 1, 'mixer', 'rot', 'dims'), 10, ValueError),
                          (('layers', 2, 'mixer', 'kv_heads'), 4, ValueError), (('layers', 3, 'mixer', 'kv_from'), 2, ValueError),
                          (('layers', 3, 'mixer', 'kv_from'), 5, ValueError), (('layers', 3, 'mixer', 'kv_rank'), 48, ValueError),
                          (('layers', 5, 'mixer', 'kv_from'), 3, ValueError), (('layers', 0, 'mixer', 'tau'), 0.0, ValueError),
                          (('layers', 0, 'mixer', 'dim'), 600, NotImplementedError), (('embedding', 'bigram', 'buckets'), 0, ValueError)):
        bad = configs.tiny_danalorn()
        node = bad
        for k in key[:-1]:
            node = node[k]
        node[key[-1]] = val
        with pytest.raises(err):
            configs.DanalornConfig(bad)


def test_registry_and_checkpoint_shapes():
    assert registry.entry_for({'architecture': 'Danalorn'}).engine == 'paged'
    assert isinstance(registry.entry_for({'architecture': 'Danalorn'}).config(configs.tiny_danalorn()), configs.DanalornConfig)
    d = configs.tiny_danalorn()
    d['layers'][6]['mixer']['decay_rank'] = 12                # read by the random-weight helper alone: checkpoints give it by a1's shape
    shapes = weights.danalorn_tensor_shapes(d)
    w = weights.random_danalorn_weights(d, 0)
    assert set(shapes) == set(w) and all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert shapes['bigram'] == (258, 96) and shapes['embed'] == (300, 96) and shapes['head'] == (300, 96)
    assert shapes['l1.mix.dq'] == (56, 96) and shapes['l1.mix.uq'] == (5 * 24, 56) and shapes['l1.mix.dkv'] == (48, 96)
    assert shapes['l1.mix.dkv.norm'] == (40,) and shapes['l1.mix.uk'] == (80, 40) and shapes['l1.mix.uv'] == (120, 40)
    assert shapes['l1.mix.sink'] == (5,) and shapes['l1.mix.o'] == (96, 120)
    assert 'l3.mix.dkv' not in shapes and 'l3.mix.dkv.norm' not in shapes and shapes['l3.mix.uk'] == (72, 40)
    assert shapes['l2.mix.q'] == (144, 96) and shapes['l2.mix.k.b'] == (72,) and shapes['l2.mix.v'] == (120, 96)
    assert shapes['l2.mix.q.norm'] == (24,) and shapes['l2.mix.g'] == (240, 96) and 'l2.norm2' not in shapes
    assert shapes['l0.mix.a1'] == (16, 96) and shapes['l6.mix.a1'] == (12, 96) and shapes['l6.mix.a2'] == (80, 12)
    assert shapes['l0.mix.norm'] == (40,) and shapes['l0.mix.a2.b'] == (72,) and shapes['l0.mlp.up'] == (136, 96)
    assert 'bigram' not in weights.danalorn_tensor_shapes(configs.tiny_danalorn(bigram=None))


def test_page_pool_allocates_nothing_for_layers_without_a_cache():
    c = configs.DanalornConfig(configs.tiny_danalorn())
    pool = PagePool(c.kv_layout(), 3 * PAGE, 2, torch.float32, 'cpu', state_layout=[1, 3 * 24 * 40])
    assert [t.numel() for t in pool.k] == [0, 3 * 64 * 48, 3 * 3 * 64 * 24, 0, 3 * 64 * 40, 3 * 64 * 72, 0]
    assert [t.numel() for t in pool.v] == [0, 0, 3 * 3 * 64 * 40, 0, 3 * 64 * 24, 0, 0]
    assert [tuple(s.shape) for s in pool.state] == [(2, 1), (2, 2880)]
    assert pool.state[0].view(torch.int32).shape == (2, 1)    # the last token of a sequence lives there as an integer


# ------------------------------------------------------------------------------------------------ the oracle's mechanisms
def test_oracle_pair_embedding_rows():
    W = 4
    w = {'embed': torch.arange(10 * W, dtype=F64).view(10, W), 'bigram': 100.0 * torch.arange(8, dtype=F64)[:, None].repeat(1, W)}
    ec = {'scale': 2.0, 'bigram': {'buckets': 7, 'mul_prev': 37, 'mul_cur': 5}}
    toks = [3, 9, 9, 0]
    x = O.embed(toks, w, ec, F64)
    rows = [7, (3 * 37 + 9 * 5) % 7, (9 * 37 + 9 * 5) % 7, (9 * 37 + 0) % 7]       # the first token takes the table's last row
    for t, (tok, r) in enumerate(zip(toks, rows)):
        assert torch.equal(x[t], w['embed'][tok] * 2.0 + 100.0 * r)
    assert torch.equal(O.embed(toks, w, {'scale': 0.5}, F64), w['embed'][torch.tensor(toks)] * 0.5)
    assert torch.equal(O.embed(toks, w, {}, F64), w['embed'][torch.tensor(toks)])


def test_oracle_rotation_pairs_neighbours_and_is_partial():
    rot = {'base': 100.0, 'dims': 4}
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64).repeat(2, 1, 1)
    out = O.rotate_pairs(v, torch.tensor([0, 3]), rot)
    assert torch.equal(out[0], v[0]) and torch.equal(out[1, 0, 4:], v[1, 0, 4:])
    a0, a1 = 3 * 1.0, 3 * 100.0 ** -0.5                       # pair i turns by position * base^(-2i/dims)
    want = [1 * math.cos(a0) - 2 * math.sin(a0), 2 * math.cos(a0) + 1 * math.sin(a0),
            3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)]
    assert torch.allclose(out[1, 0, :4], torch.tensor(want, dtype=F64))
    # a rotation of both sides leaves the product a function of the distance alone
    q, k = torch.randn(1, 1, 6, dtype=F64), torch.randn(1, 1, 6, dtype=F64)
    dot = lambda i, j: float((O.rotate_pairs(q, torch.tensor([i]), rot) * O.rotate_pairs(k, torch.tensor([j]), rot)).sum())
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9 and abs(dot(9, 4) - dot(10, 4)) > 1e-6


def test_oracle_window_and_sink():
    vis = O.causal_window(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    assert O.causal_window(4, 0).tolist() == torch.ones(4, 4).tril().bool().tolist()
    assert O.causal_window(3, 1).tolist() == torch.eye(3).bool().tolist()
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=F64)
    p = O.softmax_with_sink(s, torch.tensor([[True, False, True]]), 0.7)
    den = math.exp(0.3) + math.exp(2.0) + math.exp(0.7)       # the sink counts once, unscaled, and has no value
    assert torch.allclose(p, torch.tensor([[math.exp(0.3) / den, 0.0, math.exp(2.0) / den]], dtype=F64))
    assert float(O.softmax_with_sink(s, torch.ones(1, 3, dtype=torch.bool), 50.0).sum()) < 1e-15    # a huge sink takes all weight
    assert abs(float(O.softmax_with_sink(s, torch.ones(1, 3, dtype=torch.bool), -50.0).sum()) - 1) < 1e-12


def test_oracle_latent_attention_equals_explicit_keys_and_values():
    """the mixer against a direct per-head formulation with materialised keys and values and a loop over the window"""
    torch.manual_seed(0)
    T, W, H, d, dr, dv, R, Q, win = 11, 10, 2, 4, 6, 3, 5, 7, 4
    mc = dict(heads=H, dim=d, rot_dim=dr, vdim=dv, kv_rank=R, q_rank=Q, scale=0.3, mask={'size': win}, rot={'base': 50.0, 'dims': 4})
    w = {'p.' + n: torch.randn(s, dtype=F64) for n, s in dict(dq=(Q, W), uq=(H * (d + dr), Q), dkv=(R + dr, W), uk=(H * d, R),
                                                               uv=(H * dv, R), o=(W, H * dv)).items()}
    w['p.dq.norm'], w['p.dkv.norm'], w['p.sink'] = torch.rand(Q, dtype=F64) + 0.5, torch.rand(R, dtype=F64) + 0.5, torch.randn(H, dtype=F64)
    h = torch.randn(T, W, dtype=F64)
    got = O.latent_attention(h, w, 'p.', mc, 1e-6, O.latent_kv(h, w, 'p.', mc, 1e-6))
    rms = lambda v, g: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-6) * g
    ckv = h @ w['p.dkv'].T
    c = rms(ckv[:, :R], w['p.dkv.norm'])
    q = (rms(h @ w['p.dq'].T, w['p.dq.norm']) @ w['p.uq'].T).view(T, H, d + dr)

    def turn(v, p):                                            # the first 4 of the 6 turning numbers rotate, as neighbour pairs
        out = v.clone()
        for i in range(2):
            ang = p * 50.0 ** (-2 * i / 4)
            out[2 * i] = v[2 * i] * math.cos(ang) - v[2 * i + 1] * math.sin(ang)
            out[2 * i + 1] = v[2 * i + 1] * math.cos(ang) + v[2 * i] * math.sin(ang)
        return out
    heads = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        for t in range(T):
            js = list(range(max(0, t - win + 1), t + 1))
            sc = torch.stack([(q[t, hh, :d] @ (w['p.uk'][hh * d:(hh + 1) * d] @ c[j]) + turn(q[t, hh, d:], t) @ turn(ckv[j, R:], j)) * 0.3
                              for j in js])
            e = torch.exp(sc)
            pr = e / (e.sum() + torch.exp(w['p.sink'][hh]))
            heads[t, hh] = sum(pr[n] * (w['p.uv'][hh * dv:(hh + 1) * dv] @ c[j]) for n, j in enumerate(js))
    assert torch.allclose(got, heads.reshape(T, H * dv) @ w['p.o'].T, atol=1e-10)


def test_oracle_biased_attention_temperature_distance_bias_and_gate():
    torch.manual_seed(1)
    T, W, H, G, d, dv = 9, 8, 4, 2, 3, 5
    mc = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=0.5, q_temp={'coef': 0.45, 'every': 4})
    w = {'p.' + n: torch.randn(s, dtype=F64) for n, s in dict(q=(H * d, W), k=(G * d, W), v=(G * dv, W), g=(H * dv, W), o=(W, H * dv)).items()}
    for n, s in (('q.b', H * d), ('k.b', G * d), ('v.b', G * dv)):
        w['p.' + n] = torch.randn(s, dtype=F64)
    w['p.q.norm'], w['p.k.norm'] = torch.rand(d, dtype=F64) + 0.5, torch.rand(d, dtype=F64) + 0.5
    h = torch.randn(T, W, dtype=F64)
    got = O.biased_attention(h, w, 'p.', mc, 1e-6)
    rms = lambda v, g: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-6) * g
    q = rms((h @ w['p.q'].T + w['p.q.b']).view(T, H, d), w['p.q.norm'])
    k = rms((h @ w['p.k'].T + w['p.k.b']).view(T, G, d), w['p.k.norm'])
    v = (h @ w['p.v'].T + w['p.v.b']).view(T, G, dv)
    heads = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        for t in range(T):
            temp = 1 + 0.45 * math.log((t + 1) // 4 + 1)        # grows at positions 3, 7, ...: (t + 1) counted in steps of 4
            sc = torch.stack([(q[t, hh] * temp) @ k[j, hh // 2] * 0.5 - 2.0 ** (-8 * (hh + 1) / H) * (t - j) for j in range(t + 1)])
            e = torch.exp(sc)
            heads[t, hh] = ((e / (1 + e.sum()))[:, None] * v[:t + 1, hh // 2]).sum(0)
    ref = (heads.reshape(T, H * dv) * torch.sigmoid(h @ w['p.g'].T)) @ w['p.o'].T
    assert torch.allclose(got, ref, atol=1e-10)
    no_temp = O.biased_attention(h, w, 'p.', {k_: v_ for k_, v_ in mc.items() if k_ != 'q_temp'}, 1e-6)
    assert torch.allclose(no_temp[:3], got[:3], atol=1e-12) and not torch.allclose(no_temp[3:], got[3:], atol=1e-6)


def test_oracle_gated_linear_attention_against_its_unrolled_sum():
    """the recurrence equals the direct sum over the past: token s reaches t with the product of the decays after s, per key channel"""
    torch.manual_seed(2)
    T, W, H, d, dv, r, tau = 8, 9, 2, 3, 4, 2, 5.0
    mc = dict(heads=H, dim=d, vdim=dv, tau=tau)
    w = {'p.' + n: torch.randn(s, dtype=F64) for n, s in dict(q=(H * d, W), k=(H * d, W), v=(H * dv, W), g=(H * dv, W), o=(W, H * dv),
                                                               a1=(r, W), a2=(H * d, r)).items()}
    w['p.a2.b'], w['p.norm'] = torch.randn(H * d, dtype=F64), torch.rand(dv, dtype=F64) + 0.5
    h = torch.randn(T, W, dtype=F64)
    got = O.gated_linear_attention(h, w, 'p.', mc, 1e-6)
    q = (h @ w['p.q'].T).view(T, H, d) * d ** -0.5
    k, v = (h @ w['p.k'].T).view(T, H, d), (h @ w['p.v'].T).view(T, H, dv)
    a = torch.sigmoid((h @ w['p.a1'].T) @ w['p.a2'].T + w['p.a2.b']).pow(1 / tau).view(T, H, d)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        for t in range(T):
            for s in range(t + 1):
                reach = a[s + 1:t + 1, hh].prod(0)             # decays of the tokens after s, up to and including t
                o[t, hh] += ((q[t, hh] * reach * k[s, hh]).sum()) * v[s, hh]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-6) * w['p.norm']
    g = h @ w['p.g'].T
    assert torch.allclose(got, (o.reshape(T, H * dv) * g * torch.sigmoid(g)) @ w['p.o'].T, atol=1e-10)


def test_oracle_layers_share_a_cache_and_every_layer_is_traced():
    d = configs.tiny_danalorn()
    w = weights.random_danalorn_weights(d, 3)
    toks = [5, 17, 3, 250, 17, 17, 9]
    trace = []
    lg = O.forward(d, w, toks, F64, trace)
    assert lg.shape == (7, 300) and len(trace) == 7 and all(t.shape == (7, 96) for t in trace)
    # causal: a prefix gives the same logits; the pair embedding makes a token's row depend on the token before it
    assert torch.allclose(O.forward(d, w, toks[:4], F64), lg[:4], atol=1e-10)
    swapped = O.forward(d, w, [6] + toks[1:], F64)
    assert not torch.allclose(swapped[1], lg[1], atol=1e-6)
    # layer 3 reads layer 1's latent vectors: changing layer 1's latent projection changes layer 3's mixer even with x held fixed
    x = torch.randn(7, 96, dtype=F64)
    mc1, mc3 = d['layers'][1]['mixer'], d['layers'][3]['mixer']
    wd = {k: v.double() for k, v in w.items()}
    kv = O.latent_kv(x, wd, 'l1.mix.', mc1, 1e-5)
    y = O.latent_attention(x, wd, 'l3.mix.', mc3, 1e-5, kv)
    y2 = O.latent_attention(x, wd, 'l3.mix.', mc3, 1e-5, (kv[0] * 1.5, kv[1]))
    assert y.shape == (7, 96) and not torch.allclose(y, y2, atol=1e-6)
