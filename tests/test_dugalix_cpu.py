"""Host-side parts of the Dugalix integration that need no GPU: config parsing, the registry, checkpoint shapes, the state rows of
the page pool, the sequence records of a step, and the oracle's own mechanisms on hand-made inputs."""
import math

import pytest
import torch

import phi3_b200  # noqa: F401
from phi3_b200 import configs, registry, weights
from phi3_b200.paged import PagePool, PAGE
from oracle import dugalix_oracle as O


def test_config_reads_every_size_and_constant():
    d = configs.tiny_dugalix()
    c = configs.DugalixConfig(d)
    assert c.vocab_size == 300 and c.width == 96 and c.eps == 1e-5 and c.residual_mult == 0.7 and len(c.layers) == 4
    assert [l.mixer.kind for l in c.layers] == ['parallel', 'attention', 'parallel', 'attention']
    a0, m0 = c.layers[0].mixer.att, c.layers[0].mixer.mem
    assert (a0.kind, a0.heads, a0.kv_heads, a0.dim, a0.vdim, a0.window, a0.keep_first) == ('softmax', 6, 3, 24, 40, 37, 5)
    assert (a0.rot.dims, a0.rot.base, a0.rot.factor) == (16, 10000.0, 4.0) and (m0.heads, m0.dim, m0.vdim, m0.gate_cap) == (3, 24, 40, 15.0)
    assert (c.layers[0].mixer.att_scale, c.layers[0].mixer.mem_scale) == (0.8, 1.1)
    a1 = c.layers[1].mixer.att
    assert (a1.kind, a1.window, a1.keep_first, a1.rot.dims, a1.rot.factor) == ('sigmoid', 33, 0, 24, 1.0) and c.layers[1].mixer.mem is None
    assert c.layers[2].mixer.att.rot.factor == 1.0 and c.layers[2].ff is None and c.layers[1].ff.kind == 'dense'
    f0, f3 = c.layers[0].ff, c.layers[3].ff
    assert (f0.experts, f0.identity, f0.outputs, f0.top, f0.groups, f0.keep, f0.shared_ff) == (5, 3, 8, 3, 4, 3, 72)
    assert (f3.experts, f3.identity, f3.outputs, f3.top, f3.groups, f3.shared_ff) == (4, 0, 4, 2, 1, 0)
    assert c.kv_layout() == [(3, 24, 40), (2, 40, 40), (1, 32, 16), (3, 24, 24)]
    assert configs.rot_frequencies(a0.rot) == [10000.0 ** (-2 * i / 16) / 4.0 for i in range(8)]
    for key, val, err in ((('layers', 0, 'type'), 'recurrent', NotImplementedError), (('layers', 1, 'mixer', 'vdim'), 48, ValueError),
                          (('layers', 0, 'mlp', 'router', 'top'), 9, ValueError), (('layers', 0, 'mlp', 'router', 'identity'), 2, ValueError),
                          (('layers', 1, 'mlp', 'kind'), 'glu', NotImplementedError), (('layers', 1, 'mixer', 'rot', 'dims'), 42, ValueError),
                          (('layers', 0, 'mixer', 'left', 'kv_heads'), 4, ValueError)):
        bad = configs.tiny_dugalix()
        node = bad
        for k in key[:-1]:
            node = node[k]
        node[key[-1]] = val
        with pytest.raises(err):
            configs.DugalixConfig(bad)


def test_registry_and_checkpoint_shapes():
    assert registry.entry_for({'architecture': 'Dugalix'}).engine == 'paged'
    assert isinstance(registry.entry_for({'architecture': 'Dugalix'}).config(configs.tiny_dugalix()), configs.DugalixConfig)
    d = configs.tiny_dugalix()
    shapes = weights.dugalix_tensor_shapes(d)
    w = weights.random_dugalix_weights(d, 0)
    assert set(shapes) == set(w) and all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert shapes['l0.mix.left.q'] == (144, 96) and shapes['l0.mix.left.k.b'] == (72,) and shapes['l0.mix.left.o'] == (96, 240)
    assert shapes['l0.mix.right.i'] == (3, 96) and shapes['l0.mix.right.norm'] == (120,) and shapes['l0.mix.right.o'] == (96, 120)
    assert shapes['l1.mix.k'] == (80, 96) and shapes['l1.mix.pb'] == (4,) and 'l1.mix.v' not in shapes and 'l1.mix.q.b' not in shapes
    assert shapes['l0.mlp.router'] == (8, 96) and shapes['l0.mlp.correction'] == (8,) and 'l0.mlp.e5.up' not in shapes
    assert shapes['l0.mlp.shared.sg'] == (1, 96) and 'l3.mlp.shared.up' not in shapes and 'l2.norm2' not in shapes
    assert shapes['l1.mlp.up'] == (136, 96) and shapes['l2.shift'] == (96,)


def test_page_pool_keeps_a_state_row_per_slot():
    pool = PagePool([(2, 8, 8)], 3 * PAGE, 3, torch.float32, 'cpu', state_layout=[96, 1000])
    assert [tuple(s.shape) for s in pool.state] == [(3, 96), (3, 1000)] and all(s.dtype == torch.float32 for s in pool.state)
    assert PagePool([(2, 8, 8)], PAGE, 2, torch.float32, 'cpu').state == []


class _FakeStateful:
    def __init__(self):
        self.dev, self.batches = torch.device('cpu'), []

    def kv_layout(self):
        return [(1, 4, 4)]

    def state_layout(self):
        return [7]

    def cache_dtype(self):
        return torch.float32

    def prepare(self, n):
        pass

    def forward(self, b, pool, trace=None):
        self.batches.append(b)
        return None


def test_engine_lists_the_sequences_of_a_step():
    from phi3_b200.engine import Engine
    m = _FakeStateful()
    eng = Engine(m, 4 * PAGE, 3)
    assert eng.stateful and eng.pool.state[0].shape == (3, 7)
    eng.step([('a', list(range(70)), []), ('b', [7], []), ('c', [1, 2], [])], end=['b'])
    b = m.batches[-1]
    assert b.n_seq == 3 and b.seqs.view(-1, 4).tolist() == [[0, 70, 0, 0], [70, 1, 1, 0], [71, 2, 2, 0]]
    assert b.slot_seq.tolist() == [0, 1, 2] and b.seqs.data_ptr() % 16 == b.pf_tiles.data_ptr() % 16
    eng.step([('c', [5], []), ('d', [1, 2, 3], []), ('a', [9], [])])          # d takes b's slot; the records follow the entries
    b = m.batches[-1]
    assert b.seqs.view(-1, 4).tolist() == [[0, 1, 2, 2], [1, 3, 1, 0], [4, 1, 0, 70]] and b.slot_seq.tolist() == [2, 1, 0]
    with pytest.raises(ValueError):
        eng.step([('a', [1], []), ('a', [2], [])])                             # the state of a request advances once per step


# ------------------------------------------------------------------------------------------------ the oracle's mechanisms
def test_oracle_norm_shift_and_visibility():
    v = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(O.norm1p(v, torch.tensor([0.5, -1.0], dtype=torch.float64), 0.0), torch.tensor([[1.5 * 3 / math.sqrt(12.5), 0.0]], dtype=torch.float64))
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [4.0, 40.0]], dtype=torch.float64)
    s = torch.tensor([0.0, 0.5], dtype=torch.float64)
    assert torch.allclose(O.token_shift(h, s), torch.tensor([[1.0, 5.0], [2.0, 15.0], [4.0, 30.0]], dtype=torch.float64))
    vis = O.visible(8, 3, 2)
    assert vis[7].tolist() == [True, True, False, False, False, True, True, True]
    assert vis[3].tolist() == [True, True, True, True, False, False, False, False]
    assert O.visible(5, 2)[4].tolist() == [False, False, False, True, True] and O.visible(4, 0).tolist() == torch.ones(4, 4).tril().bool().tolist()


def test_oracle_rotation_is_partial_paired_by_halves_and_slowed():
    rot = {'base': 100.0, 'dims': 4, 'scaling': {'factor': 2.0}}
    f = O.rot_frequencies(rot)
    assert torch.allclose(f, torch.tensor([0.5, 0.05], dtype=torch.float64))
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64).repeat(2, 1, 1)
    out = O.rotate(v, torch.tensor([0, 3]), rot)
    assert torch.equal(out[0], v[0]) and torch.equal(out[1, 0, 4:], v[1, 0, 4:])
    a0, a1 = 3 * 0.5, 3 * 0.05
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)]
    assert torch.allclose(out[1, 0, :4], torch.tensor(want, dtype=torch.float64))
    assert torch.equal(O.rotate(v, torch.tensor([0, 3]), None), v)


def test_oracle_matrix_memory_against_its_unrolled_sum():
    """the recurrence with its running maximum equals the direct sum over the past with the true (unstabilised) weights"""
    torch.manual_seed(0)
    T, W, H, d, dv, cap = 9, 12, 2, 4, 3, 6.0
    mc = dict(heads=H, dim=d, vdim=dv, gate_cap=cap)
    w = {'p.' + n: torch.randn(s, dtype=torch.float64) for n, s in
         dict(q=(H * d, W), k=(H * d, W), v=(H * dv, W), g=(H * dv, W), o=(W, H * dv), i=(H, W), f=(H, W)).items()}
    w['p.i.b'], w['p.f.b'] = torch.randn(H, dtype=torch.float64) * 3, torch.randn(H, dtype=torch.float64) * 3
    w['p.norm'] = torch.rand(H * dv, dtype=torch.float64) + 0.5
    u = torch.randn(T, W, dtype=torch.float64)
    got = O.matrix_memory(u, w, 'p.', mc, 1e-6)
    q = (u @ w['p.q'].T).view(T, H, d) * d ** -0.5
    k = (u @ w['p.k'].T).view(T, H, d)
    v = (u @ w['p.v'].T).view(T, H, dv)
    a = cap * torch.tanh((u @ w['p.i'].T + w['p.i.b']) / cap)
    b = torch.nn.functional.logsigmoid(cap * torch.tanh((u @ w['p.f'].T + w['p.f.b']) / cap))
    y = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        for t in range(T):
            # true weight of token s in the memory at t: e^(a_s + sum of b over (s, t]); m_t = max(sum of b over [0, t], largest log weight)
            lw = torch.stack([a[s, h] + b[s + 1:t + 1, h].sum() for s in range(t + 1)])
            m = torch.maximum(b[:t + 1, h].sum(), lw.max())
            num = sum(torch.exp(lw[s]) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            den = sum(torch.exp(lw[s]) * (q[t, h] @ k[s, h]) for s in range(t + 1))
            y[t, h] = num * torch.exp(-m) / (torch.maximum((den * torch.exp(-m)).abs(), torch.exp(-m)) + 1e-6)
    ref = (O.unit_rms(y, 1e-6).reshape(T, H * dv) * w['p.norm'] * torch.sigmoid(u @ w['p.g'].T)) @ w['p.o'].T
    assert torch.allclose(got, ref, atol=1e-9)


def test_oracle_router_groups_identity_experts_and_negative_choice_scores():
    W, n_out = 6, 6
    w = {'r.router': torch.zeros(n_out, W), 'r.correction': torch.tensor([-5.0, -9.0, -6.0, -7.0, -1.0, -8.0])}
    w['r.router'][:, 0] = torch.tensor([0.0, 1.0, 2.0, 3.0, 0.5, 0.2])
    h = torch.zeros(2, W)
    h[:, 0] = torch.tensor([1.0, -1.0])
    rc = {'experts': 4, 'identity': 2, 'top': 2, 'groups': {'count': 3, 'keep': 2}}
    ids, wt = O.route(h, w, 'r.', rc)
    prob = torch.softmax(h @ w['r.router'].T, -1)
    # every choice score is negative; groups {0,1} {2,3} {4,5} score by their best member: the last group (-1 + p) always wins, then
    # the better of the first two; masked members must count as minus infinity, not as zero
    for t in range(2):
        ch = prob[t] + w['r.correction']
        best = sorted(range(3), key=lambda g: -max(ch[2 * g], ch[2 * g + 1]))[:2]
        allowed = sorted((e for g in best for e in (2 * g, 2 * g + 1)), key=lambda e: -ch[e])[:2]
        assert ids[t].tolist() == allowed and 4 in allowed
        assert torch.allclose(wt[t], prob[t][ids[t]])
    assert float(wt.sum(-1).max()) < 1.0                       # the probabilities are taken as they are
    # identity experts return the input times the weight; no shared unit, no real expert chosen
    w2 = {'m.router': torch.tensor([[0.0] * W, [0.0] * W, [9.0] + [0.0] * (W - 1)]), 'm.e0.up': torch.randn(5, W), 'm.e0.down': torch.randn(W, 5),
          'm.e1.up': torch.randn(5, W), 'm.e1.down': torch.randn(W, 5)}
    x = torch.randn(3, W)
    x[:, 0] = 2.0
    out = O.moe_ff(x, w2, 'm.', {'expert': {'ff': 5}, 'router': {'experts': 2, 'identity': 1, 'top': 1}})
    p_id = torch.softmax(x @ w2['m.router'].T, -1)[:, 2:3]
    assert torch.allclose(out, p_id * x, atol=1e-6)
