"""Dugalix on the continuous-batching engine against the plain CPU restatement (oracle/dugalix_oracle.py).

Small random checkpoints of several shapes; the CUDA path (model, page pool with its state rows, engine, scheduler, public API,
trace runner) must give the oracle's logits whatever the schedule: whole prompts, token-by-token decoding, portions down to two
tokens, mixed batches, reused pages and slots. Each mechanism is also probed alone at the kernel level, with inputs made so that a
fault shows (one dominant key far back, at a page border, on either side of a window's or a kept prefix's edge; saturated gates;
choice scores that are all negative; a slot's stale state).
"""
import json
import os
import random
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32, B16 = torch.float32, torch.bfloat16
TOL = {F32: 2e-4, B16: 8e-2}


@pytest.fixture(scope='module')
def lib(dev):
    import phi3_b200  # noqa: F401
    from phi3_b200 import _lib
    _lib.lib()
    return _lib


def _mods():
    import phi3_b200  # noqa: F401
    from phi3_b200 import configs, weights, engine, dugalix, paged
    from oracle import dugalix_oracle as O
    return configs, weights, engine, dugalix, paged, O


def row_err(got, ref):
    """per row: rms of the mean-free difference, relative to the spread of the reference"""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.std()


def rel_err(got, ref):
    return float(row_err(got, ref).max())


def assert_close(got, ref, dtype, what=''):
    """fp32: every row within 2e-4. bf16: rounding may flip a near-tie of the router for a few tokens (random weights have such
    ties) and such a token then differs by a whole expert's output, so nine rows in ten must be within the rounding bound and the
    median well inside it"""
    e = row_err(got, ref)
    if dtype == F32:
        assert float(e.max()) < TOL[F32], (what, float(e.max()))
    else:
        q = torch.quantile(e, torch.tensor([0.5, 0.9], dtype=e.dtype))
        assert float(q[0]) < 0.04 and float(q[1]) < TOL[B16], (what, q.tolist(), float(e.max()))


def make(cfg_dict, dtype, seed=0):
    configs, weights, engine, dugalix, paged, O = _mods()
    w = weights.random_dugalix_weights(cfg_dict, seed)
    return dugalix.DugalixB200(cfg_dict, w, dtype=dtype), w


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def poison(eng):
    """whatever an earlier owner left must never be read: finite junk in the K/V pages (a masked key is multiplied by a zero
    weight), NaN in the state rows (a new sequence must not even load them)"""
    for t in eng.pool.k + eng.pool.v:
        t.fill_(300.0)
    for s in eng.pool.state:
        s.fill_(float('nan'))


def run_schedule(model, toks, cuts, max_tokens=None, engine=None, rid='r'):
    """feed `toks` in portions of the given sizes (the rest one by one); logits of every position, in order"""
    configs, weights, eng_mod, *_ = _mods()
    eng = engine or eng_mod.Engine(model, max_tokens or len(toks) + 64, 4)
    if engine is None:
        poison(eng)
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(eng.step([(rid, toks[at:at + n], list(range(n)))]))
        at += n
    eng.finish(rid)
    return torch.cat(out, 0)


# ------------------------------------------------------------------------------------------------ whole model, schedules
@pytest.mark.parametrize('dtype', [F32, B16])
def test_whole_prompt_and_every_layer_match_the_oracle(lib, dtype):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, dtype)
    toks = tokens(150, cfg['vocab'], 1)                       # more than two pages, several windows
    ref_trace = []
    ref = O.forward(cfg, w, toks, torch.float64, ref_trace)
    eng = engine.Engine(model, 256, 4)
    poison(eng)
    trace = []
    got = eng.step([('a', toks, list(range(len(toks))))], ['a'], trace=trace)
    assert_close(got, ref, dtype)
    assert len(trace) == len(ref_trace) == 4
    if dtype == F32:
        for i, (g, r) in enumerate(zip(trace, ref_trace)):
            assert (g.cpu().double() - r).abs().max() < 2e-4, f'residual stream after layer {i}'
    assert len(eng.pool.free_pages) == eng.pool.n_pages and len(eng.pool.free_slots) == 4
    assert len(eng.pool.state) == 6                           # a shift row per layer, a memory per parallel layer


@pytest.mark.parametrize('dtype', [F32, B16])
def test_prefill_then_token_by_token_decoding(lib, dtype):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, dtype, seed=2)
    toks = tokens(140, cfg['vocab'], 3)
    ref = O.forward(cfg, w, toks, torch.float64)
    got = run_schedule(model, toks, [30])                     # 110 decoded tokens: windows, kept prefixes and page borders pass by
    assert_close(got, ref, dtype)
    whole = run_schedule(model, toks, [len(toks)])
    if dtype == F32:
        assert rel_err(got, whole) < 1e-5
    else:
        assert_close(got, whole, dtype)


@pytest.mark.parametrize('cuts', [[2, 2, 3, 31, 33, 2, 64, 1, 2], [63, 2, 63, 2], [1, 1, 64, 65], [100, 2, 2], [5, 32, 37, 3]])
def test_prompt_portions_of_any_size(lib, cuts):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, F32, seed=4)
    toks = tokens(sum(cuts) + 5, cfg['vocab'], 5)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert rel_err(run_schedule(model, toks, cuts), ref) < TOL[F32]


@pytest.mark.parametrize('dtype', [F32, B16])
def test_mixed_batch_of_unequal_requests_equals_each_alone(lib, dtype):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, dtype, seed=6)
    lens = {'a': 150, 'b': 37, 'c': 2, 'd': 90}
    toks = {k: tokens(n, cfg['vocab'], 10 + i) for i, (k, n) in enumerate(lens.items())}
    alone = {k: run_schedule(model, t, [len(t)]) for k, t in toks.items()}
    eng = engine.Engine(model, 64 * 8, 4)
    poison(eng)
    plan = {'a': [40, 1, 1, 33, 1, 2, 72], 'b': [1, 30, 1, 1, 1, 3], 'c': [1, 1], 'd': [64, 1, 25]}   # sizes per step
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    for s in range(max(len(v) for v in plan.values())):
        entries = []
        for k in toks:
            if s < len(plan[k]) and at[k] < lens[k]:
                n = min(plan[k][s], lens[k] - at[k])
                entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
                at[k] += n
        lg = eng.step(entries)
        o = 0
        for k, t, wnt in entries:
            got[k].append(lg[o:o + len(wnt)])
            o += len(wnt)
    for k in toks:
        assert at[k] == lens[k]
        if dtype == F32:
            assert rel_err(torch.cat(got[k], 0), alone[k]) < 1e-5, k
        else:
            assert_close(torch.cat(got[k], 0), alone[k], dtype, k)
        assert_close(torch.cat(got[k], 0), O.forward(cfg, w, toks[k], torch.float64), dtype, k)


def test_pages_slots_and_state_rows_are_given_back_and_used_again(lib):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, F32, seed=7)
    eng = engine.Engine(model, 64 * 4, 2)                     # four pages, two slots
    poison(eng)
    seen = []
    for r in range(5):
        n = [130, 200, 70, 256, 129][r]
        toks = tokens(n, cfg['vocab'], 20 + r)
        got = run_schedule(model, toks, [50, 3, 70], engine=eng, rid=f'r{r}')   # the slot's state is the previous request's
        assert rel_err(got, O.forward(cfg, w, toks, torch.float64)) < TOL[F32], r
        seen.append(len(eng.pool.free_pages))
    assert seen == [4] * 5 and sorted(eng.pool.free_slots) == [0, 1]
    # two live requests interleaved, one leaves, a third takes its slot, pages and state rows while the other goes on
    ta, tb, tc = tokens(100, cfg['vocab'], 31), tokens(60, cfg['vocab'], 32), tokens(120, cfg['vocab'], 33)
    la = [eng.step([('a', ta[:50], list(range(50))), ('b', tb, list(range(60)))], ['b'])]
    la.append(eng.step([('a', ta[50:], list(range(50))), ('c', tc[:64], list(range(64)))]))
    lc = [la[1][50:], eng.step([('c', tc[64:], list(range(56)))], ['a', 'c'])]
    with pytest.raises(paged.PoolExhausted):
        eng.step([('x', tokens(64 * 5, cfg['vocab'], 1), [])])
    assert rel_err(torch.cat([la[0][:50], la[1][:50]], 0), O.forward(cfg, w, ta, torch.float64)) < TOL[F32]
    assert rel_err(torch.cat(lc, 0), O.forward(cfg, w, tc, torch.float64)) < TOL[F32]


def test_first_tokens_and_long_decoding(lib):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, F32, seed=8)
    for n in (1, 2, 3):
        toks = tokens(n, cfg['vocab'], 40 + n)
        assert rel_err(run_schedule(model, toks, [n]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]
    toks = tokens(230, cfg['vocab'], 44)
    assert rel_err(run_schedule(model, toks, [1]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]   # all decoded one by one


def test_a_request_that_sits_out_steps_keeps_its_state(lib):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, F32, seed=3)
    ta, tb = tokens(90, cfg['vocab'], 81), tokens(80, cfg['vocab'], 82)
    eng = engine.Engine(model, 64 * 4, 4)
    poison(eng)
    ga = [eng.step([('a', ta[:40], list(range(40)))])]
    gb = [eng.step([('b', tb[:33], list(range(33)))])]        # a is left out ...
    gb.append(eng.step([('b', tb[33:34], [0])]))
    lg = eng.step([('b', tb[34:], list(range(46))), ('a', ta[40:], list(range(50)))])   # ... and goes on behind b
    gb.append(lg[:46])
    ga.append(lg[46:])
    assert rel_err(torch.cat(ga, 0), O.forward(cfg, w, ta, torch.float64)) < TOL[F32]
    assert rel_err(torch.cat(gb, 0), O.forward(cfg, w, tb, torch.float64)) < TOL[F32]


@pytest.mark.parametrize('dtype', [F32, B16])
def test_captured_decode_steps_equal_eager_steps(lib, dtype):
    """decode-only steps replay a CUDA graph from their third occurrence on; the logits must be those of eager launches, bit for
    bit, while requests sit out steps, leave and hand their slot, pages and state rows to a newcomer"""
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix()
    model, w = make(cfg, dtype, seed=9)
    n_prompt = {'a': 120, 'b': 5, 'c': 70, 'd': 66}
    seqs = {k: tokens(n + 24, cfg['vocab'], 50 + i) for i, (k, n) in enumerate(n_prompt.items())}

    def run(graphs):
        eng = engine.Engine(model, 64 * 10, 4)
        eng.use_graphs = graphs
        poison(eng)
        got = {k: [] for k in seqs}
        at = dict(n_prompt)

        def step(names, end=()):
            entries = []
            for k in names:
                n = n_prompt[k] if not got[k] else 1
                lo = 0 if not got[k] else at[k]
                entries.append((k, seqs[k][lo:lo + n], [n - 1]))
                at[k] = lo + n
            lg = eng.step(entries, end)
            for i, k in enumerate(names):
                got[k].append(lg[i:i + 1])

        step(['a', 'b', 'c'])
        for s in range(20):
            live = ['a', 'c'] if 8 <= s < 12 else ['a', 'b', 'c']                  # b sits out four steps
            if s < 15:
                step(live)
            elif s == 15:
                step(live, ['c'])                                                # c leaves ...
                step(['d'])                                                      # ... and d takes its slot and pages
            else:
                step(['a', 'b', 'd'])
        return {k: torch.cat(v, 0) for k, v in got.items()}, eng

    eager, _ = run(False)
    replay, eng = run(True)
    assert any('graph' in g for g in eng._graphs.values()), 'no step was captured'
    for k in seqs:
        assert torch.equal(eager[k], replay[k]), k
        n = eager[k].shape[0]
        ref = O.forward(cfg, w, seqs[k][:n_prompt[k] + n - 1], torch.float64)[n_prompt[k] - 1:]
        assert_close(replay[k], ref, dtype, k)


def _rot(dims, factor=None, base=10000.0):
    return {'base': base, 'dims': dims, **({'scaling': {'factor': factor}} if factor else {})}


def _sig(heads, kv, dim, win, rd, scale=None, base=10000.0):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=dim, scale=scale or dim ** -0.5)
    if win:
        m['mask'] = {'size': win}
    if rd:
        m['rot'] = _rot(rd, None, base)
    return {'type': 'attention', 'mixer': m}


def _par(lh, lkv, ld, lv, win, keep, rd, rh, rdim, rv, ls=0.8, rs=1.1, factor=4.0, cap=15.0):
    left = dict(heads=lh, kv_heads=lkv, dim=ld, vdim=lv, scale=ld ** -0.5)
    if win:
        left['mask'] = {'size': win, **({'keep_first': keep} if keep else {})}
    if rd:
        left['rot'] = _rot(rd, factor)
    return {'type': 'parallel', 'mixer': {'left': left, 'right': dict(heads=rh, dim=rdim, vdim=rv, gate_cap=cap),
                                          'left_scale': ls, 'right_scale': rs}}


def _moe(ff, e, ident, top, groups=None, shared=None):
    return {'kind': 'moe', 'expert': {'ff': ff},
            'router': dict(experts=e, identity=ident, top=top, **({'groups': {'count': groups[0], 'keep': groups[1]}} if groups else {})),
            **({'shared': {'ff': shared}} if shared else {})}


_dense = lambda ff: {'kind': 'dense', 'ff': ff}

OTHER = {
    # one head everywhere, sizes that are no multiple of 8 (every product on the FMA kernels), window 1 and 2, a kept prefix longer
    # than the window and longer than a page, top == router outputs, one expert per group with all groups kept
    'odd': (52, 1.0, [dict(_par(1, 1, 12, 20, 2, 70, 6, 1, 10, 7), mlp=_moe(20, 3, 1, 4, (4, 4), 12)),
                      dict(_sig(1, 1, 10, 1, 10), mlp=_dense(30)),
                      dict(_sig(3, 1, 6, 2, 2), mlp=_moe(12, 3, 0, 1, None, None))]),
    # tensor-core sizes; heads == kv heads; attention layers first and two parallel layers in a row; no rotation at all in one
    # mixer, no window in another; memory keys of 128 and values that take several column blocks
    'tiles': (128, 0.5, [dict(_sig(4, 4, 64, 48, 32), mlp=_moe(64, 8, 8, 4, (4, 2), 64)),
                         dict(_par(4, 4, 32, 32, 0, 0, 0, 2, 128, 96), mlp=_dense(256)),
                         dict(_par(8, 2, 64, 64, 40, 40, 64, 4, 64, 64, factor=None), mlp=_moe(32, 6, 2, 2, (2, 1), 128))]),
    # memory keys above 128 numbers, values that are no multiple of the column block, more memory heads than attention heads,
    # identity experts only in the best group's neighbourhood, a very small gate cap (the gates saturate)
    'wide': (96, 1.3, [dict(_par(2, 1, 40, 24, 50, 3, 16, 5, 136, 40, cap=1.5), mlp=_moe(24, 2, 4, 2, (3, 2), None)),
                       dict(_sig(2, 2, 136, 64, 24, base=500.0), mlp=None),
                       dict(_par(3, 3, 16, 72, 64, 64, 8, 1, 200, 33, ls=1.0, rs=0.25), mlp=_moe(16, 4, 1, 5, None, 40))]),
    # nothing is a multiple of 4
    'ragged': (50, 0.9, [dict(_par(3, 1, 6, 5, 9, 2, 2, 3, 7, 5), mlp=_moe(11, 5, 2, 2, None, 13)),
                         dict(_sig(2, 1, 14, 7, 6), mlp=_moe(7, 3, 3, 3, (3, 2), 9))]),
}


@pytest.mark.parametrize('name', list(OTHER))
@pytest.mark.parametrize('dtype', [F32, B16])
def test_other_sizes(lib, name, dtype):
    configs, weights, engine, dugalix, paged, O = _mods()
    width, mult, layers = OTHER[name]
    cfg = configs.tiny_dugalix(width=width, vocab=211 if name != 'ragged' else 101, layers=layers, residual_mult=mult)
    model, w = make(cfg, dtype, seed=11)
    toks = tokens(150, cfg['vocab'], 12)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert_close(run_schedule(model, toks, [70, 2, 40]), ref, dtype, name)


def test_small_batches_take_the_weight_streaming_products(lib):
    configs, weights, engine, dugalix, paged, O = _mods()
    cfg = configs.tiny_dugalix(width=128, vocab=256, layers=[dict(_par(4, 2, 32, 32, 48, 4, 32, 2, 32, 64), mlp=_moe(64, 4, 2, 2, (2, 1), 64)),
                                                             dict(_sig(4, 2, 32, 40, 16), mlp=_dense(192))])
    model, w = make(cfg, B16, seed=15)
    toks = tokens(40, cfg['vocab'], 16)
    ref = O.forward(cfg, w, toks, torch.float64)
    a = run_schedule(model, toks, [20])
    model.use_skinny = False
    b = run_schedule(model, toks, [20])
    assert_close(a, ref, B16)
    assert_close(b, ref, B16)


def _random_config(rng):
    """a configuration drawn at random: layer count and order of the two kinds, head counts and sizes (with and without the
    tensor-core kernels), windows, kept prefixes, rotation constants, memory shapes, feed-forwards of every kind or none"""
    width, vocab = rng.choice([64, 96, 128, 160, 200]), rng.choice([97, 256, 1000])
    layers = []
    for _ in range(rng.randint(1, 4)):
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        tc = rng.random() < 0.5
        dim = rng.choice([16, 32, 64]) if tc else rng.choice([6, 10, 20, 36])
        win = rng.choice([0, 1, 5, 31, 64, 100])
        rd = rng.choice([0, 2, dim // 2 * 2, dim // 4 * 2])
        if rng.random() < 0.5:
            mix = _sig(heads, kv, dim, win, rd)
        else:
            vd = rng.choice([8, 16, 40]) if tc else rng.choice([5, 12, 33])
            mix = _par(heads, kv, dim, vd, win, rng.choice([0, 1, 7, 64, 90]) if win else 0, rd, rng.choice([1, 2, 3]),
                       rng.choice([8, 24, 70]), rng.choice([8, 31, 48]), ls=rng.uniform(0.3, 1.2), rs=rng.uniform(0.3, 1.2),
                       factor=rng.choice([None, 2.0, 8.0]), cap=rng.choice([3.0, 15.0, 30.0]))
        kind = rng.choice(['none', 'dense', 'moe', 'moe'])
        if kind == 'none':
            mlp = None
        elif kind == 'dense':
            mlp = _dense(rng.choice([24, 50, 128]))
        else:
            groups = rng.choice([None, (2, 1), (3, 2), (4, 4)])
            per = rng.choice([1, 2, 3])
            n_out = (groups[0] if groups else rng.choice([2, 3, 5])) * per
            ident = rng.randint(0, n_out - 1)
            cap_top = n_out if not groups else groups[1] * per
            mlp = _moe(rng.choice([8, 24, 40]), n_out - ident, ident, rng.randint(1, cap_top), groups, rng.choice([None, 16, 48]))
        layers.append(dict(mix, mlp=mlp))
    return {'architecture': 'Dugalix', 'vocab': vocab, 'width': width, 'norm': {'eps': rng.choice([1e-6, 1e-5])},
            'residual_mult': rng.choice([1.0, 0.5, 1.4]), 'layers': layers}


@pytest.mark.parametrize('seed', [21, 22, 23, 24, 25, 26])
def test_random_configurations_under_random_schedules(lib, seed):
    """five requests of random lengths through four slots and a pool too small for all of them at once, in steps that mix portions of
    random sizes (from two tokens) with single tokens and idle steps; every logit against the oracle"""
    configs, weights, engine, dugalix, paged, O = _mods()
    rng = random.Random(seed)
    cfg = _random_config(rng)
    dtype = F32 if seed % 2 else B16
    model, w = make(cfg, dtype, seed=seed)
    lens = [rng.choice([1, 2, 3, 40, 64, 65, 130, 190]) for _ in range(5)]
    toks = [tokens(n, cfg['vocab'], seed * 10 + i) for i, n in enumerate(lens)]
    eng = engine.Engine(model, 64 * 7, 4)
    poison(eng)
    at, got, waiting, live = [0] * 5, [[] for _ in range(5)], list(range(5)), []
    while waiting or live:
        while waiting and len(live) < 4 and eng.can_take(waiting[0], lens[waiting[0]]) \
                and sum(-(-lens[i] // 64) for i in live + [waiting[0]]) <= 7:
            live.append(waiting.pop(0))
        entries, end = [], []
        for i in live:
            if rng.random() < 0.2:
                continue                                       # sits this step out
            n = min(rng.choice([1, 1, 2, 3, 17, 64, 70]), lens[i] - at[i])
            entries.append((i, toks[i][at[i]:at[i] + n], list(range(n))))
            at[i] += n
            if at[i] == lens[i]:
                end.append(i)
        if not entries:
            continue
        lg = eng.step(entries, end)
        o = 0
        for i, t, wnt in entries:
            got[i].append(lg[o:o + len(wnt)])
            o += len(wnt)
        live = [i for i in live if i not in end]
    for i in range(5):
        assert_close(torch.cat(got[i], 0), O.forward(cfg, w, toks[i], torch.float64), dtype, (seed, i, json.dumps(cfg)[:300]))


# ------------------------------------------------------------------------------------------------ mechanisms alone
def _attention_case(dtype, H, G, d, dv, n_ctx, window, keep, hot, sigmoid, scale=1.0, seed=0, tile_rows=32, n_splits=1, out_scale=1.0):
    """random queries, keys and values with a few dominant (query, key) pairs `hot` = [(i, j)]: both rows get a large common
    component, so that the weight of that pair dwarfs the rest when it is visible and a lost, misplaced or wrongly masked key
    changes the output completely. With sigmoid weights the bias is very negative: only a dominant pair has a weight near 1.
    Returns (prefill result, decode result, plain reference)."""
    from phi3_b200._lib import AttnWindowArgs, call_struct, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_ctx, H, d, generator=g) * 0.5
    k = torch.randn(n_ctx, G, d, generator=g) * 0.5
    v = torch.randn(n_ctx, G, dv, generator=g)
    for n, (i, j) in enumerate(hot):
        u = torch.zeros(d)
        u[n % d] = 6.0
        q[i] += u
        k[j] += u
    bias = torch.full((H,), -14.0) + torch.arange(H) * 0.25
    if dtype == B16:
        q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
    ii, jj = torch.arange(n_ctx)[:, None], torch.arange(n_ctx)[None, :]
    vis = (jj <= ii) & ((ii - jj < window) | (jj < keep) if window else torch.ones(n_ctx, n_ctx, dtype=torch.bool))
    ref = torch.zeros(n_ctx, H, dv, dtype=torch.float64)
    for h in range(H):
        sc = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        wgt = torch.sigmoid(sc + bias[h].double()) * vis if sigmoid else torch.softmax(sc.masked_fill(~vis, float('-inf')), -1)
        ref[:, h] = wgt @ v[:, h // (H // G)].double() * out_scale
    n_pg = -(-n_ctx // 64)
    perm = torch.randperm(n_pg + 3, generator=g)[:n_pg]
    kp, vp = torch.full((n_pg + 3, G, 64, d), 50.0), torch.full((n_pg + 3, G, 64, dv), -70.0)
    for p in range(n_pg):
        n = min(64, n_ctx - 64 * p)
        kp[perm[p], :, :n] = k[64 * p:64 * p + n].transpose(0, 1)
        vp[perm[p], :, :n] = v[64 * p:64 * p + n].transpose(0, 1)
    bt = torch.zeros(2, n_pg + 3, dtype=torch.int32)
    bt[1, :n_pg] = perm.int()
    kp, vp, bt = kp.to(dev, dtype), vp.to(dev, dtype), bt.to(dev)
    qd, bd = q.reshape(n_ctx, H * d).to(dev, dtype).contiguous(), bias.to(dev)
    outs = []
    for kind in ('prefill', 'decode'):
        if kind == 'prefill':
            tiles = [(r0, min(tile_rows, n_ctx - r0), 1, r0) for r0 in range(0, n_ctx, tile_rows)]
        else:
            tiles = [(r, 1, 1, r) for r in range(n_ctx)]
        td = torch.tensor(tiles, dtype=torch.int32, device=dev).reshape(-1)
        out = torch.zeros(n_ctx, H * dv, dtype=dtype, device=dev)
        a_ = AttnWindowArgs()
        a_.q, a_.ld_q, a_.k_pool, a_.v_pool, a_.block_table, a_.bt_stride = ptr(qd), H * d, ptr(kp), ptr(vp), ptr(bt), bt.stride(0)
        a_.out, a_.ld_out = ptr(out), H * dv
        a_.n_heads, a_.n_kv, a_.dim, a_.vdim, a_.scale, a_.window, a_.keep_first = H, G, d, dv, scale, window, keep
        a_.sig_bias, a_.out_scale = (ptr(bd) if sigmoid else None), out_scale
        a_.act_f32 = a_.cache_f32 = int(dtype == F32)
        a_.tiles, a_.n_tiles = ptr(td), len(tiles)
        if kind == 'decode' and n_splits > 1:
            ws = torch.empty(len(tiles) * H * n_splits * (dv + 2), device=dev)
            a_.n_splits, a_.ws = n_splits, ptr(ws)
        call_struct('p3_attn_window_' + kind, a_, 0)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().reshape(n_ctx, H, dv))
    return outs[0], outs[1], ref


def _tile_rows(lib, dtype, H, G, d, dv, window, keep, sigmoid):
    import ctypes as C
    a = lib.AttnWindowArgs()
    a.q = a.out = a.k_pool = a.v_pool = a.block_table = a.tiles = 256
    a.ld_q, a.ld_out, a.n_heads, a.n_kv, a.dim, a.vdim, a.window, a.keep_first = H * d, H * dv, H, G, d, dv, window, keep
    a.sig_bias = 256 if sigmoid else None
    a.act_f32 = a.cache_f32 = int(dtype == F32)
    return int(lib.lib().p3_attn_window_tile_rows(C.byref(a)))


@pytest.mark.parametrize('shape', [(3, 1, 28, 20), (4, 2, 80, 40), (4, 2, 64, 64), (8, 2, 128, 128), (6, 3, 24, 40), (20, 1, 32, 16),
                                   (2, 1, 264, 40), (4, 2, 160, 136)])
@pytest.mark.parametrize('sigmoid', [False, True])
@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('n_splits', [1, 3])
def test_attention_windows_kept_first_tokens_far_keys_and_page_borders(lib, shape, sigmoid, dtype, n_splits):
    """a window with the first tokens kept (softmax), or the window alone (sigmoid weights; there the values are given their own
    pool like any others). Dominant pairs sit just inside and just outside the window, just inside and outside the kept prefix seen
    from far away and from nearby, at page borders, at the query's own position and at the first positions."""
    H, G, d, dv = shape
    if sigmoid:
        dv = d
    n, window, keep = 300, 36, (0 if sigmoid else 12)
    inside, outside = window - 1, window                      # distances of the last visible and the first hidden key
    hot = [(299, 0), (298, keep - 1 if keep else 1), (297, keep), (296, 296 - inside), (295, 295 - outside), (294, 256), (293, 255),
           (200, 200 - inside), (201, 201 - outside), (131, 63), (132, 64), (133, 128), (64, 64), (63, 63), (128, 128), (1, 0), (2, 2),
           (keep + inside, keep), (keep + outside, keep), (keep + outside - 1, keep - 1 if keep else 0), (70, keep - 1 if keep else 3),
           (191, 191 - inside), (192, 192 - outside), (255 + inside, 255), (256 + inside, 256), (256 + outside, 256), (100, 5), (90, 64),
           (64 + outside, 64), (63 + inside, 63)]
    tile = _tile_rows(lib, dtype, H, G, d, dv, window, keep, sigmoid)
    pf, dc, ref = _attention_case(dtype, H, G, d, dv, n, window, keep, hot, sigmoid, scale=0.7, tile_rows=tile, n_splits=n_splits,
                                  out_scale=0.6)
    tol = 1e-4 if dtype == F32 else 3e-2
    assert (pf.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    assert (dc.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize('window,keep', [(1, 0), (1, 3), (2, 64), (64, 65), (5, 200), (0, 9), (130, 1)])
def test_attention_window_and_prefix_sizes(lib, window, keep):
    hot = [(150, 0), (151, 2), (152, 3), (149, 148), (148, 146), (147, 64), (146, 65), (145, 63), (199, 70), (198, 69), (197, 68)]
    for sigmoid in (False, True):
        pf, dc, ref = _attention_case(F32, 4, 2, 16, 16, 200, window, keep, hot, sigmoid, scale=0.5, seed=3)
        assert (pf.double() - ref).abs().max() < 1e-4 and (dc.double() - ref).abs().max() < 1e-4


@pytest.mark.parametrize('W', [70, 72])                       # scalar and 16-byte paths
def test_token_shift_carries_the_last_row_of_a_slot(lib, W):
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    n_slots = 3
    g = torch.Generator().manual_seed(5)
    shift = torch.rand(W, generator=g)
    state = torch.full((n_slots, W), float('nan'))
    hist = {1: torch.randn(9, W, generator=g), 2: torch.randn(4, W, generator=g)}
    # step 1: slot 2 brings rows 0..2 (first position 0: the NaN row must not be read), slot 1 brings row 0
    # step 2: slot 1 brings rows 1..8, slot 2 brings row 3
    plans = [[(2, 0, 3), (1, 0, 1)], [(1, 1, 8), (2, 3, 1)]]
    sd = state.to(dev)
    got = {1: [], 2: []}
    for plan in plans:
        rows, seqs, tok_slot, slot_seq = [], [], [], [0] * n_slots
        for slot, p0, n in plan:
            slot_seq[slot] = len(seqs)
            seqs.append((len(tok_slot), n, slot, p0))
            tok_slot += [slot] * n
            rows.append(hist[slot][p0:p0 + n])
        h = torch.cat(rows, 0).to(dev)
        out = torch.empty_like(h)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev).reshape(-1)
        keep = [shift.to(dev), i32(seqs), i32(slot_seq), i32(tok_slot)]      # device copies must outlive the launch
        call('p3_token_shift', ptr(h), ptr(keep[0]), ptr(sd), ptr(keep[1]), ptr(keep[2]), ptr(keep[3]), ptr(out), 1, h.shape[0], W, 0)
        torch.cuda.synchronize()
        o = 0
        for slot, p0, n in plan:
            got[slot].append(out[o:o + n].cpu())
            o += n
    for slot, hs in hist.items():
        prev = torch.cat([torch.zeros(1, W), hs[:-1]], 0)
        assert torch.allclose(torch.cat(got[slot], 0), hs + (prev - hs) * shift, atol=1e-6)
        assert torch.equal(sd[slot].cpu(), hs[-1])
    assert torch.isnan(sd[0]).all()                           # a slot without tokens is not touched


@pytest.mark.parametrize('shape', [(2, 24, 40), (1, 7, 5), (3, 64, 64), (2, 128, 96), (1, 200, 33), (5, 136, 70), (1, 300, 40)])
@pytest.mark.parametrize('cap,rs', [(15.0, 0), (1.5, 0), (15.0, 2), (15.0, 4), (15.0, 8)])
def test_matrix_memory_scan_in_portions_and_with_saturated_gates(lib, shape, cap, rs):
    """the recurrence alone: whole sequences against the token loop of the oracle, then the same sequences in portions (the state
    rows carry on) with a second sequence in the batch, bit for bit equal to the whole run. Gate pre-activations are made large so
    that the caps, the stabiliser and the lower bound of the denominator are all exercised. rs: the shape of a warp (0: the launch's own choice)"""
    configs, weights, engine, dugalix, paged, O = _mods()
    from phi3_b200._lib import MatrixMemoryArgs, call_struct, call, ptr
    dev = torch.device('cuda')
    H, d, dv = shape
    g = torch.Generator().manual_seed(7)
    T = {0: 83, 1: 37}
    cols = 2 * H * d + 2 * H * dv + 2 * H
    off = dict(q=0, k=H * d, v=2 * H * d, g=2 * H * d + H * dv, i=2 * H * d + 2 * H * dv, f=2 * H * d + 2 * H * dv + H)
    proj = {s: torch.randn(n, cols, generator=g) for s, n in T.items()}
    for s in proj:
        proj[s][:, off['i']:] *= 6.0                          # gate pre-activations far beyond a small cap, on both sides
        proj[s][20:30, off['f']:] = -20.0                     # the memory is wiped ...
        proj[s][30:35, off['i']:off['f']] = -20.0             # ... and then fed with next to nothing: the denominator's floor decides
    ib, fb = torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0
    gain = torch.rand(H * dv, generator=g) + 0.5
    eye = lambda n: torch.eye(n, dtype=torch.float64)
    ref = {}
    for s in proj:                                             # the oracle's mixer with identity projections: u = proj itself
        pw = {'p.q': eye(cols)[off['q']:off['k']], 'p.k': eye(cols)[off['k']:off['v']], 'p.v': eye(cols)[off['v']:off['g']],
              'p.g': eye(cols)[off['g']:off['i']], 'p.i': eye(cols)[off['i']:off['f']], 'p.f': eye(cols)[off['f']:],
              'p.i.b': ib.double(), 'p.f.b': fb.double(), 'p.norm': gain.double(), 'p.o': eye(H * dv)}
        ref[s] = O.matrix_memory(proj[s].double(), pw, 'p.', dict(heads=H, dim=d, vdim=dv, gate_cap=cap), 1e-6)
    n_state = int(lib.lib().p3_matrix_memory_state_floats(H, d, dv))

    def run(plans):
        state = torch.full((3, n_state), float('nan'), device=dev)
        got = {s: [] for s in T}
        for plan in plans:
            seqs, rows = [], []
            r0 = 0
            for slot, p0, n in plan:
                seqs.append((r0, n, slot, p0))
                rows.append(proj[slot - 1][p0:p0 + n])
                r0 += n
            pd = torch.cat(rows, 0).to(dev)
            y, out, den = torch.empty(r0, H * dv, device=dev), torch.empty(r0, H * dv, device=dev), torch.empty(r0, H, device=dev)
            sq = torch.tensor(seqs, dtype=torch.int32, device=dev).reshape(-1)
            a = MatrixMemoryArgs()
            a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.i_off, a.f_off = ptr(pd), cols, off['q'], off['k'], off['v'], off['i'], off['f']
            ibd, fbd, gd = ib.to(dev), fb.to(dev), gain.to(dev)
            a.i_bias, a.f_bias, a.n_heads, a.dim, a.vdim, a.q_scale, a.gate_cap = ptr(ibd), ptr(fbd), H, d, dv, d ** -0.5, cap
            a.state, a.seqs, a.n_seqs, a.out, a.ld_out, a.den, a.rs_force = ptr(state), ptr(sq), len(seqs), ptr(y), H * dv, ptr(den), rs
            call_struct('p3_matrix_memory_scan', a, 0)
            call('p3_headnorm_gate', ptr(y), H * dv, ptr(den), H, dv, ptr(gd), ptr(pd[:, off['g']:]), cols, 1.0, 1e-6, ptr(out), H * dv, 1, r0, 0)
            torch.cuda.synchronize()
            o = 0
            for slot, p0, n in plan:
                got[slot - 1].append(out[o:o + n].cpu())
                o += n
        return {s: torch.cat(v, 0) for s, v in got.items()}

    whole = run([[(1, 0, 83), (2, 0, 37)]])                    # sequence s lives in slot s + 1
    parts = run([[(1, 0, 17)], [(2, 0, 2), (1, 17, 1)], [(1, 18, 16), (2, 2, 33)], [(1, 34, 1)], [(2, 35, 2), (1, 35, 48)]])
    for s in T:
        scale = float(ref[s].abs().max())
        assert (whole[s].double() - ref[s]).abs().max() < 2e-4 * max(1.0, scale), s
        assert torch.equal(whole[s], parts[s]), s


@pytest.mark.parametrize('case', ['random', 'negative', 'no_groups', 'single', 'many'])
def test_router_softmax_scores_correction_groups_and_plain_weights(lib, case):
    configs, weights, engine, dugalix, paged, O = _mods()
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(9)
    T = 57
    E, top, groups, keep = {'random': (12, 3, 3, 2), 'negative': (8, 3, 4, 2), 'no_groups': (7, 2, 1, 1), 'single': (4, 4, 4, 4),
                            'many': (96, 6, 8, 3)}[case]
    z = torch.randn(T, E + 3, generator=g) * 2.0               # the logits are columns of a wider product
    corr = torch.randn(E, generator=g) * 0.2 - (3.0 if case == 'negative' else 0.0)
    W = 5
    rw = {'r.router': torch.eye(E + 3, dtype=torch.float64)[:E], 'r.correction': corr.double()}
    rc = {'experts': E, 'top': top, **({'groups': {'count': groups, 'keep': keep}} if groups > 1 else {})}
    ids_ref, wt_ref = O.route(z.double(), rw, 'r.', rc)
    ids = torch.empty(T, top, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top, device=dev)
    zd, cd = z.to(dev), corr.to(dev)
    call('p3_router_groups', ptr(zd), E + 3, ptr(cd), T, E, top, groups, keep, 1.0, lib.ROUTER_SOFTMAX | lib.ROUTER_GROUP_MAX | lib.ROUTER_PLAIN_WEIGHTS,
         ptr(ids), ptr(wts), 0)
    for t in range(T):
        ref = {int(e): float(v) for e, v in zip(ids_ref[t], wt_ref[t])}
        got = {int(e): float(v) for e, v in zip(ids[t].cpu(), wts[t].cpu())}
        assert got.keys() == ref.keys(), (t, got, ref)
        assert max(abs(got[k] - ref[k]) for k in ref) < 1e-6
    if groups > 1:
        assert all(len({int(e) // (E // groups) for e in ids[t].cpu()}) <= keep for t in range(T))


@pytest.mark.parametrize('dtype', [F32, B16])
def test_rotation_biases_and_keys_that_double_as_values(lib, dtype):
    configs, weights, engine, dugalix, paged, O = _mods()
    from phi3_b200._lib import QkvRopePostArgs, call_struct, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(11)
    for H, G, d, dv, rot_n, values in ((4, 2, 24, 40, 16, True), (3, 3, 20, 20, 20, False), (2, 1, 9, 9, 0, False), (2, 2, 66, 10, 6, True)):
        T = 5
        pos = torch.tensor([0, 1, 63, 64, 300])
        cols = (H + G) * d + (G * dv if values else 0) + 3
        proj, bias = torch.randn(T, cols, generator=g), torch.randn(cols, generator=g)
        rot = {'base': 10000.0, 'dims': rot_n, 'scaling': {'factor': 2.0}} if rot_n else None
        freq = torch.tensor(configs.rot_frequencies(configs.DugalixConfig._attention(0, dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=1.0, rot=rot), 'softmax').rot),
                            dtype=torch.float64).float().to(dev) if rot_n else None
        full = (proj + bias).double()
        q_ref = O.rotate(full[:, :H * d].view(T, H, d), pos, rot)
        k_plain = full[:, H * d:(H + G) * d].view(T, G, d)
        k_ref = O.rotate(k_plain, pos, rot)
        v_ref = full[:, (H + G) * d:(H + G) * d + G * dv].view(T, G, dv) if values else k_plain
        n_pages = 17
        kp, vp = torch.zeros(n_pages, G, 64, d, dtype=dtype, device=dev), torch.zeros(n_pages, G, 64, dv, dtype=dtype, device=dev)
        bt = torch.arange(n_pages - 1, -1, -1, dtype=torch.int32, device=dev).reshape(1, -1).contiguous()
        qo = torch.empty(T, H * d, dtype=dtype, device=dev)
        pd, bd = proj.to(dev), bias.to(dev)
        slot, pd_pos = torch.zeros(T, dtype=torch.int32, device=dev), pos.int().to(dev)
        a = QkvRopePostArgs()
        a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.bias = ptr(pd), cols, 0, H * d, ((H + G) * d if values else -1), ptr(bd)
        a.n_heads, a.n_kv, a.dim, a.vdim, a.rot_n, a.freq = H, G, d, dv, rot_n, ptr(freq)
        a.q_out, a.ld_q, a.k_pool, a.v_pool, a.block_table, a.bt_stride = ptr(qo), H * d, ptr(kp), ptr(vp), ptr(bt), n_pages
        a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(slot), ptr(pd_pos), T, int(dtype == F32), int(dtype == F32)
        call_struct('p3_qkv_rope_post', a, 0)
        torch.cuda.synchronize()
        tol = 2e-4 if dtype == F32 else 3e-2                    # position 300 times a frequency in fp32: some 1e-5 of an angle
        assert (qo.float().cpu().view(T, H, d).double() - q_ref).abs().max() < tol
        for t, p in enumerate(pos.tolist()):
            page = n_pages - 1 - p // 64
            assert (kp[page, :, p % 64].float().cpu().double() - k_ref[t]).abs().max() < tol
            assert (vp[page, :, p % 64].float().cpu().double() - v_ref[t]).abs().max() < tol


def test_sandwich_norms_relu2_unit_and_identity_combine(lib):
    configs, weights, engine, dugalix, paged, O = _mods()
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(13)
    for W in (50, 128, 1100, 8200):                           # the last one is longer than the threads' registers hold
        T = 7
        x, y, yb = torch.randn(T, W, generator=g), torch.randn(T, W + 3, generator=g) * 3, torch.randn(W, generator=g)
        g1, g2 = torch.randn(W, generator=g) * 0.1, torch.randn(W, generator=g) * 0.1
        r, eps = 0.6, 1e-5
        x_ref = x.double() + r * O.norm1p(y[:, :W].double() + yb.double(), g1.double(), eps)
        h_ref = O.norm1p(x_ref, g2.double(), eps)
        xd, yd = x.to(dev), y.to(dev)
        h32, hb = torch.empty(T, W, device=dev), torch.empty(T, W, dtype=B16, device=dev)
        post, pre, ybd = ((1 + g1) * r).to(dev), (1 + g2).to(dev), yb.to(dev)
        call('p3_postnorm_prenorm', ptr(yd), W + 3, ptr(ybd), ptr(post), ptr(xd), ptr(pre), ptr(h32), ptr(hb), 0, T, W, eps, 0)
        assert (xd.cpu().double() - x_ref).abs().max() < 1e-5 and (h32.cpu().double() - h_ref).abs().max() < 1e-5
        assert (hb.float().cpu().double() - h_ref).abs().max() < 3e-2
        x2 = x.to(dev)
        call('p3_postnorm_prenorm', None, 0, None, None, ptr(x2), ptr(pre), ptr(h32), None, 1, T, W, eps, 0)   # the first norm of a step
        assert torch.equal(x2.cpu(), x) and (h32.cpu().double() - O.norm1p(x.double(), g2.double(), eps)).abs().max() < 1e-5
    for R, F, pad in ((9, 37, 2), (9, 40, 4)):                # scalar and 16-byte paths
        u, gate = torch.randn(R, F + pad, generator=g), torch.randn(R, 4, generator=g)
        ud, gd = u.to(dev), gate.to(dev)
        out, outb = torch.empty(R, F, device=dev), torch.empty(R, F, dtype=B16, device=dev)
        call('p3_relu2', ptr(ud), F + pad, ptr(gd[:, 1:]), 4, ptr(out), F, 1, R, F, 0)
        ref = O.relu2(u[:, :F].double()) * torch.sigmoid(gate[:, 1:2].double())
        assert (out.cpu().double() - ref).abs().max() < 1e-5
        call('p3_relu2', ptr(ud), F + pad, ptr(gd[:, 1:]), 4, ptr(outb), F, 0, R, F, 0)
        assert (outb.float().cpu().double() - ref).abs().max() < 3e-2 * float(ref.abs().max())
        call('p3_relu2', ptr(ud), F + pad, None, 0, ptr(out), F, 1, R, F, 0)
        assert (out.cpu().double() - O.relu2(u[:, :F].double())).abs().max() < 1e-5
    # weighted sum over sorted expert rows, identity experts and the shared unit's rows
    T, top, W, n_real = 6, 3, 20, 4
    ids = torch.stack([torch.randperm(7, generator=g)[:top] for _ in range(T)]).int()
    wts, h, add = torch.rand(T, top, generator=g), torch.randn(T, W, generator=g), torch.randn(T, W + 1, generator=g)
    where = torch.randperm(T * top, generator=g).int()
    yrows = torch.randn(T * top, W, generator=g)
    yrows[where.long()[(ids >= n_real).reshape(-1)]] = float('nan')      # rows of identity pairs are never produced, never read
    ref = torch.stack([sum(wts[t, j].double() * (yrows[where[t * top + j]].double() if ids[t, j] < n_real else h[t].double())
                           for j in range(top)) + add[t, :W].double() for t in range(T)])
    out = torch.empty(T, W, device=dev)
    keep = [t.to(dev) for t in (yrows, where, ids, wts, h, add)]           # device copies must outlive the launch
    call('p3_moe_combine_identity', ptr(keep[0]), W, ptr(keep[1]), ptr(keep[2]), ptr(keep[3]), top, n_real, ptr(keep[4]), ptr(keep[5]),
         W + 1, ptr(out), T, W, 0)
    assert (out.cpu().double() - ref).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------ public entry points
def test_greedy_generation_through_load_generate_and_the_scheduler(lib, tmp_path):
    configs, weights, engine, dugalix, paged, O = _mods()
    from phi3_b200 import api
    from safetensors.torch import save_file
    cfg = configs.tiny_dugalix()
    w = weights.random_dugalix_weights(cfg, 13)
    json.dump(cfg, open(tmp_path / 'config.json', 'w'))
    save_file(w, str(tmp_path / 'model.safetensors'))
    model, proc = api.load(model_path=str(tmp_path), dtype=F32)
    assert type(model).__name__ == 'DugalixB200'
    prompts = [tokens(n, cfg['vocab'], 60 + n) for n in (70, 3, 130, 20, 65)]
    n_new = 12
    # five requests through two slots and a pool of 8 pages: queueing, portions, slot, page and state reuse
    from phi3_b200.engine import generate_tokens
    outs = generate_tokens(model, prompts, max_new=n_new, max_tokens=64 * 8, n_slots=2, token_budget=96, chunk=40)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(O.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        assert o == seq[len(p):]
    assert api.generate_batch(prompts[:2], preload=(model, proc), max_tokens=n_new, return_tokens=True) == outs[:2]
    text = api.generate('hello there', preload=(model, proc), max_tokens=5, verbose=False)
    assert isinstance(text, str)


def test_trace_runner_replays_steps(lib, tmp_path):
    configs, weights, engine, dugalix, paged, O = _mods()
    from safetensors.torch import save_file
    import numpy as np
    cfg = configs.tiny_dugalix()
    w = weights.random_dugalix_weights(cfg, 14)
    mdir, out = tmp_path / 'm', tmp_path / 'out'
    mdir.mkdir()
    json.dump(cfg, open(mdir / 'config.json', 'w'))
    save_file(w, str(mdir / 'model.safetensors'))
    a, b = tokens(80, cfg['vocab'], 70), tokens(9, cfg['vocab'], 71)
    steps = [{'step': 0, 'entries': [{'id': 'a', 'tokens': a[:70], 'want': [0, 69]}, {'id': 'b', 'tokens': b[:2], 'want': []}], 'end': []},
             {'step': 1, 'entries': [{'id': 'b', 'tokens': b[2:], 'want': [6]}], 'end': ['b']},
             {'step': 2, 'entries': [{'id': 'a', 'tokens': a[70:71], 'want': []}], 'end': []},
             {'step': 3, 'entries': [{'id': 'a', 'tokens': a[71:], 'want': [8]}], 'end': ['a']}]
    for dt, tol in (('float32', TOL[F32]), ('bfloat16', TOL[B16])):
        r = subprocess.run([os.path.join(ROOT, 'bin', 'trace_run'), '--model', str(mdir), '--dtype', dt, '--out', str(out),
                            '--max-tokens', '192'], input='\n'.join(json.dumps(s) for s in steps) + '\n', capture_output=True,
                           text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith('done')] == ['done 0', 'done 1', 'done 2', 'done 3']
        ra, rb = O.forward(cfg, w, a, torch.float64), O.forward(cfg, w, b, torch.float64)
        rd = lambda n: torch.from_numpy(np.fromfile(out / f'{n}.f32', dtype='<f4').reshape(-1, cfg['vocab']))
        assert not (out / '2.f32').exists()
        assert rel_err(rd(0), ra[[0, 69]]) < tol and rel_err(rd(1), rb[[8]]) < tol and rel_err(rd(3), ra[[79]]) < tol
        for f in out.iterdir():
            f.unlink()
