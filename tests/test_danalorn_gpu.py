"""Danalorn on the continuous-batching engine against the plain CPU restatement (oracle/danalorn_oracle.py).

Small random checkpoints of several shapes; the CUDA path (model, page pool with its state rows, engine, scheduler, public API,
trace runner) must give the oracle's logits whatever the schedule: whole prompts, token-by-token decoding, portions down to two
tokens, mixed batches, reused pages and slots. Each mechanism is also probed alone at the kernel level, with inputs made so that a
fault shows (one dominant key far back, at a page border, on either side of a window's edge; a sink that takes most of the weight;
decays at both ends of their range; a slot's stale state).
"""
import json
import math
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
    from phi3_b200 import configs, weights, engine, danalorn, paged
    from oracle import danalorn_oracle as O
    return configs, weights, engine, danalorn, paged, O


def row_err(got, ref):
    """per row: rms of the mean-free difference, relative to the spread of the reference"""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.std()


def rel_err(got, ref):
    return float(row_err(got, ref).max())


def assert_close(got, ref, dtype, what='', loose=False):
    """fp32: every row within 2e-4. bf16: every row within the rounding bound and the median well inside it. loose (random
    configurations in bf16): nine rows in ten. The read-out of a recurrent head is divided by its own root mean square, so where a
    sequence's first tokens happen to give q . k near zero the rounding of the inputs decides the sign of the whole head, and such a
    row differs by a head's output however exact the kernels are."""
    e = row_err(got, ref)
    if dtype == F32:
        assert float(e.max()) < TOL[F32], (what, float(e.max()))
    elif loose:
        q = torch.quantile(e, torch.tensor([0.5, 0.9], dtype=e.dtype))
        assert float(q[0]) < 0.03 and float(q[1]) < TOL[B16], (what, q.tolist(), float(e.max()))
    else:
        assert float(e.median()) < 0.03 and float(e.max()) < TOL[B16], (what, float(e.median()), float(e.max()))


def make(cfg_dict, dtype, seed=0):
    configs, weights, engine, danalorn, paged, O = _mods()
    w = weights.random_danalorn_weights(cfg_dict, seed)
    return danalorn.DanalornB200(cfg_dict, w, dtype=dtype), w


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def poison(eng):
    """whatever an earlier owner left must never be read: finite junk in the cache pages (a masked key is multiplied by a zero
    weight), NaN in the matrix states (a new sequence must not even load them), a junk token in the last-token row"""
    for t in eng.pool.k + eng.pool.v:
        t.fill_(300.0)
    eng.pool.state[0].view(torch.int32).fill_(12345)
    for s in eng.pool.state[1:]:
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
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
    model, w = make(cfg, dtype)
    toks = tokens(150, cfg['vocab'], 1)                       # more than two pages, several windows
    ref_trace = []
    ref = O.forward(cfg, w, toks, torch.float64, ref_trace)
    eng = engine.Engine(model, 256, 4)
    poison(eng)
    trace = []
    got = eng.step([('a', toks, list(range(len(toks))))], ['a'], trace=trace)
    assert_close(got, ref, dtype)
    assert len(trace) == len(ref_trace) == 7
    if dtype == F32:
        for i, (g, r) in enumerate(zip(trace, ref_trace)):
            assert (g.cpu().double() - r).abs().max() < 2e-4 * float(r.abs().max()), f'residual stream after layer {i}'
    assert len(eng.pool.free_pages) == eng.pool.n_pages and len(eng.pool.free_slots) == 4
    assert len(eng.pool.state) == 3                           # the last token, a matrix state per recurrent layer


@pytest.mark.parametrize('dtype', [F32, B16])
def test_prefill_then_token_by_token_decoding(lib, dtype):
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
    model, w = make(cfg, dtype, seed=2)
    toks = tokens(140, cfg['vocab'], 3)
    ref = O.forward(cfg, w, toks, torch.float64)
    got = run_schedule(model, toks, [30])                     # 110 decoded tokens: windows and page borders pass by
    assert_close(got, ref, dtype)
    whole = run_schedule(model, toks, [len(toks)])
    if dtype == F32:
        assert rel_err(got, whole) < 1e-5
    else:
        assert_close(got, whole, dtype)


@pytest.mark.parametrize('cuts', [[2, 2, 3, 31, 33, 2, 64, 1, 2], [63, 2, 63, 2], [1, 1, 64, 65], [100, 2, 2], [5, 32, 37, 3]])
def test_prompt_portions_of_any_size(lib, cuts):
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
    model, w = make(cfg, F32, seed=4)
    toks = tokens(sum(cuts) + 5, cfg['vocab'], 5)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert rel_err(run_schedule(model, toks, cuts), ref) < TOL[F32]


@pytest.mark.parametrize('dtype', [F32, B16])
def test_mixed_batch_of_unequal_requests_equals_each_alone(lib, dtype):
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
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
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
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
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
    model, w = make(cfg, F32, seed=8)
    for n in (1, 2, 3):
        toks = tokens(n, cfg['vocab'], 40 + n)
        assert rel_err(run_schedule(model, toks, [n]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]
    toks = tokens(230, cfg['vocab'], 44)
    assert rel_err(run_schedule(model, toks, [1]), O.forward(cfg, w, toks, torch.float64)) < TOL[F32]   # all decoded one by one


def test_a_request_that_sits_out_steps_keeps_its_state(lib):
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
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
    configs, weights, engine, danalorn, paged, O = _mods()
    cfg = configs.tiny_danalorn()
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


# ------------------------------------------------------------------------------------------------ other sizes
def _la(heads, dim, rd, vdim, rank, qrank, win, rdims=None, base=10000.0, kv_from=None, scale=None):
    return {'type': 'latent_attention',
            'mixer': dict(heads=heads, dim=dim, rot_dim=rd, vdim=vdim, kv_rank=rank, q_rank=qrank, scale=scale or (dim + rd) ** -0.5,
                          rot={'base': base, 'dims': rdims or rd}, **({'mask': {'size': win}} if win else {}),
                          **({'kv_from': kv_from} if kv_from is not None else {}))}


def _att(heads, kv, dim, vdim, qt=None, scale=None):
    return {'type': 'attention', 'mixer': dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale or dim ** -0.5,
                                               **({'q_temp': {'coef': qt[0], 'every': qt[1]}} if qt else {}))}


def _gla(heads, dim, vdim, tau, rank=16):
    return {'type': 'gla', 'mixer': dict(heads=heads, dim=dim, vdim=vdim, tau=tau, decay_rank=rank)}


def _dense(ff):
    return {'kind': 'dense', 'ff': ff}


OTHER = {
    # every head count 1, window 1 (a token sees itself alone), one bucket, tau 1, a query temperature that grows every token
    'ones': (64, dict(bigram=(1, 1, 1), embed_scale=1.0),
             [dict(_la(1, 16, 16, 16, 16, 16, 1), mlp=_dense(64)), dict(_att(1, 1, 16, 16, (1.0, 1)), mlp=_dense(64)),
              dict(_gla(1, 16, 16, 1.0, 1), mlp=None), dict(_la(1, 8, 16, 8, 16, 8, 2, kv_from=0), mlp=_dense(16))]),
    # sizes that tile the tensor-core kernels and equal each other; the borrowing layer comes right after its source
    'tiled': (128, dict(bigram=(1031, 37, 11), embed_scale=11.3),
              [dict(_la(4, 32, 32, 32, 96, 64, 64), mlp=_dense(256)), dict(_la(8, 32, 32, 64, 96, 128, 65, kv_from=0), mlp=_dense(128)),
               dict(_att(8, 2, 64, 64, (0.25, 32)), mlp=_dense(256)), dict(_gla(4, 64, 64, 12.0), mlp=_dense(256)),
               dict(_att(4, 4, 128, 128), mlp=_dense(128)), dict(_gla(2, 128, 128, 20.0, 32), mlp=_dense(128))]),
    # nothing is a multiple of 8: every product goes through the any-shape kernel, every attention through the fp32 kernels; the last
    # layer has no turning part at all
    'ragged': (50, dict(bigram=(97, 1000003, 999983), embed_scale=0.5),
               [dict(_gla(3, 7, 9, 2.5, 3), mlp=_dense(33)), dict(_la(3, 10, 6, 7, 11, 13, 63, rdims=2), mlp=_dense(21)),
                dict(_att(6, 2, 10, 14, (2.0, 3)), mlp=None), dict(_la(2, 5, 6, 9, 11, 9, 0, rdims=2, kv_from=1), mlp=_dense(19)),
                dict(_gla(1, 130, 5, 30.0, 5), mlp=_dense(10)), dict(_la(2, 12, 0, 10, 20, 6, 9), mlp=_dense(12))]),
    # no pair table, two sources with two borrowers each way around, a window longer than anything fed, wide heads, a decay
    # projection of rank 80 (products of its own) and one of rank 33
    'wide': (96, dict(bigram=None, embed_scale=3.0),
             [dict(_la(2, 64, 64, 96, 128, 48, 1000), mlp=_dense(96)), dict(_la(3, 24, 16, 40, 56, 24, 40), mlp=None),
              dict(_la(2, 16, 16, 24, 56, 40, 20, kv_from=1), mlp=_dense(48)), dict(_la(4, 32, 64, 32, 128, 96, 33, kv_from=0), mlp=None),
              dict(_att(12, 1, 24, 200), mlp=_dense(48)), dict(_gla(2, 260, 72, 9.0, 80), mlp=_dense(40)), dict(_gla(2, 16, 24, 5.0, 33), mlp=None)]),
}


@pytest.mark.parametrize('name', list(OTHER))
@pytest.mark.parametrize('dtype', [F32, B16])
def test_other_sizes(lib, name, dtype):
    configs, weights, engine, danalorn, paged, O = _mods()
    width, emb, layers = OTHER[name]
    cfg = configs.tiny_danalorn(width=width, vocab=211 if name != 'ragged' else 101, layers=layers, **emb)
    model, w = make(cfg, dtype, seed=11)
    toks = tokens(150, cfg['vocab'], 12)
    ref = O.forward(cfg, w, toks, torch.float64)
    assert_close(run_schedule(model, toks, [70, 2, 40]), ref, dtype, name)


def test_small_batches_take_the_weight_streaming_products(lib):
    configs, weights, engine, danalorn, paged, O = _mods()
    width, emb, layers = OTHER['tiled']
    cfg = configs.tiny_danalorn(width=width, vocab=256, layers=layers, **emb)
    model, w = make(cfg, B16, seed=15)
    toks = tokens(40, cfg['vocab'], 16)
    ref = O.forward(cfg, w, toks, torch.float64)
    a = run_schedule(model, toks, [20])
    model.use_skinny = False
    b = run_schedule(model, toks, [20])
    assert_close(a, ref, B16)
    assert_close(b, ref, B16)


def _random_config(rng):
    """a random order of the three mixers with random sizes; a latent layer borrows an earlier latent layer's cache now and then"""
    width = rng.choice([48, 64, 72, 96])
    layers, sources = [], []
    for i in range(rng.randint(2, 6)):
        kind = rng.choice(['latent_attention', 'attention', 'gla'])
        mlp = _dense(rng.choice([24, 40, 64])) if rng.random() < 0.8 else None
        if kind == 'latent_attention':
            heads, dim, vdim = rng.randint(1, 5), rng.choice([8, 16, 24]), rng.choice([8, 16, 40])
            win = rng.choice([0, 1, 5, 33, 64, 100])
            if sources and rng.random() < 0.5:
                j = rng.choice(sources)
                sm = layers[j]['mixer']
                lay = _la(heads, dim, sm['rot_dim'], vdim, sm['kv_rank'], rng.choice([8, 24, 40]), win, rdims=sm['rot']['dims'],
                          base=sm['rot']['base'], kv_from=j)
            else:
                rd = rng.choice([2, 8, 16])
                lay = _la(heads, dim, rd, vdim, rng.choice([16, 24, 56]), rng.choice([8, 24, 40]), win,
                          rdims=rng.choice([d for d in (2, 4, 8, 16) if d <= rd]), base=rng.choice([100.0, 10000.0, 1000000.0]))
                sources.append(i)
        elif kind == 'attention':
            kv = rng.randint(1, 3)
            lay = _att(kv * rng.randint(1, 3), kv, rng.choice([8, 16, 40]), rng.choice([8, 24, 32]),
                       rng.choice([None, (0.25, 32), (0.7, 5), (0.1, 1)]))
        else:
            lay = _gla(rng.randint(1, 4), rng.choice([8, 24, 40, 72]), rng.choice([8, 24, 40, 70]), rng.choice([1.0, 4.0, 12.0]),
                       rng.choice([2, 8, 16]))
        layers.append(dict(lay, mlp=mlp))
    bigram = rng.choice([None, (rng.choice([5, 64, 509]), rng.randint(1, 99), rng.randint(1, 99))])
    return configs_mod().tiny_danalorn(width=width, vocab=rng.choice([77, 128, 300]), layers=layers, bigram=bigram,
                                       embed_scale=rng.choice([1.0, 4.0, 12.0]))


def configs_mod():
    return _mods()[0]


@pytest.mark.parametrize('seed', [21, 22, 23, 24, 25, 26])
def test_random_configurations_under_random_schedules(lib, seed):
    """random layer orders and sizes, random requests fed in random portions beside each other through a pool that forces pages,
    slots and state rows to change hands"""
    configs, weights, engine, danalorn, paged, O = _mods()
    rng = random.Random(seed)
    cfg = _random_config(rng)
    dtype = F32 if seed % 2 else B16
    model, w = make(cfg, dtype, seed=seed)
    lens = [rng.choice([1, 2, 3, 30, 64, 65, 100, 129, 190]) for _ in range(6)]
    toks = [tokens(n, cfg['vocab'], seed * 10 + i) for i, n in enumerate(lens)]
    ref = [O.forward(cfg, w, t, torch.float64) for t in toks]
    eng = engine.Engine(model, 64 * 8, 3)
    poison(eng)
    fed, got = [0] * 6, [[] for _ in range(6)]
    live, nxt = [], 0
    while nxt < 6 or live:
        while nxt < 6 and len(live) < 3 and eng.can_take(f'r{nxt}', min(lens[nxt], 64)) and \
                sum(-(-lens[i] // 64) for i in live) + -(-lens[nxt] // 64) <= 8:
            live.append(nxt)
            nxt += 1
        entries, end = [], []
        for i in live:
            if rng.random() < 0.2 and len(live) > 1 and entries:
                continue                                       # sits this step out
            n = min(lens[i] - fed[i], rng.choice([1, 1, 2, 3, 17, 64, 100]))
            entries.append((f'r{i}', toks[i][fed[i]:fed[i] + n], list(range(n))))
            fed[i] += n
            if fed[i] == lens[i]:
                end.append(f'r{i}')
        lg = eng.step(entries, end)
        o = 0
        for rid, t, _ in entries:
            got[int(rid[1:])].append(lg[o:o + len(t)])
            o += len(t)
        live = [i for i in live if fed[i] < lens[i]]
    if dtype == F32:
        for i in range(6):
            assert_close(torch.cat(got[i], 0), ref[i], dtype, (seed, i))
    else:
        assert_close(torch.cat([torch.cat(g, 0) for g in got], 0), torch.cat(ref, 0), dtype, seed, loose=True)


# ------------------------------------------------------------------------------------------------ mechanisms alone
def _attention_case(dtype, H, G, d, dv, n_ctx, window, hot, *, scale=1.0, seed=0, tile_rows=32, n_splits=1, sink=None, slope=None,
                    gate=False, shared_row=False):
    """random queries, keys and values with a few dominant (query, key) pairs `hot` = [(i, j)]: both rows get a large common
    component, so that the weight of that pair dwarfs the rest when it is visible and a lost, misplaced or wrongly masked key
    changes the output completely. sink: per-head numbers in the softmax denominator; slope: per-head linear distance bias (as a
    table); gate: element-wise sigmoid gate on the outputs; shared_row: ONE key row per token serves all heads and its leading dv
    numbers are the value (the latent cache layout). Returns (prefill result, decode result, plain reference)."""
    from phi3_b200._lib import AttnWindowArgs, call_struct, ptr
    dev = torch.device('cuda')
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_ctx, H, d, generator=g) * 0.5
    k = torch.randn(n_ctx, G, d, generator=g) * 0.5
    v = torch.randn(n_ctx, G, dv, generator=g)
    for n, (i, j) in enumerate(hot):
        u = torch.zeros(d)
        u[d - 1 - n % 4] = 6.0                                 # in the trailing numbers: the leading ones double as values
        q[i] += u
        k[j] += u
    if shared_row:
        assert G == 1 and dv <= d
        v = k[:, :, :dv].clone()
    logits = torch.randn(n_ctx, H * dv, generator=g) * 2.0
    if dtype == B16:
        q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
    ii, jj = torch.arange(n_ctx)[:, None], torch.arange(n_ctx)[None, :]
    vis = (jj <= ii) & ((ii - jj < window) if window else torch.ones(n_ctx, n_ctx, dtype=torch.bool))
    ref = torch.zeros(n_ctx, H, dv, dtype=torch.float64)
    for h in range(H):
        sc = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        if slope is not None:
            sc = sc - float(torch.tensor(slope[h], dtype=torch.float32)) * (ii - jj).double()
        sc = sc.masked_fill(~vis, float('-inf'))
        if sink is None:
            wgt = torch.softmax(sc, -1)
        else:
            m = torch.clamp(sc.max(-1, keepdim=True).values, min=float(sink[h]))
            e = torch.exp(sc - m)
            wgt = e / (e.sum(-1, keepdim=True) + torch.exp(sink[h].double() - m))
        ref[:, h] = wgt @ v[:, h // (H // G)].double()
    if gate:
        ref = ref * torch.sigmoid(logits.double()).view(n_ctx, H, dv)
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
    qd = q.reshape(n_ctx, H * d).to(dev, dtype).contiguous()
    keep = [None if sink is None else sink.float().to(dev), logits.to(dev)]
    if slope is not None:
        keep.append((torch.tensor(slope, dtype=torch.float32)[:, None] * torch.arange(n_ctx, dtype=torch.float32)[None, :]).to(dev))
    outs = []
    for kind in ('prefill', 'decode'):
        if kind == 'prefill':
            tiles = [(r0, min(tile_rows, n_ctx - r0), 1, r0) for r0 in range(0, n_ctx, tile_rows)]
        else:
            tiles = [(r, 1, 1, r) for r in range(n_ctx)]
        td = torch.tensor(tiles, dtype=torch.int32, device=dev).reshape(-1)
        out = torch.zeros(n_ctx, H * dv, dtype=dtype, device=dev)
        a_ = AttnWindowArgs()
        a_.q, a_.ld_q, a_.k_pool, a_.block_table, a_.bt_stride = ptr(qd), H * d, ptr(kp), ptr(bt), bt.stride(0)
        a_.v_pool, a_.v_ld = (ptr(kp), d) if shared_row else (ptr(vp), 0)
        a_.out, a_.ld_out = ptr(out), H * dv
        a_.n_heads, a_.n_kv, a_.dim, a_.vdim, a_.scale, a_.window = H, G, d, dv, scale, window
        a_.sink = ptr(keep[0])
        if slope is not None:
            a_.penalty, a_.n_penalty = ptr(keep[2]), n_ctx
        if gate:
            a_.elem_gate, a_.ld_elem_gate = ptr(keep[1]), H * dv
        a_.act_f32 = a_.cache_f32 = int(dtype == F32)
        a_.tiles, a_.n_tiles = ptr(td), len(tiles)
        if kind == 'decode' and n_splits > 1:
            ws = torch.empty(len(tiles) * H * n_splits * (dv + 2), device=dev)
            a_.n_splits, a_.ws = n_splits, ptr(ws)
        call_struct('p3_attn_window_' + kind, a_, 0)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().reshape(n_ctx, H, dv))
    return outs[0], outs[1], ref


def _tile_rows(lib, dtype, H, G, d, dv, v_ld):
    import ctypes as C
    a = lib.AttnWindowArgs()
    a.q = a.out = a.k_pool = a.v_pool = a.block_table = a.tiles = 256
    a.ld_q, a.ld_out, a.n_heads, a.n_kv, a.dim, a.vdim, a.v_ld = H * d, H * dv, H, G, d, dv, v_ld
    a.act_f32 = a.cache_f32 = int(dtype == F32)
    return int(lib.lib().p3_attn_window_tile_rows(C.byref(a)))


@pytest.mark.parametrize('shape', [(3, 28, 20), (6, 96, 64), (4, 48, 40), (2, 264, 200), (5, 160, 128)])
@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('n_splits', [1, 3])
def test_latent_rows_window_edges_sink_far_keys_and_page_borders(lib, shape, dtype, n_splits):
    """one shared key row per token whose leading numbers are the value, a sliding window and a sink per head. Dominant pairs sit
    just inside and just outside the window, at page borders, at the query's own position and at the first positions; one head's
    sink outweighs every ordinary key, another's is negligible."""
    H, d, dv = shape
    n, window = 300, 36
    inside, outside = window - 1, window                      # distances of the last visible and the first hidden key
    hot = [(299, 0), (296, 296 - inside), (295, 295 - outside), (294, 256), (293, 255), (200, 200 - inside), (201, 201 - outside),
           (131, 63 + 64), (132, 132 - inside), (64, 64), (63, 63), (128, 128), (1, 0), (2, 2), (inside, 0), (outside, 0),
           (191, 191 - inside), (192, 192 - outside), (255 + inside, 255), (256 + inside, 256), (256 + outside, 256),
           (64 + outside, 64), (63 + inside, 63), (127, 127 - inside), (100, 100 - outside)]
    sink = torch.linspace(-6.0, 5.0, H)
    tile = _tile_rows(lib, dtype, H, 1, d, dv, d)
    pf, dc, ref = _attention_case(dtype, H, 1, d, dv, n, window, hot, scale=0.7, tile_rows=tile, n_splits=n_splits, sink=sink,
                                  shared_row=True)
    tol = 1e-4 if dtype == F32 else 3e-2
    assert (pf.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    assert (dc.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    # the sink matters: without it the weights of a row add up to one
    _, _, plain = _attention_case(dtype, H, 1, d, dv, n, window, hot, scale=0.7, shared_row=True)
    assert (plain - ref).abs().max() > 0.05


@pytest.mark.parametrize('shape', [(4, 2, 48, 48), (6, 3, 24, 40), (8, 2, 64, 64), (12, 1, 40, 200), (1, 1, 128, 128)])
@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('n_splits', [1, 4])
def test_causal_attention_with_linear_distance_bias_unit_sink_and_gate(lib, shape, dtype, n_splits):
    """no window: a dominant key hundreds of tokens back must still be found, weakened by exactly slope * distance; one is added to
    the denominator; every output number has a gate of its own"""
    H, G, d, dv = shape
    n = 400
    hot = [(399, 0), (398, 63), (397, 64), (396, 396), (395, 200), (300, 1), (257, 255), (256, 256), (255, 0), (129, 128), (64, 0),
           (63, 62), (1, 0), (0, 0), (390, 127), (391, 128), (392, 320)]
    slope = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    tile = _tile_rows(lib, dtype, H, G, d, dv, 0)
    pf, dc, ref = _attention_case(dtype, H, G, d, dv, n, 0, hot, scale=0.5, tile_rows=tile, n_splits=n_splits,
                                  sink=torch.zeros(H), slope=slope, gate=True)
    tol = 1e-4 if dtype == F32 else 3e-2
    assert (pf.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    assert (dc.double() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    _, _, flat = _attention_case(dtype, H, G, d, dv, n, 0, hot, scale=0.5, sink=torch.zeros(H), gate=True)
    assert (flat - ref).abs().max() > 0.05                     # the distance bias changes the answer


@pytest.mark.parametrize('window', [1, 2, 63, 64, 65, 130, 0])
def test_window_sizes_around_a_page(lib, window):
    hot = [(150, 0), (151, 150), (152, 150), (149, 86), (148, 85), (147, 84), (146, 83), (145, 81), (199, 70), (198, 134), (197, 133), (196, 131)]
    pf, dc, ref = _attention_case(F32, 4, 1, 16, 8, 200, window, hot, scale=0.5, seed=3, sink=torch.tensor([0.0, 1.0, -1.0, 3.0]),
                                  shared_row=True)
    assert (pf.double() - ref).abs().max() < 1e-4 and (dc.double() - ref).abs().max() < 1e-4


@pytest.mark.parametrize('W', [40, 44, 2048])                  # 16-byte path, scalar path, rows longer than one pass of the CTA
def test_pair_embedding_carries_the_last_token_of_a_slot(lib, W):
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    V, buckets, mp, mc, n_slots = 50, 13, 1000003, 7, 3
    g = torch.Generator().manual_seed(5)
    table, pairs = torch.randn(V, W, generator=g).bfloat16(), torch.randn(buckets + 1, W, generator=g).bfloat16()
    hist = {1: torch.randint(0, V, (9,), generator=g).tolist(), 2: torch.randint(0, V, (4,), generator=g).tolist()}
    state = torch.full((n_slots, 1), 777, dtype=torch.int32, device=dev)       # junk: position 0 must not read it
    # step 1: slot 2 brings tokens 0..2, slot 1 brings token 0; step 2: slot 1 brings tokens 1..8, slot 2 brings token 3
    plans = [[(2, 0, 3), (1, 0, 1)], [(1, 1, 8), (2, 3, 1)]]
    td, pd = table.to(dev), pairs.to(dev)
    got = {1: [], 2: []}
    for plan in plans:
        ids, seqs, tok_slot, slot_seq = [], [], [], [0] * n_slots
        for slot, p0, n in plan:
            slot_seq[slot] = len(seqs)
            seqs.append((len(tok_slot), n, slot, p0))
            tok_slot += [slot] * n
            ids += hist[slot][p0:p0 + n]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev).reshape(-1)
        keep = [i32(ids), i32(seqs), i32(slot_seq), i32(tok_slot)]
        x = torch.empty(len(ids), W, device=dev)
        call('p3_embed_pair_rows_f32', ptr(td), ptr(pd), ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), ptr(keep[3]), ptr(state), 1, ptr(x),
             len(ids), W, V, 3.0, buckets, mp, mc, 0)
        torch.cuda.synchronize()
        o = 0
        for slot, p0, n in plan:
            got[slot].append(x[o:o + n].cpu())
            o += n
    for slot, toks in hist.items():
        rows = [buckets] + [(toks[t - 1] * mp + toks[t] * mc) % buckets for t in range(1, len(toks))]
        want = table[torch.tensor(toks)].float() * 3.0 + pairs[torch.tensor(rows)].float()
        assert torch.equal(torch.cat(got[slot], 0), want), slot
        assert int(state[slot, 0]) == toks[-1]
    assert int(state[0, 0]) == 777                             # a slot without tokens is not touched
    # without a pair table the rows are the scaled token rows, and the last token is still recorded
    x = torch.empty(2, W, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev).reshape(-1)
    keep = [i32([4, 5]), i32([(0, 2, 0, 7)]), i32([0, 0, 0]), i32([0, 0])]
    call('p3_embed_pair_rows_f32', ptr(td), None, ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), ptr(keep[3]), ptr(state), 1, ptr(x), 2, W, V,
         0.5, 1, 0, 0, 0)
    torch.cuda.synchronize()
    assert torch.equal(x.cpu(), table[torch.tensor([4, 5])].float() * 0.5) and int(state[0, 0]) == 5


@pytest.mark.parametrize('dtype', [F32, B16])
@pytest.mark.parametrize('sizes', [(3, 16, 8, 24, 40, 8), (2, 7, 6, 5, 11, 2), (4, 32, 32, 32, 64, 32), (2, 8, 4, 1100, 16, 4)])
def test_latent_post_norms_neighbour_pairs_and_both_calls(lib, dtype, sizes):
    """the two calls of the latent post kernel against plain torch: low-rank query vector and latent vector normed, the shared key
    part rotated as neighbour pairs into the cache row; then the query parts from a second product split and rotated"""
    from phi3_b200._lib import LatentPostArgs, call_struct, ptr
    configs, weights, engine, danalorn, paged, O = _mods()
    dev = torch.device('cuda')
    H, d, dr, Q, R, rot_n = sizes
    T, eps = 70, 1e-5
    g = torch.Generator().manual_seed(9)
    proj = torch.randn(T, Q + R + dr + 3, generator=g)        # a few unrelated columns behind
    qf = torch.randn(T, H * (d + dr), generator=g)
    cq_gain, c_gain = torch.rand(Q, generator=g) + 0.5, torch.rand(R, generator=g) + 0.5
    rot = {'base': 300.0, 'dims': rot_n}
    freq = torch.tensor([300.0 ** (-2.0 * i / rot_n) for i in range(rot_n // 2)], dtype=torch.float64).float()
    pos = torch.arange(T) * 37 % 200                           # positions in two sequences' pages, out of order
    slot = (torch.arange(T) % 2).int()
    bt = torch.tensor([[5, 1, 3, 0], [2, 6, 4, 7]], dtype=torch.int32)
    cache = torch.full((8, 1, 64, R + dr), 9.0, dtype=dtype, device=dev)
    cq, qp, ql = (torch.zeros(T, n, dtype=dtype, device=dev) for n in (Q, H * d, H * (R + dr)))
    keep = [proj.to(dev), qf.to(dev), cq_gain.to(dev), c_gain.to(dev), freq.to(dev), bt.to(dev), slot.to(dev), pos.int().to(dev)]
    a = LatentPostArgs()
    a.proj, a.ld_proj, a.c_off, a.cq_off, a.q_rank = ptr(keep[0]), proj.shape[1], Q, 0, Q
    a.n_heads, a.dim, a.rot_dim, a.kv_rank, a.rot_n, a.pair_mode = 0, d, dr, R, rot_n, 1
    a.c_gain, a.cq_gain, a.eps, a.freq, a.rot_mag = ptr(keep[3]), ptr(keep[2]), eps, ptr(keep[4]), 1.0
    a.cq_out, a.ld_cq, a.cache = ptr(cq), Q, ptr(cache)
    a.block_table, a.bt_stride, a.tok_slot, a.tok_pos, a.T = ptr(keep[5]), 4, ptr(keep[6]), ptr(keep[7]), T
    a.act_f32 = a.cache_f32 = int(dtype == F32)
    call_struct('p3_latent_post', a, 0)
    b = LatentPostArgs()
    b.q_src, b.ld_qsrc = ptr(keep[1]), qf.shape[1]
    b.n_heads, b.dim, b.rot_dim, b.kv_rank, b.rot_n, b.pair_mode = H, d, dr, R, rot_n, 1
    b.eps, b.freq, b.rot_mag = eps, ptr(keep[4]), 1.0
    b.q_plain, b.ld_qp, b.q_lat, b.ld_ql = ptr(qp), H * d, ptr(ql), H * (R + dr)
    b.block_table, b.bt_stride, b.tok_slot, b.tok_pos, b.T = ptr(keep[5]), 4, ptr(keep[6]), ptr(keep[7]), T
    b.act_f32 = b.cache_f32 = int(dtype == F32)
    call_struct('p3_latent_post', b, 0)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == F32 else 2e-2
    assert (cq.float().cpu() - O.rms_norm(proj[:, :Q], cq_gain, eps)).abs().max() < tol
    c_ref = O.rms_norm(proj[:, Q:Q + R], c_gain, eps)
    kr_ref = O.rotate_pairs(proj[:, Q + R:Q + R + dr].reshape(T, 1, dr), pos, rot)[:, 0]
    rows = torch.stack([cache[int(bt[int(slot[t]), int(pos[t]) // 64]), 0, int(pos[t]) % 64] for t in range(T)]).float().cpu()
    assert (rows[:, :R] - c_ref).abs().max() < tol and (rows[:, R:] - kr_ref).abs().max() < 2 * tol
    q3 = qf.view(T, H, d + dr)
    assert (qp.float().cpu().view(T, H, d) - q3[..., :d]).abs().max() < tol
    assert (ql.float().cpu().view(T, H, R + dr)[..., R:] - O.rotate_pairs(q3[..., d:], pos, rot)).abs().max() < 2 * tol
    assert float(ql.float().abs().view(T, H, R + dr)[..., :R].max()) == 0.0     # left for the product with the key up-projection


@pytest.mark.parametrize('dtype', [F32, B16])
def test_query_key_norm_with_biases_and_query_temperature(lib, dtype):
    from phi3_b200._lib import QkvPostArgs, call_struct, ptr
    configs, weights, engine, danalorn, paged, O = _mods()
    dev = torch.device('cuda')
    H, G, d, dv, every, coef, eps = 6, 2, 24, 40, 8, 0.6, 1e-5
    g = torch.Generator().manual_seed(4)
    pos = torch.tensor([0, 1, 6, 7, 8, 14, 15, 16, 63, 64, 127, 190, 191])      # on both sides of multiples of `every`, minus one
    T = len(pos)
    nq, nk, nv = H * d, G * d, G * dv
    proj, bias = torch.randn(T, nq + nk + nv + 5, generator=g), torch.randn(nq + nk + nv, generator=g)
    qg, kg = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    bt = torch.tensor([[2, 0, 1]], dtype=torch.int32)
    kp, vp = torch.zeros(3, G, 64, d, dtype=dtype, device=dev), torch.zeros(3, G, 64, dv, dtype=dtype, device=dev)
    q = torch.zeros(T, nq, dtype=dtype, device=dev)
    keep = [proj.to(dev), bias.to(dev), qg.to(dev), kg.to(dev), bt.to(dev), torch.zeros(T, dtype=torch.int32, device=dev), pos.int().to(dev)]
    a = QkvPostArgs()
    a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.bias = ptr(keep[0]), proj.shape[1], 0, nq, nq + nk, ptr(keep[1])
    a.n_heads, a.n_kv, a.dim, a.vdim, a.q_gain, a.k_gain, a.eps = H, G, d, dv, ptr(keep[2]), ptr(keep[3]), eps
    a.q_temp_coef, a.q_temp_every = coef, every
    a.q_out, a.ld_q, a.k_pool, a.v_pool = ptr(q), nq, ptr(kp), ptr(vp)
    a.block_table, a.bt_stride, a.tok_slot, a.tok_pos, a.T = ptr(keep[4]), 3, ptr(keep[5]), ptr(keep[6]), T
    a.act_f32 = a.cache_f32 = int(dtype == F32)
    call_struct('p3_qkv_post', a, 0)
    torch.cuda.synchronize()
    temp = 1.0 + coef * torch.log(torch.div(pos + 1, every, rounding_mode='floor').float() + 1.0)
    assert float(temp[3]) > 1.0 and float(temp[2]) == 1.0     # position 7 is the first with a whole step behind it
    xb = proj[:, :nq + nk + nv] + bias
    q_ref = O.rms_norm(xb[:, :nq].view(T, H, d), qg, eps) * temp[:, None, None]
    k_ref = O.rms_norm(xb[:, nq:nq + nk].view(T, G, d), kg, eps)
    v_ref = xb[:, nq + nk:].view(T, G, dv)
    tol = 1e-5 if dtype == F32 else 3e-2
    assert (q.float().cpu().view(T, H, d) - q_ref).abs().max() < tol
    for t in range(T):
        pg, off = int(bt[0, int(pos[t]) // 64]), int(pos[t]) % 64
        assert (kp[pg, :, off].float().cpu() - k_ref[t]).abs().max() < tol and (vp[pg, :, off].float().cpu() - v_ref[t]).abs().max() < tol


@pytest.mark.parametrize('shape', [(2, 24, 40), (1, 7, 5), (3, 20, 64), (3, 64, 64), (2, 128, 96), (1, 200, 33), (5, 136, 70), (1, 300, 40)])
@pytest.mark.parametrize('tau,rs', [(12.0, 0), (1.0, 0), (4.0, 2), (4.0, 4), (4.0, 8)])
def test_gla_scan_in_portions_and_with_decays_at_both_ends(lib, shape, tau, rs):
    """the recurrence alone: whole sequences against the token loop of the oracle, then the same sequences in portions (the state
    rows carry on) with a second sequence in the batch, bit for bit equal to the whole run. Decay logits reach far to both sides:
    channels that forget at once and channels that keep everything for the whole sequence. rs: the shape of a warp (0: the
    launch's own choice)"""
    configs, weights, engine, danalorn, paged, O = _mods()
    from phi3_b200._lib import GlaArgs, call_struct, call, ptr
    dev = torch.device('cuda')
    H, d, dv = shape
    g = torch.Generator().manual_seed(7)
    T = {0: 83, 1: 37}
    cols = 2 * H * d + 2 * H * dv
    off = dict(q=0, k=H * d, v=2 * H * d, g=2 * H * d + H * dv)
    proj = {s: torch.randn(n, cols, generator=g) for s, n in T.items()}
    z = {s: torch.randn(n, H * d, generator=g) * 4.0 for s, n in T.items()}
    for s in z:
        z[s][20:24] = -60.0                                    # every channel forgets all it held ...
        z[s][24:30, ::2] = 40.0                                # ... then half of them keep everything
    zb, gain = torch.randn(H * d, generator=g), torch.rand(dv, generator=g) + 0.5
    eye = lambda n: torch.eye(n, dtype=torch.float64)
    ref = {}
    for s in proj:       # the oracle's mixer with identity projections: its input is [proj | z], the decay projection passes z through
        n_in = cols + H * d
        pw = {'p.q': eye(n_in)[off['q']:off['k']], 'p.k': eye(n_in)[off['k']:off['v']], 'p.v': eye(n_in)[off['v']:off['g']],
              'p.g': eye(n_in)[off['g']:cols], 'p.a1': eye(n_in)[cols:], 'p.a2': eye(H * d), 'p.a2.b': zb.double(),
              'p.norm': gain.double(), 'p.o': eye(H * dv)}
        ref[s] = O.gated_linear_attention(torch.cat([proj[s], z[s]], 1).double(), pw, 'p.', dict(heads=H, dim=d, vdim=dv, tau=tau), 1e-6)
    n_state = int(lib.lib().p3_gla_state_floats(H, d, dv))
    assert n_state == H * d * dv

    def run(plans):
        state = torch.full((3, n_state), float('nan'), device=dev)
        got = {s: [] for s in T}
        for plan in plans:
            seqs, rows, zrows = [], [], []
            r0 = 0
            for slot, p0, n in plan:
                seqs.append((r0, n, slot, p0))
                rows.append(proj[slot - 1][p0:p0 + n])
                zrows.append(z[slot - 1][p0:p0 + n])
                r0 += n
            pd, zd = torch.cat(rows, 0).to(dev), torch.cat(zrows, 0).to(dev)
            y, out = torch.empty(r0, H * dv, device=dev), torch.empty(r0, H * dv, device=dev)
            sq = torch.tensor(seqs, dtype=torch.int32, device=dev).reshape(-1)
            zbd, gd = zb.to(dev), gain.to(dev)
            a = GlaArgs()
            a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off = ptr(pd), cols, off['q'], off['k'], off['v']
            a.z, a.ld_z, a.z_bias, a.inv_tau = ptr(zd), H * d, ptr(zbd), 1.0 / tau
            a.n_heads, a.dim, a.vdim, a.q_scale = H, d, dv, d ** -0.5
            a.state, a.seqs, a.n_seqs, a.out, a.ld_out, a.rs_force, a.n_rows = ptr(state), ptr(sq), len(seqs), ptr(y), H * dv, rs, r0
            call_struct('p3_gla_scan', a, 0)
            call('p3_headnorm_gate_x', ptr(y), H * dv, None, H, dv, ptr(gd), 1, ptr(pd[:, off['g']:]), cols, 1, 1.0, 1e-6, ptr(out),
                 H * dv, 1, r0, 0)
            torch.cuda.synchronize()
            o = 0
            for slot, p0, n in plan:
                got[slot - 1].append(out[o:o + n].cpu())
                o += n
        return {s: torch.cat(v, 0) for s, v in got.items()}

    whole = run([[(1, 0, 83), (2, 0, 37)]])                    # sequence s lives in slot s + 1
    if rs == 0:
        # the same logits as a low-rank product formed by the scan's first launch: z = a2 lr, with a2 = [I | 0] and lr = [z | junk]
        if H * d <= 64:
            lr_all = {s_: torch.cat([z[s_], torch.randn(T[s_], 3, generator=g)], 1) for s_ in T}
            a2m = torch.cat([torch.eye(H * d), torch.zeros(H * d, 3)], 1)
            state = torch.full((3, n_state), float('nan'), device=dev)
            for s_ in T:
                n = T[s_]
                pd, ld_, a2d = proj[s_].to(dev), lr_all[s_].to(dev), a2m.to(dev)
                zd = torch.full((n, H * d), float('nan'), device=dev)
                y, out = torch.empty(n, H * dv, device=dev), torch.empty(n, H * dv, device=dev)
                sq = torch.tensor([(0, n, s_ + 1, 0)], dtype=torch.int32, device=dev).reshape(-1)
                zbd, gd = zb.to(dev), gain.to(dev)
                a = GlaArgs()
                a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off = ptr(pd), cols, off['q'], off['k'], off['v']
                a.z, a.ld_z, a.z_bias, a.inv_tau = ptr(zd), H * d, ptr(zbd), 1.0 / tau
                a.lr, a.ld_lr, a.a2, a.rank = ptr(ld_), ld_.shape[1], ptr(a2d), a2m.shape[1]
                a.n_heads, a.dim, a.vdim, a.q_scale = H, d, dv, d ** -0.5
                a.state, a.seqs, a.n_seqs, a.out, a.ld_out, a.n_rows = ptr(state), ptr(sq), 1, ptr(y), H * dv, n
                call_struct('p3_gla_scan', a, 0)
                call('p3_headnorm_gate_x', ptr(y), H * dv, None, H, dv, ptr(gd), 1, ptr(pd[:, off['g']:]), cols, 1, 1.0, 1e-6, ptr(out),
                     H * dv, 1, n, 0)
                torch.cuda.synchronize()
                assert (out.cpu().double() - ref[s_]).abs().max() < 2e-4 * max(1.0, float(ref[s_].abs().max())), s_
    parts = run([[(1, 0, 17)], [(2, 0, 2), (1, 17, 1)], [(1, 18, 16), (2, 2, 33)], [(1, 34, 1)], [(2, 35, 2), (1, 35, 48)]])
    for s in T:
        scale = float(ref[s].abs().max())
        assert (whole[s].double() - ref[s]).abs().max() < 2e-4 * max(1.0, scale), s
        assert torch.equal(whole[s], parts[s]), s


def test_linear_distance_table_and_head_norm_choices(lib):
    from phi3_b200._lib import call, ptr
    dev = torch.device('cuda')
    slope = torch.tensor([2.0 ** (-8.0 * (h + 1) / 3) for h in range(3)], dtype=torch.float64).float()
    pen = torch.empty(3, 500, device=dev)
    sd = slope.to(dev)
    call('p3_distance_linear_table', ptr(sd), ptr(pen), 3, 500, 0)
    torch.cuda.synchronize()
    assert torch.equal(pen.cpu(), slope[:, None] * torch.arange(500, dtype=torch.float32)[None, :])
    g = torch.Generator().manual_seed(1)
    T, H, dv = 9, 3, 20
    y, gate, gain = torch.randn(T, H * dv, generator=g), torch.randn(T, H * dv, generator=g), torch.rand(dv, generator=g) + 0.5
    yd, gd, nd = y.to(dev), gate.to(dev), gain.to(dev)
    out = torch.empty(T, H * dv, device=dev)
    unit = y.view(T, H, dv) / torch.sqrt((y.view(T, H, dv) ** 2).mean(-1, keepdim=True) + 1e-6) * gain
    for silu in (0, 1):
        call('p3_headnorm_gate_x', ptr(yd), H * dv, None, H, dv, ptr(nd), 1, ptr(gd), H * dv, silu, 1.0, 1e-6, ptr(out), H * dv, 1, T, 0)
        torch.cuda.synchronize()
        want = unit.reshape(T, H * dv) * (torch.nn.functional.silu(gate) if silu else torch.sigmoid(gate))
        assert (out.cpu() - want).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------ entry points
def test_greedy_generation_through_load_generate_and_the_scheduler(lib, tmp_path):
    configs, weights, engine, danalorn, paged, O = _mods()
    from phi3_b200 import api
    from safetensors.torch import save_file
    cfg = configs.tiny_danalorn()
    w = weights.random_danalorn_weights(cfg, 13)
    json.dump(cfg, open(tmp_path / 'config.json', 'w'))
    save_file(w, str(tmp_path / 'model.safetensors'))
    model, proc = api.load(model_path=str(tmp_path), dtype=F32)
    assert type(model).__name__ == 'DanalornB200'
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
    configs, weights, engine, danalorn, paged, O = _mods()
    from safetensors.torch import save_file
    import numpy as np
    cfg = configs.tiny_danalorn()
    w = weights.random_danalorn_weights(cfg, 14)
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
