"""Danalorn on B200: a decoder-only language model with an RMS norm before AND after every sublayer,
x <- x + N(mixer(N(x))), x <- x + N(ff(N(x))), an fp32 residual stream, and an embedding that adds the row of a hashed
(previous token, current token) pair to the scaled token row. Three kinds of mixers, in any order:

  'latent_attention'  latent-vector attention: the queries pass a normed low-rank vector, a token caches one normed latent vector
                      and one rotated key part that all heads share, neighbouring numbers rotate as pairs, a sliding window, a
                      learned per-head sink in the softmax denominator. A layer with `kv_from` has no latent projection: it reads
                      the cache rows another layer wrote in the same step, through up-projections of its own;
  'attention'         grouped-query attention with projection biases, per-head query/key RMS norm, no rotation, queries that grow
                      with the logarithm of the position, a linear distance bias per head, one added to the softmax denominator
                      and an element-wise sigmoid gate on the head outputs;
  'gla'               gated linear attention: a matrix state per head with one decay per key channel and token (low-rank
                      projection), read out by the query, normed per head and gated by silu.
Feed-forwards are relu^2 units.

The model owns weights and launches kernels; it has no cache, no state and no loop of its own. `forward(batch, pool)` runs ONE step
of the engine (engine.py): a ragged batch of new tokens of several sequences against the shared page pool (paged.py), which also
holds, per sequence slot, the state of the recurrent parts: the last token (for the pair embedding) and the matrix states.

Latent attention runs in the latent space, as for Tapalix: the key up-projection is folded into the query (one batched product per
layer), attention reads the cache rows as ONE shared key/value head (key = the whole row, value = its leading kv_rank numbers) and the
value up-projection is applied to the attention output.

Kernels per layer (csrc/): p3_embed_pair_rows_f32 -> p3_postnorm_prenorm ->
  latent:    ONE product [query down | latent down] -> p3_latent_post (norms, rotation of the shared key part, cache write) -> query
             up product -> p3_latent_post (rotation of the query parts) -> per-head query absorption -> p3_attn_window_prefill /
             _decode (window, sink) -> per-head value up-projection -> output product
  attention: ONE product [q | k | v | gate] -> p3_qkv_post (biases, head norms, query temperature, paged K/V write) ->
             p3_attn_window_prefill / _decode (distance table, unit sink, element-wise gate in the epilogue) -> output product
  gla:       ONE product [q | k | v | gate | decay down] -> p3_gla_scan (decay up-projection, bias and decays in one pass, then the
             scan) -> p3_headnorm_gate_x -> output product
-> p3_postnorm_prenorm -> up product -> p3_relu2 -> down product -> p3_postnorm_prenorm.

Precision. dtype=bfloat16 (serving): matrices, activations that feed a matrix product and the caches are bf16, accumulation is fp32;
positions, angles, scores, softmax, norms, the residual sum, decays and their logarithms, the recurrent state and its sums are fp32.
dtype=float32: everything is fp32 on the FMA pipes (no TF32).
"""
import ctypes as C
import os

import torch
from . import _lib
from ._lib import call, call_struct, ptr
from .configs import DanalornConfig
from .lm_base import PagedLM, _page_slices, _stream


class DanalornB200(PagedLM):
    arch = 'Danalorn'

    def __init__(self, cfg, weights, device='cuda', dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError('DanalornB200 needs a CUDA device (sm_100a); there is no CPU fallback')
        _lib.lib()
        if isinstance(cfg, dict):
            cfg = DanalornConfig(cfg)
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError('dtype must be torch.bfloat16 or torch.float32')
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.W, self.V, self.eps = cfg.width, cfg.vocab_size, cfg.eps
        self._init_products()
        w, W = weights, self.W
        mat = lambda t: t.to(self.dev, dtype).contiguous()                     # matrices: the compute type
        f32 = lambda t: t.to(self.dev, torch.float32).contiguous()            # everything that enters fp32 arithmetic
        b16 = lambda t: t.to(self.dev, torch.bfloat16).contiguous()

        def rows16(parts):
            """stacked projection rows, padded with zero rows to a multiple of 16 (small batches keep the weight-streaming kernel)"""
            n = sum(p.shape[0] for p in parts)
            return mat(torch.cat(parts + ([torch.zeros(-n % 16, parts[0].shape[1], dtype=parts[0].dtype, device=parts[0].device)] if n % 16 else []), 0))

        def expect(name, shape):
            if name not in w:
                raise KeyError(f'the checkpoint has no tensor {name!r}')
            if tuple(w[name].shape) != tuple(shape):
                raise ValueError(f'{name}: shape {tuple(w[name].shape)}, the config gives {tuple(shape)}')

        expect('embed', (self.V, W)); expect('head', (self.V, W))
        self.embed = b16(w['embed'])                                           # bf16 values are exact in both modes
        self.pair_table = None
        if cfg.bigram is not None:
            expect('bigram', (cfg.bigram.buckets + 1, W))
            self.pair_table = b16(w['bigram'])
        self.final_gain, self.head = f32(w['final.norm']), mat(w['head'])
        self.layers = []
        self._state_layout = [1]                                               # buffer 0: the last token of the sequence (an int32)
        for i, lc in enumerate(cfg.layers):
            p, m, f = f'l{i}.', lc.mixer, lc.ff
            a = p + 'mix.'
            L = dict(cfg=lc, pre1=f32(w[p + 'norm1']), post1=f32(w[p + 'norm1b']))
            if m.kind == 'latent_attention':
                H, d, dr, dv, R, Q = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
                if R + dr > 4096:
                    raise NotImplementedError(f'layer {i}: a cache row of kv_rank + rot_dim = {R + dr} numbers; the attention kernels '
                                              'take at most 4096')
                expect(a + 'dq', (Q, W)); expect(a + 'uq', (H * (d + dr), Q)); expect(a + 'uk', (H * d, R)); expect(a + 'uv', (H * dv, R))
                expect(a + 'o', (W, H * dv)); expect(a + 'sink', (H,))
                parts = [w[a + 'dq']]
                L['own_cache'] = m.kv_from is None
                L['cache_layer'] = i if m.kv_from is None else m.kv_from
                if L['own_cache']:
                    expect(a + 'dkv', (R + dr, W))
                    parts.append(w[a + 'dkv'])
                    L['c_gain'] = f32(w[a + 'dkv.norm'])
                L['in_w'] = rows16(parts)
                L['cq_gain'], L['uq'] = f32(w[a + 'dq.norm']), mat(w[a + 'uq'])
                # the key up-projection is folded into the query: per head [kv_rank, dim]; the value up-projection stays [vdim, kv_rank]
                L['uk_t'] = mat(w[a + 'uk'].view(H, d, R).transpose(1, 2))
                L['uv'], L['out_w'], L['sink'] = mat(w[a + 'uv']), mat(w[a + 'o']), f32(w[a + 'sink'])
                if m.rot is not None:
                    fr = [m.rot.base ** (-2.0 * k / m.rot.dims) for k in range(m.rot.dims // 2)]
                    L['freq'], L['rot_n'] = torch.tensor(fr, dtype=torch.float64).to(self.dev, torch.float32), m.rot.dims
                else:
                    L['freq'], L['rot_n'] = None, 0
                L['tile_rows'] = self._attention_tile_rows(H, 1, R + dr, R, R + dr)
            elif m.kind == 'attention':
                H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
                expect(a + 'q', (H * d, W)); expect(a + 'k', (G * d, W)); expect(a + 'v', (G * dv, W)); expect(a + 'g', (H * dv, W))
                expect(a + 'o', (W, H * dv)); expect(a + 'q.norm', (d,)); expect(a + 'k.norm', (d,))
                L['in_w'] = rows16([w[a + 'q'], w[a + 'k'], w[a + 'v'], w[a + 'g']])
                L['in_b'] = torch.cat([f32(w[a + 'q.b']), f32(w[a + 'k.b']), f32(w[a + 'v.b'])])
                L['q_gain'], L['k_gain'], L['out_w'] = f32(w[a + 'q.norm']), f32(w[a + 'k.norm']), mat(w[a + 'o'])
                L['slope'] = torch.tensor(cfg.slopes(H), dtype=torch.float64).to(self.dev, torch.float32)
                L['sink'] = torch.zeros(H, dtype=torch.float32, device=self.dev)           # exp(0) = the one in the denominator
                L['pen'] = None
                L['tile_rows'] = self._attention_tile_rows(H, G, d, dv, 0)
            else:
                H, d, dv = m.heads, m.dim, m.vdim
                expect(a + 'q', (H * d, W)); expect(a + 'k', (H * d, W)); expect(a + 'v', (H * dv, W)); expect(a + 'g', (H * dv, W))
                expect(a + 'o', (W, H * dv)); expect(a + 'norm', (dv,)); expect(a + 'a2.b', (H * d,))
                r = w[a + 'a1'].shape[0]                                       # rank of the decay projection: the tensors give it
                expect(a + 'a1', (r, W)); expect(a + 'a2', (H * d, r))
                # decay ranks up to 64: the down projection's rows ride in the layer's input product and the scan's first launch forms
                # the logits from them (fp32); above that the two decay projections are products of their own
                L['rank'], L['fused_decay'] = r, r <= 64 and os.environ.get('P3_GLA_FUSED_DECAY', '1') != '0'
                L['in_w'] = rows16([w[a + 'q'], w[a + 'k'], w[a + 'v'], w[a + 'g']] + ([w[a + 'a1']] if L['fused_decay'] else []))
                if L['fused_decay']:
                    L['a2_32'] = f32(w[a + 'a2'])
                else:
                    L['a1'], L['a2'] = mat(w[a + 'a1']), mat(w[a + 'a2'])
                L['a2_b'], L['gain'], L['out_w'] = f32(w[a + 'a2.b']), f32(w[a + 'norm']), mat(w[a + 'o'])
                L['state'] = len(self._state_layout)
                self._state_layout.append(int(_lib.lib().p3_gla_state_floats(H, d, dv)))
                L['tile_rows'] = 64
            if f is not None:
                q = p + 'mlp.'
                expect(q + 'up', (f.ff, W)); expect(q + 'down', (W, f.ff))
                L['pre2'], L['post2'] = f32(w[p + 'norm2']), f32(w[p + 'norm2b'])
                L['up'], L['down'] = mat(w[q + 'up']), mat(w[q + 'down'])
            self.layers.append(L)
        # query rows per attention tile the engine cuts prompt portions into: 64 when every attention takes the tensor-core prefill
        # kernel (csrc/attention_window.cu), else 32
        self.q_tile = min(L['tile_rows'] for L in self.layers)
        self._pen_len = 0

    def _attention_tile_rows(self, H, G, key, val, v_ld):
        """query rows per prefill tile that the attention launch takes for these sizes (64: its tensor-core kernels); asked of the
        library itself so that the engine's tiles and the kernel's choice cannot disagree"""
        a = _lib.AttnWindowArgs()
        a.q = a.out = a.k_pool = a.v_pool = a.block_table = a.tiles = 256              # aligned stand-ins: nothing is launched
        a.ld_q, a.ld_out, a.n_heads, a.n_kv, a.dim, a.vdim, a.v_ld = H * key, H * val, H, G, key, val, v_ld
        a.act_f32 = a.cache_f32 = self.f32
        return int(_lib.lib().p3_attn_window_tile_rows(C.byref(a)))

    # ------------------------------------------------------------------ what the engine asks of a model
    def kv_layout(self):
        return self.cfg.kv_layout()

    def state_layout(self):
        """fp32 numbers per sequence slot and state buffer: one for the sequence's last token (kept as an int32 in that place),
        then one matrix state per recurrent layer (L['state'] indexes the pool's state buffers)"""
        return list(self._state_layout)

    def prepare(self, max_context):
        """tables of the linear distance bias, slope_h * distance, for every distance a query can see (the attention mixers have no
        window: up to the longest sequence the pool can hold)"""
        if max_context <= self._pen_len:
            return
        for L in self.layers:
            m = L['cfg'].mixer
            if m.kind != 'attention':
                continue
            n = max(int(max_context), 1)
            L['pen'] = torch.empty((m.heads, n), dtype=torch.float32, device=self.dev)
            call('p3_distance_linear_table', ptr(L['slope']), ptr(L['pen']), m.heads, n, _stream())
        self._pen_len = max_context

    def graph_safe(self, b):
        """may this step be captured as a CUDA graph? Always: no kernel of this design needs a host read."""
        return True

    # ------------------------------------------------------------------ one engine step
    def _norms(self, y, post, x, pre, T):
        """x += N(y) * post (y None: x stays); -> N(x) * pre in the activation type (None without pre)"""
        h = torch.empty((T, self.W), dtype=self.dtype, device=self.dev) if pre is not None else None
        nb = T * self.W * ((12 if y is not None else 4) + (0 if pre is None else (4 if self.f32 else 2)))
        self.rows('norm', nb, 'p3_postnorm_prenorm', ptr(y), y.stride(0) if y is not None else 0, None, ptr(post), ptr(x),
                  ptr(pre), ptr(h) if self.f32 else None, None if self.f32 else ptr(h), self.f32, T, self.W, self.eps, _stream())
        return h

    def forward(self, b, pool, trace=None):
        """b: StepBatch, pool: paged.PagePool -> fp32 logits [b.R, vocab] (None when no row is wanted).
        `trace` (a list) receives a copy of the residual stream after every layer."""
        st, dev, T, W, cfg = _stream(), self.dev, b.T, self.W, self.cfg
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        x = e(T, W)
        bg = cfg.bigram
        self.rows('embed', T * W * 8, 'p3_embed_pair_rows_f32', ptr(self.embed), ptr(self.pair_table), ptr(b.ids), ptr(b.seqs),
                  ptr(b.slot_seq), ptr(b.tok_slot), ptr(pool.state[0]), pool.state[0].stride(0), ptr(x), T, W, self.V, cfg.embed_scale,
                  bg.buckets if bg else 1, bg.mul_prev if bg else 0, bg.mul_cur if bg else 0, st)
        h = self._norms(None, None, x, self.layers[0]['pre1'], T)
        for li, L in enumerate(self.layers):
            m, f = L['cfg'].mixer, L['cfg'].ff
            nxt_pre = self.layers[li + 1]['pre1'] if li + 1 < len(self.layers) else None
            y = {'latent_attention': self._latent, 'attention': self._attention, 'gla': self._gla}[m.kind](L, li, h, b, pool)
            if f is None:
                h = self._norms(y, L['post1'], x, nxt_pre, T)
            else:
                h2 = self._norms(y, L['post1'], x, L['pre2'], T)
                h = self._norms(self._dense(L, f, h2, T), L['post2'], x, nxt_pre, T)
            if trace is not None:
                trace.append(x.clone())
        if not b.R:
            return None
        xn = e(b.R, W, dt=self.dtype)
        call('p3_rmsnorm_rows_f32', ptr(x), ptr(b.want_rows), ptr(self.final_gain), ptr(xn), self.f32, b.R, W, self.eps, st)
        logits = e(b.R, self.V)
        self.linear(xn, self.head, logits)
        return logits

    def _attend(self, w, L, b, G, key, val, span_of, kv_bytes):
        """the prefill tiles and the single-token requests of the step through p3_attn_window_*; span_of(n) = keys a query at
        position n - 1 sees"""
        st, H = _stream(), w.n_heads
        esz = 4 if self.f32 else 2
        if b.n_pf:
            w.tiles, w.n_tiles = ptr(b.pf_tiles), b.n_pf
            ev = self._ev()
            call_struct('p3_attn_window_prefill', w, st)
            span = span_of(b.max_pos + 1) if w.window else (b.max_pos + 1) // 2
            self._ev(ev, 'attn_prefill', 2 * (b.T - b.n_dec) * H * span * (key + val), 0)
        if b.n_dec:
            w.tiles, w.n_tiles = ptr(b.dec_tiles), b.n_dec
            span = span_of(b.max_pos + 1)
            if L['tile_rows'] == 64:
                if G == 1 and H > 1:
                    # one shared K/V head: a request is one CTA per slice (two when the values take two column blocks)
                    w.n_splits = _page_slices(b.n_dec * (-(-val // 128) if key > 128 else 1), 2 * -(-span // 128) + 1, merge=0.4)
                else:
                    w.n_splits = _page_slices(b.n_dec * G, 2 * -(-span // 128) + 1)
            else:
                # one key per lane: enough CTAs for eight per SM, at least 128 keys (one pass of a CTA) per slice
                w.n_splits = max(1, min(-(-8 * 148 // (b.n_dec * G)), -(-span // 128)))
            ws = torch.empty(b.n_dec * H * w.n_splits * (val + 2), dtype=torch.float32, device=self.dev) if w.n_splits > 1 else None
            w.ws = ptr(ws)
            ev = self._ev()
            call_struct('p3_attn_window_decode', w, st)
            self._ev(ev, 'attn_decode', 2 * b.n_dec * H * span * (key + val), b.n_dec * span * kv_bytes * esz)

    def _latent(self, L, li, h, b, pool):
        """normed input h (act [T, W]) -> mixer output before its norm, fp32 [T, W]"""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        m = L['cfg'].mixer
        H, d, dr, dv, R, Q = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
        key = R + dr
        cache = pool.k[L['cache_layer']]
        proj = e(T, L['in_w'].shape[0])
        self.linear(h, L['in_w'], proj, nxt=L['uq'])
        cq = e(T, Q, dt=act)
        a = _lib.LatentPostArgs()
        a.proj, a.ld_proj, a.c_off = ptr(proj), proj.stride(0), Q
        a.n_heads, a.dim, a.rot_dim, a.kv_rank, a.rot_n, a.pair_mode = 0, d, dr, R, L['rot_n'], 1
        a.eps, a.freq, a.rot_mag = self.eps, ptr(L['freq']), 1.0
        a.cq_off, a.q_rank, a.cq_gain, a.cq_out, a.ld_cq = 0, Q, ptr(L['cq_gain']), ptr(cq), cq.stride(0)
        if L['own_cache']:
            a.cache, a.c_gain = ptr(cache), ptr(L['c_gain'])
        a.block_table, a.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
        esz = 4 if self.f32 else 2
        self.rows('latent_post', T * ((Q + (key if L['own_cache'] else 0)) * (4 + esz)), 'p3_latent_post', a)
        qf = e(T, H * (d + dr))
        self.linear(cq, L['uq'], qf, nxt=L['out_w'])
        qp, ql, olat = e(T, H * d, dt=act), e(T, H * key, dt=act), e(T, H * R, dt=act)
        a2 = _lib.LatentPostArgs()
        a2.q_src, a2.ld_qsrc = ptr(qf), qf.stride(0)
        a2.n_heads, a2.dim, a2.rot_dim, a2.kv_rank, a2.rot_n, a2.pair_mode = H, d, dr, R, L['rot_n'], 1
        a2.eps, a2.freq, a2.rot_mag = self.eps, ptr(L['freq']), 1.0
        a2.q_plain, a2.ld_qp, a2.q_lat, a2.ld_ql = ptr(qp), qp.stride(0), ptr(ql), ql.stride(0)
        a2.block_table, a2.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        a2.tok_slot, a2.tok_pos, a2.T, a2.act_f32, a2.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
        self.rows('latent_post', T * H * (d + dr) * (4 + esz), 'p3_latent_post', a2)
        # queries into the latent space: ql[:, h, :R] = U_h^T q_h
        ev = self._ev()
        self.gemm_any(qp, L['uk_t'], ql, N=R, K=d, ldw=d, batch=(H, d, R * d, key))
        self._ev(ev, 'head_gemm', 2 * T * H * R * d, L['uk_t'].numel() * L['uk_t'].element_size())
        w = _lib.AttnWindowArgs()
        w.q, w.ld_q, w.k_pool, w.v_pool, w.v_ld = ptr(ql), ql.stride(0), ptr(cache), ptr(cache), key
        w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        w.out, w.ld_out, w.sink = ptr(olat), olat.stride(0), ptr(L['sink'])
        w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window = H, 1, key, R, m.scale, m.window
        w.act_f32, w.cache_f32 = self.f32, self.f32
        self._attend(w, L, b, 1, key, R, (lambda n: min(m.window, n)) if m.window else (lambda n: n), key)
        # values out of the latent space: hid[:, h, :] = V_h olat[:, h, :]
        hid = e(T, H * dv, dt=act)
        ev = self._ev()
        self.gemm_any(olat, L['uv'], hid, N=dv, K=R, ldw=R, batch=(H, R, dv * R, dv))
        self._ev(ev, 'head_gemm', 2 * T * H * R * dv, L['uv'].numel() * L['uv'].element_size())
        y = e(T, W)
        self.linear(hid, L['out_w'], y, nxt=L.get('up'))
        return y

    def _attention(self, L, li, h, b, pool):
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        m = L['cfg'].mixer
        H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
        nq, nk, nv = H * d, G * d, G * dv
        proj = e(T, L['in_w'].shape[0])
        self.linear(h, L['in_w'], proj, nxt=L['out_w'])
        q, att = e(T, nq, dt=act), e(T, H * dv, dt=act)
        a = _lib.QkvPostArgs()
        a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.g_off = ptr(proj), proj.stride(0), 0, nq, nq + nk, nq + nk + nv
        a.n_heads, a.n_kv, a.dim, a.vdim = H, G, d, dv
        a.q_gain, a.k_gain, a.eps, a.bias = ptr(L['q_gain']), ptr(L['k_gain']), self.eps, ptr(L['in_b'])
        a.q_temp_coef, a.q_temp_every = m.q_temp_coef, m.q_temp_every
        a.q_out, a.ld_q = ptr(q), q.stride(0)
        a.k_pool, a.v_pool = ptr(pool.k[li]), ptr(pool.v[li])
        a.block_table, a.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
        esz = 4 if self.f32 else 2
        self.rows('qkv_post', T * (nq + nk + nv) * (4 + esz), 'p3_qkv_post', a)
        w = _lib.AttnWindowArgs()
        w.q, w.ld_q, w.k_pool, w.v_pool = ptr(q), q.stride(0), ptr(pool.k[li]), ptr(pool.v[li])
        w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        w.sink, w.penalty, w.n_penalty = ptr(L['sink']), ptr(L['pen']), L['pen'].shape[1]
        w.elem_gate, w.ld_elem_gate = ptr(proj[:, nq + nk + nv:]), proj.stride(0)
        w.out, w.ld_out = ptr(att), att.stride(0)
        w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window = H, G, d, dv, m.scale, 0
        w.act_f32, w.cache_f32 = self.f32, self.f32
        self._attend(w, L, b, G, d, dv, lambda n: n, G * (d + dv))
        y = e(T, W)
        self.linear(att, L['out_w'], y, nxt=L.get('up'))
        return y

    def _gla(self, L, li, h, b, pool):
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        m = L['cfg'].mixer
        H, d, dv = m.heads, m.dim, m.vdim
        proj = e(T, L['in_w'].shape[0])
        self.linear(h, L['in_w'], proj, nxt=L['out_w'])
        z = e(T, H * d)                                       # decay logits, then decays
        y = e(T, H * dv)
        r = _lib.GlaArgs()
        if L['fused_decay']:
            lr = proj[:, 2 * H * d + 2 * H * dv:]
            r.lr, r.ld_lr, r.a2, r.rank = ptr(lr), proj.stride(0), ptr(L['a2_32']), L['rank']
        else:
            lr = e(T, L['rank'], dt=act)
            self.linear(h, L['a1'], lr)
            self.linear(lr, L['a2'], z)
        r.proj, r.ld_proj, r.q_off, r.k_off, r.v_off = ptr(proj), proj.stride(0), 0, H * d, 2 * H * d
        r.z, r.ld_z, r.z_bias, r.inv_tau = ptr(z), z.stride(0), ptr(L['a2_b']), 1.0 / m.tau
        r.n_heads, r.dim, r.vdim, r.q_scale = H, d, dv, d ** -0.5
        r.state, r.seqs, r.n_seqs = ptr(pool.state[L['state']]), ptr(b.seqs), b.n_seq
        r.out, r.ld_out, r.n_rows = ptr(y), y.stride(0), T
        ev = self._ev()
        call_struct('p3_gla_scan', r, st)
        self._ev(ev, 'gla_scan', 4 * T * H * d * dv, T * (3 * H * d + 2 * H * dv) * 4)
        cat = e(T, H * dv, dt=act)
        g_off = 2 * H * d + H * dv
        esz = 4 if self.f32 else 2
        self.rows('headnorm', T * H * dv * (8 + esz), 'p3_headnorm_gate_x', ptr(y), y.stride(0), None, H, dv, ptr(L['gain']), 1,
                  ptr(proj[:, g_off:]), proj.stride(0), 1, 1.0, self.eps, ptr(cat), cat.stride(0), self.f32, T, st)
        out = e(T, W)
        self.linear(cat, L['out_w'], out, nxt=L.get('up'))
        return out

    def _dense(self, L, f, h, T):
        st = _stream()
        up = torch.empty((T, f.ff), dtype=torch.float32, device=self.dev)
        hid = torch.empty((T, f.ff), dtype=self.dtype, device=self.dev)
        y = torch.empty((T, self.W), dtype=torch.float32, device=self.dev)
        self.linear(h, L['up'], up, nxt=L['down'])
        self.rows('activation', T * f.ff * (4 + (4 if self.f32 else 2)), 'p3_relu2', ptr(up), up.stride(0), None, 0, ptr(hid),
                  hid.stride(0), self.f32, T, f.ff, st)
        self.linear(hid, L['down'], y)
        return y
