"""Tagenex on B200: a decoder-only language model whose layers put the RMS norm on each sublayer's OUTPUT
(x <- x + N1(mixer(x)), x <- x + N2(ff(x))), with an fp32 residual stream, and whose mixer is grouped-query attention with
per-head query/key RMS norm, no rotation, a logarithmic distance penalty, a sliding window, a sink in the softmax denominator,
value mixing with the first mixing layer's values and a per-head sigmoid output gate. Feed-forwards are a clamped gated-linear
unit with biases, or a top-k mixture of such units without biases.

The model owns weights and launches kernels; it has no cache and no loop of its own. `forward(batch, pool)` runs ONE step of the
engine (engine.py): a ragged batch of new tokens of several sequences against the shared page pool (paged.py), logits only for
the rows the caller wants. Prompt portions and single decoded tokens share the step; only the attention launch differs
(32-row tiles vs one CTA per request and K/V head).

Kernels per layer (csrc/): fused q|k|v|gate projection (one GEMM) -> p3_qkv_post (head norms, value mixing, gate sigmoid, paged
K/V write) -> p3_attn_window_prefill / _decode (window, sink, penalty table, gate in the epilogue) -> output projection ->
p3_postnorm_residual (norm of the sublayer output + residual add + activation copy) -> gate|up GEMM (+bias) -> p3_glu_clamped ->
down GEMM (+bias) -> p3_postnorm_residual; mixture layers: p3_router_topk -> p3_moe_sort -> grouped gate|up GEMM over gathered
rows -> p3_glu_clamped -> grouped down GEMM -> p3_moe_combine.

Precision. dtype=bfloat16 (serving): matrices, activations that feed a matrix product and the cache are bf16, accumulation is
fp32; positions, penalties, scores, softmax, norms, router, gates, value mixing and the residual sum are fp32. dtype=float32:
everything is fp32 on the FMA pipes (no TF32). Dense bf16 products with K % 8 == 0 run on the tcgen05 GEMM (p3_gemm), everything
else on p3_gemm_any.
"""
import torch
from . import _lib
from ._lib import call, call_struct, ptr
from .lm_base import PagedLM, StepBatch, _page_slices, _stream  # noqa: F401  (StepBatch is re-exported for engine.py)
from .configs import TagenexConfig
from .paged import PAGE


class TagenexB200(PagedLM):
    arch = 'Tagenex'

    def __init__(self, cfg, weights, device='cuda', dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError('TagenexB200 needs a CUDA device (sm_100a); there is no CPU fallback')
        _lib.lib()
        if isinstance(cfg, dict):
            cfg = TagenexConfig(cfg)
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError('dtype must be torch.bfloat16 or torch.float32')
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.W, self.V, self.eps = cfg.width, cfg.vocab_size, cfg.eps
        self._init_products()
        w = weights
        mat = lambda t: t.to(self.dev, dtype).contiguous()                     # matrices: the compute type
        f32 = lambda t: t.to(self.dev, torch.float32).contiguous()            # everything that enters fp32 arithmetic
        b16 = lambda t: t.to(self.dev, torch.bfloat16).contiguous()
        self.embed = b16(w['embed'])                                           # bf16 values are exact in both modes
        self.final_gain, self.head = f32(w['final.norm']), mat(w['head'])
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, m = f'l{i}.', lc.mixer
            L = dict(cfg=lc, norm1=f32(w[p + 'norm1']))
            a = p + 'mix.'
            L['qkvg'] = mat(torch.cat([w[a + 'q'], w[a + 'k'], w[a + 'v'], w[a + 'g']], 0))
            L['q_gain'], L['k_gain'] = f32(w[a + 'q.norm']), f32(w[a + 'k.norm'])
            L['r1'], L['r2'], L['sink'] = f32(w[a + 'r1']), f32(w[a + 'r2']), f32(w[a + 'sink'])
            L['lam'] = float(w[a + 'vmix'].float()) if m.v_role == 'mix' else 0.0
            L['o'] = mat(w[a + 'o'])
            L['pen'] = None
            L['mma'] = bool(_lib.ATTN_WINDOW_MMA and not self.f32 and m.dim % 16 == 0 and m.vdim % 8 == 0 and m.dim <= 128 and m.vdim <= 128)
            f = lc.ff
            if f is not None:
                L['norm2'] = f32(w[p + 'norm2'])
                q = p + 'mlp.'
                if f.kind == 'dense':
                    L['gu'] = mat(torch.cat([w[q + 'gate'], w[q + 'up']], 0))
                    L['down'] = mat(w[q + 'down'])
                    L['gu_b32'], L['down_b32'] = f32(torch.cat([w[q + 'gate.b'], w[q + 'up.b']], 0)), f32(w[q + 'down.b'])
                    L['gu_b16'], L['down_b16'] = b16(torch.cat([w[q + 'gate.b'], w[q + 'up.b']], 0)), b16(w[q + 'down.b'])
                else:
                    L['gu'] = mat(torch.stack([torch.cat([w[f'{q}e{e}.gate'], w[f'{q}e{e}.up']], 0) for e in range(f.experts)], 0))
                    L['down'] = mat(torch.stack([w[f'{q}e{e}.down'] for e in range(f.experts)], 0))
                    L['router'], L['router_b'] = f32(w[q + 'router']), f32(w[q + 'router.b'])
            self.layers.append(L)
        self._pen_len = 0
        # query rows per attention tile the engine cuts prompt portions into: 64 when every layer takes the tensor-core prefill
        # kernel (bf16, key size % 16 == 0, value size % 8 == 0, both <= 128; csrc/attention_window.cu), else 32
        self.q_tile = 64 if all(L['mma'] for L in self.layers) else 32

    # ------------------------------------------------------------------ what the engine asks of a model
    def kv_layout(self):
        return self.cfg.kv_layout()

    def prepare(self, max_context):
        """distance-penalty tables r1_h ln(1 + r2_h d) for every distance a query can see: d < window, or < the longest
        sequence the pool can hold when the layer has no window"""
        if max_context <= self._pen_len:
            return
        for L in self.layers:
            m = L['cfg'].mixer
            n = min(m.window, max_context) if m.window > 0 else max_context
            n = max(n, 1)
            if L['pen'] is None or L['pen'].shape[1] < n:
                L['pen'] = torch.empty((m.heads, n), dtype=torch.float32, device=self.dev)
                call('p3_distance_penalty_table', ptr(L['r1']), ptr(L['r2']), ptr(L['pen']), m.heads, n, _stream())
        self._pen_len = max_context

    def graph_safe(self, b):
        """may this step be captured as a CUDA graph? Not when a mixture layer would read its segment offsets back."""
        return not any(l.ff is not None and l.ff.kind == 'moe' and self.experts_dense(l.ff, b.T) for l in self.cfg.layers)

    # ------------------------------------------------------------------ one engine step
    def forward(self, b, pool, trace=None):
        """b: StepBatch, pool: paged.PagePool -> fp32 logits [b.R, vocab] (None when no row is wanted).
        `trace` (a list) receives a copy of the residual stream after every layer."""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        x, xa = e(T, W), e(T, W, dt=act)
        call('p3_embed_rows_f32', ptr(self.embed), ptr(b.ids), ptr(x), ptr(xa), self.f32, T, W, self.V, 1.0, W, st)
        v_first = None
        y = e(T, W)
        for li, L in enumerate(self.layers):
            m = L['cfg'].mixer
            H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
            nq, nk, nv = H * d, G * d, G * dv
            proj = e(T, nq + nk + nv + H)
            self.linear(xa, L['qkvg'], proj, nxt=L['o'])
            q, gate, att = e(T, nq, dt=act), e(T, H), e(T, H * dv, dt=act)
            if m.v_role != 'none' and v_first is None:
                v_first = e(T, nv)
            a = _lib.QkvPostArgs()
            a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.g_off = ptr(proj), proj.stride(0), 0, nq, nq + nk, nq + nk + nv
            a.n_heads, a.n_kv, a.dim, a.vdim = H, G, d, dv
            a.q_gain, a.k_gain, a.eps = ptr(L['q_gain']), ptr(L['k_gain']), self.eps
            a.v_mode = {'none': 0, 'source': 1, 'mix': 2}[m.v_role]
            a.v_first, a.v_lambda = (ptr(v_first) if a.v_mode else None), L['lam']
            a.q_out, a.ld_q, a.gate_out = ptr(q), q.stride(0), ptr(gate)
            a.k_pool, a.v_pool = ptr(pool.k[li]), ptr(pool.v[li])
            a.block_table, a.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
            a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
            self.rows('qkv_post', T * (proj.shape[1] * 4 + (nq + nk + nv) * (4 if self.f32 else 2)), 'p3_qkv_post', a)
            w = _lib.AttnWindowArgs()
            w.q, w.ld_q, w.k_pool, w.v_pool = ptr(q), q.stride(0), ptr(pool.k[li]), ptr(pool.v[li])
            w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
            w.sink, w.penalty, w.n_penalty, w.gate = ptr(L['sink']), ptr(L['pen']), L['pen'].shape[1], ptr(gate)
            w.out, w.ld_out = ptr(att), att.stride(0)
            w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window = H, G, d, dv, m.scale, m.window
            w.act_f32, w.cache_f32 = self.f32, self.f32
            esz = 4 if self.f32 else 2
            if b.n_pf:
                w.tiles, w.n_tiles = ptr(b.pf_tiles), b.n_pf
                ev = self._ev()
                call_struct('p3_attn_window_prefill', w, st)
                span = min(m.window, b.max_pos + 1) if m.window else (b.max_pos + 1) // 2
                self._ev(ev, 'attn_prefill', 2 * (T - b.n_dec) * H * span * (d + dv), 0)
            if b.n_dec:
                w.tiles, w.n_tiles = ptr(b.dec_tiles), b.n_dec
                span = min(m.window, b.max_pos + 1) if m.window else b.max_pos + 1
                if L['mma']:
                    w.n_splits = _page_slices(b.n_dec * G, 2 * -(-span // 128) + 1)
                else:
                    # one key per lane: enough CTAs for eight per SM, at least 128 keys (one pass of a CTA) per slice
                    w.n_splits = max(1, min(-(-8 * 148 // (b.n_dec * G)), -(-span // 128)))
                ws = e(b.n_dec * H * w.n_splits * (dv + 2)) if w.n_splits > 1 else None
                w.ws = ptr(ws)
                ev = self._ev()
                call_struct('p3_attn_window_decode', w, st)
                span = min(m.window, b.max_pos + 1) if m.window else b.max_pos + 1
                self._ev(ev, 'attn_decode', 2 * b.n_dec * H * span * (d + dv), b.n_dec * G * span * (d + dv) * esz)
            f = L['cfg'].ff
            after = self.layers[li + 1]['qkvg'] if li + 1 < len(self.layers) else self.head
            self.linear(att, L['o'], y, nxt=L['gu'] if f is not None and f.kind == 'dense' else (after if f is None else None))
            self.rows('norm', T * W * (12 + (4 if self.f32 else 2)), 'p3_postnorm_residual', ptr(y), y.stride(0), None, ptr(L['norm1']),
                      ptr(x), ptr(xa), self.f32, T, W, self.eps, st)
            f = L['cfg'].ff
            if f is not None:
                if f.kind == 'dense':
                    gu, hid = e(T, 2 * f.ff), e(T, f.ff, dt=act)
                    left = self.linear(xa, L['gu'], gu, L['gu_b32'], L['gu_b16'], nxt=L['down'])
                    self.rows('activation', T * f.ff * (8 + (4 if self.f32 else 2)), 'p3_glu_clamped', ptr(gu), gu.stride(0), ptr(hid),
                              hid.stride(0), self.f32, T, f.ff, f.limit, TagenexConfig.GLU_ALPHA, ptr(left), st)
                    left = self.linear(hid, L['down'], y, L['down_b32'], L['down_b16'], nxt=after)
                else:
                    self._moe(L, f, xa, y, T)
                    left = None
                self.rows('norm', T * W * (12 + (4 if self.f32 else 2)), 'p3_postnorm_residual', ptr(y), y.stride(0), ptr(left),
                          ptr(L['norm2']), ptr(x), ptr(xa), self.f32, T, W, self.eps, st)
            if trace is not None:
                trace.append(x.clone())
        if not b.R:
            return None
        xn = e(b.R, W, dt=act)
        call('p3_rmsnorm_rows_f32', ptr(x), ptr(b.want_rows), ptr(self.final_gain), ptr(xn), self.f32, b.R, W, self.eps, st)
        logits = e(b.R, self.V)
        self.linear(xn, self.head, logits)
        return logits

    def _moe(self, L, f, xa, y, T):
        """top-k mixture: route (softmax over the chosen logits), then the grouped expert products of the base class"""
        st = _stream()
        ids = torch.empty((T, f.top), dtype=torch.int32, device=self.dev)
        wts = torch.empty((T, f.top), dtype=torch.float32, device=self.dev)
        call('p3_router_topk', ptr(xa), xa.stride(0), self.f32, ptr(L['router']), ptr(L['router_b']), T, self.W, f.experts, f.top,
             ptr(ids), ptr(wts), st)
        glu = lambda gu, hid, n: call('p3_glu_clamped', ptr(gu), gu.stride(0), ptr(hid), hid.stride(0), self.f32, n, f.ff, f.limit,
                                      TagenexConfig.GLU_ALPHA, None, st)
        self.experts(L['gu'], L['down'], f, xa, y, T, ids, wts, glu)
