"""Dugalix on B200: a decoder-only language model with an RMS norm (gain stored around zero) before AND after every sublayer,
x <- x + r N(mixer(shift(N(x)))), x <- x + r N(ff(N(x))), an fp32 residual stream, and a token shift in front of every mixer (each
channel of the normed input is blended with the same channel of the token before it). Two kinds of layers:

  'attention'  grouped-query attention over a sliding window whose values are the keys BEFORE their rotation (no value projection)
               and whose weights are sigmoid(score + per-head bias), not normalised over the keys;
  'parallel'   two mixers read the same input and their outputs are added with fixed factors: softmax attention with projection
               biases, a linearly slowed partial rotation and a window that also keeps the first tokens of the sequence; and a
               matrix-memory recurrence (exponential input gate, sigmoid forget gate, both soft-capped, running-maximum stabiliser)
               with a per-head unit norm, a gain and a sigmoid output gate.

Feed-forwards are relu^2 units, dense or as a mixture: softmax router over real and identity experts (an identity expert returns
its input), choice by corrected scores inside the best expert groups, the plain probabilities as weights, plus a shared unit behind
a per-token sigmoid gate.

The model owns weights and launches kernels; it has no cache, no state and no loop of its own. `forward(batch, pool)` runs ONE step
of the engine (engine.py): a ragged batch of new tokens of several sequences against the shared page pool (paged.py), which also
holds, per sequence slot, the state of the recurrent parts: the last normed row in front of every mixer (token shift) and the
matrix memories. A sequence's rows are walked in order by p3_token_shift and p3_matrix_memory_scan from the step's sequence
records; a first row at position 0 starts from zeros.

Kernels per layer (csrc/): p3_token_shift -> ONE product for all input projections of the layer (q | k [| v | memory q | k | v |
output gate | gate pre-activations]) -> p3_qkv_rope_post (biases, rotation, paged K/V write) -> p3_attn_window_prefill / _decode
(window, kept first tokens, softmax or sigmoid weights, output factor) and p3_matrix_memory_scan -> p3_headnorm_gate -> ONE output
product over [attention heads | memory heads] -> p3_postnorm_prenorm (norm of the sublayer output, residual add, norm in front of
the next sublayer) -> feed-forward: up product (dense) or shared up | shared gate | router logits product -> p3_relu2 -> down
product; mixtures: p3_router_groups -> p3_moe_sort -> grouped up product -> p3_relu2 -> grouped down product ->
p3_moe_combine_identity (identity experts and the shared unit join the sum) -> p3_postnorm_prenorm.

Precision. dtype=bfloat16 (serving): matrices, activations that feed a matrix product and the K/V cache are bf16, accumulation is
fp32; positions, angles, scores, attention weights, norms, router, the residual sum, the token-shift state, the gates of the
recurrence, its state and its sums are fp32. dtype=float32: everything is fp32 on the FMA pipes (no TF32).
"""
import ctypes as C

import torch
from . import _lib
from ._lib import call, call_struct, ptr
from .configs import DugalixConfig, rot_frequencies
from .lm_base import PagedLM, _page_slices, _stream


class DugalixB200(PagedLM):
    arch = 'Dugalix'

    def __init__(self, cfg, weights, device='cuda', dtype=torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError('DugalixB200 needs a CUDA device (sm_100a); there is no CPU fallback')
        _lib.lib()
        if isinstance(cfg, dict):
            cfg = DugalixConfig(cfg)
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError('dtype must be torch.bfloat16 or torch.float32')
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.W, self.V, self.eps = cfg.width, cfg.vocab_size, cfg.eps
        self._init_products()
        w, W, r = weights, self.W, cfg.residual_mult
        mat = lambda t: t.to(self.dev, dtype).contiguous()                     # matrices: the compute type
        f32 = lambda t: t.to(self.dev, torch.float32).contiguous()            # everything that enters fp32 arithmetic
        gain = lambda t, k=1.0: ((1.0 + t.to(self.dev, torch.float32)) * k).contiguous()   # weights stored around zero
        pad16 = lambda parts: parts + ([torch.zeros(-sum(p.shape[0] for p in parts) % 16, W, dtype=parts[0].dtype, device=parts[0].device)]
                                       if sum(p.shape[0] for p in parts) % 16 else [])

        def expect(name, shape):
            if tuple(w[name].shape) != tuple(shape):
                raise ValueError(f'{name}: shape {tuple(w[name].shape)}, the config gives {tuple(shape)}')

        self.embed = w['embed'].to(self.dev, torch.bfloat16).contiguous()      # bf16 values are exact in both modes
        self.final_gain, self.head = gain(w['final.norm']), mat(w['head'])
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, m, f = f'l{i}.', lc.mixer, lc.ff
            at, mem = m.att, m.mem
            L = dict(cfg=lc, pre1=gain(w[p + 'norm1']), post1=gain(w[p + 'norm1b'], r), shift=f32(w[p + 'shift']))
            a = p + ('mix.left.' if mem is not None else 'mix.')
            H, G, d, dv = at.heads, at.kv_heads, at.dim, at.vdim
            expect(a + 'q', (H * d, W)); expect(a + 'k', (G * d, W)); expect(a + 'o', (W, H * dv))
            parts = [w[a + 'q'], w[a + 'k']]
            L['q_off'], L['k_off'], L['v_off'] = 0, H * d, -1
            off = (H + G) * d
            if at.kind == 'softmax':
                expect(a + 'v', (G * dv, W))
                parts.append(w[a + 'v'])
                L['v_off'], off = off, off + G * dv
                L['in_b'] = torch.cat([f32(w[a + 'q.b']), f32(w[a + 'k.b']), f32(w[a + 'v.b'])])
                L['out_b'] = (f32(w[a + 'o.b']) * m.att_scale).contiguous()
                L['pb'] = None
            else:
                L['in_b'], L['out_b'], L['pb'] = None, None, f32(w[a + 'pb'])
            out_parts = [w[a + 'o']]
            if mem is not None:
                b = p + 'mix.right.'
                Hm, dm, dvm = mem.heads, mem.dim, mem.vdim
                expect(b + 'q', (Hm * dm, W)); expect(b + 'v', (Hm * dvm, W)); expect(b + 'o', (W, Hm * dvm)); expect(b + 'i', (Hm, W))
                L['mq_off'], L['mk_off'], L['mv_off'] = off, off + Hm * dm, off + 2 * Hm * dm
                L['mg_off'] = L['mv_off'] + Hm * dvm
                L['mi_off'], L['mf_off'] = L['mg_off'] + Hm * dvm, L['mg_off'] + Hm * dvm + Hm
                parts += [w[b + 'q'], w[b + 'k'], w[b + 'v'], w[b + 'g'], w[b + 'i'], w[b + 'f']]
                L['mi_b'], L['mf_b'], L['m_gain'] = f32(w[b + 'i.b']), f32(w[b + 'f.b']), f32(w[b + 'norm'])
                out_parts.append(w[b + 'o'])
            # all input projections of the layer are one product (rows padded to a multiple of 16 so that small batches keep the
            # weight-streaming kernel); the output projections of both halves read one concatenated activation row
            L['in_w'] = mat(torch.cat(pad16(parts), 0))
            L['out_w'] = mat(torch.cat(out_parts, 1))
            L['freq'] = (torch.tensor(rot_frequencies(at.rot), dtype=torch.float64).to(self.dev, torch.float32)
                         if at.rot is not None else None)
            L['rot_n'] = at.rot.dims if at.rot is not None else 0
            L['tile_rows'] = self._attention_tile_rows(at)
            if f is not None:
                q = p + 'mlp.'
                L['pre2'], L['post2'] = gain(w[p + 'norm2']), gain(w[p + 'norm2b'], r)
                if f.kind == 'dense':
                    L['up'], L['down'] = mat(w[q + 'up']), mat(w[q + 'down'])
                else:
                    # shared unit's up rows | its gate row | router rows ride in one product (fp32 accumulation of exact bf16
                    # products; all-fp32 in the fp32 mode)
                    sff = f.shared_ff
                    expect(q + 'router', (f.outputs, W))
                    parts2 = ([w[q + 'shared.up'], w[q + 'shared.sg']] if sff else []) + [w[q + 'router']]
                    L['sg_off'], L['r_off'] = sff, sff + (1 if sff else 0)
                    L['in2_w'] = mat(torch.cat(pad16(parts2), 0))
                    L['sh_down'] = mat(w[q + 'shared.down']) if sff else None
                    if f.experts:
                        L['up'] = mat(torch.stack([w[f'{q}e{e}.up'] for e in range(f.experts)], 0))
                        L['down'] = mat(torch.stack([w[f'{q}e{e}.down'] for e in range(f.experts)], 0))
                    L['correction'] = f32(w[q + 'correction']) if (q + 'correction') in w else None
            self.layers.append(L)
        # query rows per attention tile the engine cuts prompt portions into: 64 when every layer takes the tensor-core prefill
        # kernel (csrc/attention_window.cu), else 32
        self.q_tile = min(L['tile_rows'] for L in self.layers)
        self._state_layout = []
        for L in self.layers:
            mem = L['cfg'].mixer.mem
            L['shift_state'] = len(self._state_layout)
            self._state_layout.append(W)
            if mem is not None:
                L['mem_state'] = len(self._state_layout)
                self._state_layout.append(int(_lib.lib().p3_matrix_memory_state_floats(mem.heads, mem.dim, mem.vdim)))

    def _attention_tile_rows(self, at):
        """query rows per prefill tile that the attention launch takes for this mixer; asked of the library itself so that the
        engine's tiles and the kernel's choice cannot disagree"""
        a = _lib.AttnWindowArgs()
        a.q = a.out = a.k_pool = a.v_pool = a.block_table = a.tiles = 256              # aligned stand-ins: nothing is launched
        a.ld_q, a.ld_out, a.n_heads, a.n_kv, a.dim, a.vdim = at.heads * at.dim, 8 * at.heads * at.vdim, at.heads, at.kv_heads, at.dim, at.vdim
        a.window, a.keep_first = at.window, at.keep_first
        a.sig_bias = 256 if at.kind == 'sigmoid' else None
        a.act_f32 = a.cache_f32 = self.f32
        return int(_lib.lib().p3_attn_window_tile_rows(C.byref(a)))

    # ------------------------------------------------------------------ what the engine asks of a model
    def kv_layout(self):
        return self.cfg.kv_layout()

    def state_layout(self):
        """fp32 numbers per sequence slot and state buffer: per layer the token-shift row, then (parallel layers) the matrix
        memories; L['shift_state'] / L['mem_state'] index the pool's state buffers"""
        return list(self._state_layout)

    def prepare(self, max_context):
        """nothing depends on the longest context: angles are formed from the positions in the kernels"""

    def graph_safe(self, b):
        """may this step be captured as a CUDA graph? Not when a mixture layer would read its segment offsets back."""
        return not any(l.ff is not None and l.ff.kind == 'moe' and self.experts_dense(l.ff, b.T) for l in self.cfg.layers)

    # ------------------------------------------------------------------ one engine step
    def _norms(self, y, y_bias, post, x, pre, T, want32=False):
        """x += N(y + y_bias) * post (y None: x stays); -> (h fp32 or None, h in the activation type or None) = N(x) * pre"""
        if pre is None:
            h32 = ha = None
        elif self.f32 or want32:
            h32 = torch.empty((T, self.W), dtype=torch.float32, device=self.dev)
            ha = h32 if self.f32 else torch.empty((T, self.W), dtype=self.dtype, device=self.dev)
        else:
            h32, ha = None, torch.empty((T, self.W), dtype=self.dtype, device=self.dev)
        nb = T * self.W * ((12 if y is not None else 4) + (0 if pre is None else (4 if h32 is not None else 0) + (0 if self.f32 else 2)))
        self.rows('norm', nb, 'p3_postnorm_prenorm', ptr(y), y.stride(0) if y is not None else 0, ptr(y_bias), ptr(post), ptr(x),
                  ptr(pre), ptr(h32), None if self.f32 else ptr(ha), self.f32, T, self.W, self.eps, _stream())
        return h32, ha

    def forward(self, b, pool, trace=None):
        """b: StepBatch, pool: paged.PagePool -> fp32 logits [b.R, vocab] (None when no row is wanted).
        `trace` (a list) receives a copy of the residual stream after every layer."""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        x = e(T, W)
        call('p3_embed_rows_f32', ptr(self.embed), ptr(b.ids), ptr(x), None, self.f32, T, W, self.V, 1.0, W, st)
        h32, _ = self._norms(None, None, None, x, self.layers[0]['pre1'], T, want32=True)
        for li, L in enumerate(self.layers):
            f = L['cfg'].ff
            nxt_pre = self.layers[li + 1]['pre1'] if li + 1 < len(self.layers) else None
            y = self._mixer(L, li, h32, b, pool)
            if f is None:
                h32, _ = self._norms(y, L['out_b'], L['post1'], x, nxt_pre, T, want32=True)
            else:
                identity = f.kind == 'moe' and f.identity > 0
                h2_32, h2 = self._norms(y, L['out_b'], L['post1'], x, L['pre2'], T, want32=identity)
                y2 = self._dense(L, f, h2, T) if f.kind == 'dense' else self._moe(L, f, h2, h2_32, T)
                h32, _ = self._norms(y2, None, L['post2'], x, nxt_pre, T, want32=True)
            if trace is not None:
                trace.append(x.clone())
        if not b.R:
            return None
        xn = e(b.R, W, dt=act)
        call('p3_rmsnorm_rows_f32', ptr(x), ptr(b.want_rows), ptr(self.final_gain), ptr(xn), self.f32, b.R, W, self.eps, st)
        logits = e(b.R, self.V)
        self.linear(xn, self.head, logits)
        return logits

    def _mixer(self, L, li, h32, b, pool):
        """normed input h32 (fp32 [T, W]) -> mixer output before its norm, fp32 [T, W] (the output bias, if any, is still to add)"""
        st, dev, T, W = _stream(), self.dev, b.T, self.W
        act = self.dtype
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        m = L['cfg'].mixer
        at, mem = m.att, m.mem
        H, G, d, dv = at.heads, at.kv_heads, at.dim, at.vdim
        u = e(T, W, dt=act)
        self.rows('shift', T * W * (4 + (4 if self.f32 else 2)), 'p3_token_shift', ptr(h32), ptr(L['shift']),
                  ptr(pool.state[L['shift_state']]), ptr(b.seqs), ptr(b.slot_seq), ptr(b.tok_slot), ptr(u), self.f32, T, W, st)
        proj = e(T, L['in_w'].shape[0])
        self.linear(u, L['in_w'], proj, nxt=L['out_w'])
        n_att = H * dv
        cat = e(T, L['out_w'].shape[1], dt=act)               # [attention heads | memory heads]: the input of the output product
        q = e(T, H * d, dt=act)
        a = _lib.QkvRopePostArgs()
        a.proj, a.ld_proj, a.q_off, a.k_off, a.v_off, a.bias = ptr(proj), proj.stride(0), L['q_off'], L['k_off'], L['v_off'], ptr(L['in_b'])
        a.n_heads, a.n_kv, a.dim, a.vdim, a.rot_n, a.freq = H, G, d, dv, L['rot_n'], ptr(L['freq'])
        a.q_out, a.ld_q = ptr(q), q.stride(0)
        a.k_pool, a.v_pool = ptr(pool.k[li]), ptr(pool.v[li])
        a.block_table, a.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        a.tok_slot, a.tok_pos, a.T, a.act_f32, a.cache_f32 = ptr(b.tok_slot), ptr(b.tok_pos), T, self.f32, self.f32
        esz = 4 if self.f32 else 2
        self.rows('qkv_post', T * ((H + G) * d + max(0, G * dv)) * (4 + esz), 'p3_qkv_rope_post', a)
        w = _lib.AttnWindowArgs()
        w.q, w.ld_q, w.k_pool, w.v_pool = ptr(q), q.stride(0), ptr(pool.k[li]), ptr(pool.v[li])
        w.block_table, w.bt_stride = ptr(pool.block_table), pool.block_table.stride(0)
        w.out, w.ld_out = ptr(cat), cat.stride(0)
        w.n_heads, w.n_kv, w.dim, w.vdim, w.scale, w.window, w.keep_first = H, G, d, dv, at.scale, at.window, at.keep_first
        w.sig_bias, w.out_scale = ptr(L['pb']), m.att_scale
        w.act_f32, w.cache_f32 = self.f32, self.f32
        seen = lambda n: (min(at.window, n) + min(at.keep_first, max(0, n - at.window))) if at.window else n   # keys a query at n - 1 sees
        if b.n_pf:
            w.tiles, w.n_tiles = ptr(b.pf_tiles), b.n_pf
            ev = self._ev()
            call_struct('p3_attn_window_prefill', w, st)
            span = seen(b.max_pos + 1) if at.window else (b.max_pos + 1) // 2
            self._ev(ev, 'attn_prefill', 2 * (T - b.n_dec) * H * span * (d + dv), 0)
        if b.n_dec:
            w.tiles, w.n_tiles = ptr(b.dec_tiles), b.n_dec
            span = seen(b.max_pos + 1)
            if L['tile_rows'] == 64:
                w.n_splits = _page_slices(b.n_dec * G, 2 * -(-span // 128) + 1)
            else:
                # one key per lane: enough CTAs for eight per SM, at least 128 keys (one pass of a CTA) per slice
                w.n_splits = max(1, min(-(-8 * 148 // (b.n_dec * G)), -(-span // 128)))
            ws = e(b.n_dec * H * w.n_splits * (dv + 2)) if w.n_splits > 1 else None
            w.ws = ptr(ws)
            ev = self._ev()
            call_struct('p3_attn_window_decode', w, st)
            self._ev(ev, 'attn_decode', 2 * b.n_dec * H * span * (d + dv), b.n_dec * G * span * (d + dv) * esz)
        if mem is not None:
            Hm, dm, dvm = mem.heads, mem.dim, mem.vdim
            ym = e(T, Hm * dvm)
            r = _lib.MatrixMemoryArgs()
            r.proj, r.ld_proj = ptr(proj), proj.stride(0)
            r.q_off, r.k_off, r.v_off, r.i_off, r.f_off = L['mq_off'], L['mk_off'], L['mv_off'], L['mi_off'], L['mf_off']
            r.i_bias, r.f_bias, r.n_heads, r.dim, r.vdim = ptr(L['mi_b']), ptr(L['mf_b']), Hm, dm, dvm
            r.q_scale, r.gate_cap = dm ** -0.5, mem.gate_cap
            r.state, r.seqs, r.n_seqs = ptr(pool.state[L['mem_state']]), ptr(b.seqs), b.n_seq
            den = e(T, Hm)
            r.out, r.ld_out, r.den = ptr(ym), ym.stride(0), ptr(den)
            ev = self._ev()
            call_struct('p3_matrix_memory_scan', r, st)
            self._ev(ev, 'memory_scan', 4 * T * Hm * dm * dvm, T * L['in_w'].shape[0] * 4)
            self.rows('headnorm', T * Hm * dvm * (8 + esz), 'p3_headnorm_gate', ptr(ym), ym.stride(0), ptr(den), Hm, dvm, ptr(L['m_gain']),
                      ptr(proj[:, L['mg_off']:]), proj.stride(0), m.mem_scale, self.eps, ptr(cat[:, n_att:]), cat.stride(0), self.f32, T, st)
        y = e(T, W)
        f = L['cfg'].ff
        after = L.get('up') if f is not None and f.kind == 'dense' else (L.get('in2_w') if f is not None else None)
        self.linear(cat, L['out_w'], y, nxt=after)
        return y

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

    def _moe(self, L, f, h, h32, T):
        """mixture: shared unit (behind its per-token sigmoid gate), softmax group router, real and identity experts"""
        st, dev, W = _stream(), self.dev, self.W
        e = lambda *s, dt=torch.float32: torch.empty(s, dtype=dt, device=dev)
        p2 = e(T, L['in2_w'].shape[0])
        self.linear(h, L['in2_w'], p2, nxt=L['sh_down'])
        ysh = None
        if f.shared_ff:
            shid, ysh = e(T, f.shared_ff, dt=self.dtype), e(T, W)
            call('p3_relu2', ptr(p2), p2.stride(0), ptr(p2[:, L['sg_off']:]), p2.stride(0), ptr(shid), shid.stride(0), self.f32, T,
                 f.shared_ff, st)
            self.linear(shid, L['sh_down'], ysh)
        ids = torch.empty((T, f.top), dtype=torch.int32, device=dev)
        wts = torch.empty((T, f.top), dtype=torch.float32, device=dev)
        mode = _lib.ROUTER_SOFTMAX | _lib.ROUTER_GROUP_MAX | _lib.ROUTER_PLAIN_WEIGHTS
        call('p3_router_groups', ptr(p2[:, L['r_off']:]), p2.stride(0), ptr(L['correction']), T, f.outputs, f.top, f.groups, f.keep,
             1.0, mode, ptr(ids), ptr(wts), st)
        y = e(T, W)
        # identity experts return the layer's input: its fp32 copy, which forward() keeps when the layer has such experts
        combine = lambda dn, where: call('p3_moe_combine_identity', ptr(dn), dn.stride(0), ptr(where), ptr(ids), ptr(wts), f.top,
                                         f.experts, ptr(h32), ptr(ysh), ysh.stride(0) if ysh is not None else 0, ptr(y), T, W, st)
        relu2 = lambda up, hid, n: call('p3_relu2', ptr(up), up.stride(0), None, 0, ptr(hid), hid.stride(0), self.f32, n, f.ff, st)
        self.experts(L['up'], L['down'], f, h, y, T, ids, wts, relu2, n_sorted=f.outputs, combine=combine)
        return y
