"""What the engine models (decoders with an fp32 residual stream that run a ragged token batch against the shared page pool) have in
common: the description of a step, the choice of the matrix-product kernel, the grouped expert products and the key-slice cost model
of the decode attention. A design (tagenex.py, tapalix.py, dugalix.py, danalorn.py) owns its weights and the order of its kernels; it has no cache and no loop
of its own.

Matrix products. Dense bf16 products with K % 8 == 0 run on the tcgen05 GEMM (p3_gemm); batches of at most 16 tokens on the
weight-streaming kernel (p3_gemm_skinny); everything else (fp32 = true 32-bit on the FMA pipes, grouped expert products, products
per attention head over column blocks, odd shapes) on p3_gemm_any.
"""
import os
import torch
from . import _lib
from ._lib import call, call_struct, ptr


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _page_slices(pairs, pages, slots=2 * 148, merge=0.0):
    """slices of the visible pages per (request, K/V head) for the tensor-core decode attention (two CTAs per SM). Cost model in
    units of the memory latency: a CTA pays one latency to fill its copy ring and half of one per page after that (two pages in
    flight); equal CTAs run in whole rounds of the resident ones. `merge`: what every further slice adds to the merge kernel, which
    walks the slices of a head one after the other (it matters when one K/V head serves many query heads: few CTAs, so the model
    would otherwise cut the keys into very many slices)."""
    best, best_cost = 1, float('inf')
    for ns in range(1, max(1, min(pages, 32)) + 1):
        per = -(-pages // ns)
        cost = -(-pairs * ns // slots) * (1.0 + per / 2.0) + (merge * ns if ns > 1 else 0.0)
        if cost < best_cost - 1e-9:
            best, best_cost = ns, cost
    return best


class StepBatch:
    """Device-side description of one engine step (built by engine.Engine.step)."""
    __slots__ = ('T', 'ids', 'tok_slot', 'tok_pos', 'pf_tiles', 'n_pf', 'dec_tiles', 'n_dec', 'want_rows', 'R', 'max_pos', 'flat',
                 'seqs', 'n_seq', 'slot_seq', 'n_slots')


class PagedLM:
    """base of the engine models: subclasses set self.dev, self.dtype, self.W (width), self.eps and call _init_products()"""

    def _init_products(self):
        self.f32 = int(self.dtype == torch.float32)
        self.use_tc = os.environ.get('P3_LM_TC', '1') != '0'
        self.moe_dense_rows = int(os.environ.get('P3_LM_MOE_DENSE_ROWS', '1024'))   # (token, choice) pairs from which experts run as dense GEMMs
        self.use_skinny = os.environ.get('P3_LM_SKINNY', '1') != '0' and hasattr(_lib.lib(), 'p3_gemm_skinny')
        self.profile = None      # bench.py: list of (kind, ev0, ev1, flops, bytes) when instrumenting

    def cache_dtype(self):
        return self.dtype

    def _ev(self, start=None, kind=None, flops=0, nbytes=0):
        if self.profile is None:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        if start is not None:
            self.profile.append((kind, start, e, flops, nbytes))
        return e

    def rows(self, kind, nbytes, name, *args):
        """a row kernel (norms, rotations, activations, routing) launched through _lib.call, or through _lib.call_struct when
        `args` is (argument struct,); bench.py's instrumentation times it under `kind` with the bytes it moves"""
        ev = self._ev()
        if len(args) == 1 and hasattr(args[0], '_fields_'):
            call_struct(name, args[0], _stream())
        else:
            call(name, *args)
        self._ev(ev, kind, 0, nbytes)

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, bias32=None, bias16=None, nxt=None):
        """out[M,N] (fp32 or act type, by out.dtype) = x[M,K] w[N,K]^T (+ bias). Returns the bias (fp32) that is STILL TO ADD: None
        when the product added it, bias32 when the kernel has no bias input (the weight-streaming kernel of small batches); the
        consumer kernel (activation / output norm) then adds it. `nxt`: the matrix of the next product; the weight-streaming
        kernel pulls its first megabytes into L2 so that they arrive while the small kernels in between run."""
        M, K = x.shape
        N = w.shape[0]
        ev = self._ev()
        try:
            return self._linear(x, w, out, bias32, bias16, nxt)
        finally:
            self._ev(ev, 'gemm', 2 * M * N * K, w.numel() * w.element_size() + x.numel() * x.element_size() + out.numel() * out.element_size())

    L2_PREFETCH_CAP = int(os.environ.get('P3_LM_PF_CAP_MB', '16')) << 20

    def _linear(self, x, w, out, bias32=None, bias16=None, nxt=None):
        M, K = x.shape
        N = w.shape[0]
        aligned = (not self.f32 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
        if (self.use_skinny and aligned and M <= 16 and K % 64 == 0 and N % 16 == 0 and out.dtype == torch.float32
                and w.is_contiguous()):
            # <= 16 tokens: the product is a stream of the weights; the Phi-3 decode kernel does that at HBM speed
            pf = 0 if nxt is None else min(nxt.numel() * nxt.element_size(), self.L2_PREFETCH_CAP)
            call('p3_gemm_skinny', ptr(x), x.stride(0), None, self.eps, ptr(w), ptr(out), out.stride(0), None, M, N, K,
                 _lib.EPI_F32, None, 0, None, ptr(nxt) if pf else None, pf, _stream())
            return bias32
        if self.use_tc and aligned and (bias32 is None or bias16 is not None):
            epi = _lib.EPI_F32 if out.dtype == torch.float32 else _lib.EPI_NONE
            call('p3_gemm', ptr(x), x.stride(0), ptr(w), w.stride(0), ptr(bias16), ptr(out), out.stride(0), None, None,
                 M, N, K, epi, 0, _stream())
            return None
        self.gemm_any(x, w, out, bias32)
        return None

    def gemm_any(self, x, w, out, bias=None, rows=None, row_div=1, seg=None, n_groups=0, M=None, N=None, K=None, ldw=None,
                 batch=None, gate=None):
        """out = x w^T on p3_gemm_any. rows / row_div: gathered activation rows; seg / n_groups: row segments that each take their
        own matrix w[g]. batch = (n, x stride, w stride, out stride): n products over column blocks of x and out (N, K, ldw give the
        shape of one), gate: fp32 logits whose sigmoid multiplies the result."""
        a = _lib.GemmAnyArgs()
        a.X, a.ldx, a.x_f32 = ptr(x), x.stride(0), self.f32
        a.x_rows, a.x_row_div = ptr(rows), row_div
        a.W, a.ldw, a.w_f32 = ptr(w), (w.stride(-2) if ldw is None else ldw), self.f32
        a.w_group_stride = w.stride(0) if (w.dim() == 3 and batch is None) else 0
        a.bias, a.bias_group_stride = ptr(bias), (bias.stride(0) if bias is not None and bias.dim() == 2 else 0)
        a.out, a.ldo, a.out_f32 = ptr(out), out.stride(0), int(out.dtype == torch.float32)
        a.M = x.shape[0] if M is None else M
        a.N, a.K = (w.shape[-2] if N is None else N), (w.shape[-1] if K is None else K)
        a.seg_offsets, a.n_groups = ptr(seg), n_groups
        if batch is not None:
            a.n_batch, a.x_batch_stride, a.w_batch_stride, a.out_batch_stride = batch
        if gate is not None:
            a.gate, a.ld_gate = ptr(gate), gate.stride(0)
        call_struct('p3_gemm_any', a, _stream())
        return out

    # ------------------------------------------------------------------ mixture of experts behind a router
    def experts(self, gu_w, down_w, f, xa, y, T, ids, wts, glu, n_sorted=None, combine=None):
        """ids / wts [T, top] from the design's router -> y fp32 [T, W] = sum of the chosen experts' outputs. gu_w [E, 2 ff, W] holds
        every expert's gate rows over its up rows, down_w [E, W, ff]; glu(gu fp32 [n, 2 ff], hid act [n, ff], n) is the design's
        activation. The (token, choice) pairs are sorted by expert and run as two grouped products over the sorted rows.
        A unit without a gate passes its up matrices alone ([E, ff, W]; the activation then gets [n, ff]). n_sorted: the router
        scores this many outputs, of which only the first f.experts have matrices (the pairs of the others are sorted behind them
        and skipped by the products); combine(dn, where) then replaces the plain weighted sum."""
        st, dev, n = _stream(), self.dev, T * f.top
        n_sorted = f.experts if n_sorted is None else n_sorted
        up = gu_w.shape[1]
        seg = torch.empty(n_sorted + 1, dtype=torch.int32, device=dev)
        order = torch.empty(n, dtype=torch.int32, device=dev)
        where = torch.empty(n, dtype=torch.int32, device=dev)
        call('p3_moe_sort', ptr(ids), n, n_sorted, ptr(seg), ptr(order), ptr(where), st)
        gu = torch.empty((n, up), dtype=torch.float32, device=dev)
        hid = torch.empty((n, f.ff), dtype=self.dtype, device=dev)
        dn = torch.empty((n, self.W), dtype=torch.float32, device=dev)
        # Large batches (prompt portions): the segment offsets are read back (one small D2H per mixture layer) and every expert's
        # rows go through the tcgen05 GEMM as a dense product over the gathered, expert-ordered activations. Small batches stay
        # on the device-side grouped kernel, which needs no host knowledge of the counts.
        dense = self.experts_dense(f, T)
        ev = self._ev()
        if dense:
            xs = torch.empty((n, self.W), dtype=self.dtype, device=dev)
            call('p3_gather_rows', ptr(xa), xa.stride(0), self.f32, ptr(order), f.top, ptr(xs), n, self.W, st)
            cut = seg.tolist()
            for ex in range(f.experts):
                a0, a1 = cut[ex], cut[ex + 1]
                if a1 > a0:
                    call('p3_gemm', ptr(xs[a0:a1]), xs.stride(0), ptr(gu_w[ex]), gu_w.stride(1), None, ptr(gu[a0:a1]), gu.stride(0),
                         None, None, a1 - a0, up, self.W, _lib.EPI_F32, 0, st)
        else:
            self.gemm_any(xa, gu_w, gu, rows=order, row_div=f.top, seg=seg, n_groups=f.experts, M=n)
        self._ev(ev, 'moe_gemm', 2 * n * up * self.W, gu_w.numel() * gu_w.element_size())
        glu(gu, hid, n)
        ev = self._ev()
        if dense:
            for ex in range(f.experts):
                a0, a1 = cut[ex], cut[ex + 1]
                if a1 > a0:
                    call('p3_gemm', ptr(hid[a0:a1]), hid.stride(0), ptr(down_w[ex]), down_w.stride(1), None, ptr(dn[a0:a1]),
                         dn.stride(0), None, None, a1 - a0, self.W, f.ff, _lib.EPI_F32, 0, st)
        else:
            self.gemm_any(hid, down_w, dn, seg=seg, n_groups=f.experts, M=n)
        self._ev(ev, 'moe_gemm', 2 * n * f.ff * self.W, down_w.numel() * down_w.element_size())
        if combine is not None:
            combine(dn, where)
        else:
            call('p3_moe_combine', ptr(dn), dn.stride(0), ptr(where), ptr(wts), f.top, ptr(y), T, self.W, st)

    def experts_dense(self, f, T):
        """do the experts of a step with T tokens run as dense per-expert products (which reads the segment offsets back)?"""
        return bool(self.use_tc and not self.f32 and T * f.top >= self.moe_dense_rows and self.W % 8 == 0 and f.ff % 8 == 0)
