// Paged attention over a ragged batch with a sliding window, a per-head sink in the softmax denominator and a per-head distance
// penalty: score(i, j) = scale * q_i . k_j - pen[h][i - j], visible when 0 <= i - j < window (window 0: every earlier key),
// weights = exp(score) / (exp(sink_h) + sum over visible exp(score)); optional output gates per (token, head) and per output number
// (the sigmoid of a logit, applied in the epilogue). Head sizes of
// keys (dim) and values (vdim) are independent run-time numbers, grouped-query heads share K/V (head h reads h / (H/G)). The fp32
// kernels take any size (rows above 256 numbers in key chunks and value column blocks), the tensor-core kernels sizes up to 256.
// With no window, sink or penalty this is plain causal attention; with v_pool == k_pool and v_ld == dim the value of a token is
// the leading part of its key row, which is how a latent-vector cache (one shared "head" that every query head reads, the
// up-projections folded into the queries and applied to the outputs) is served.
//
// All keys come from the page pools ([page][kv head][64 tokens][dim | vdim], fp32 or bf16): the caller writes the step's own K/V
// first. Scores, softmax and the P.V sums are fp32 on the FMA pipes in both storage modes, which is what the all-fp32 serving mode
// needs; the sink is folded in as the INITIAL state of the online softmax (running max = sink, denominator = 1, no value).
//   attn_window_prefill_kernel: one CTA = 32 consecutive query tokens of one sequence x one head, key tiles = whole pages, only
//                               the pages that hold a visible key are visited
//   attn_window_prefill_mma_kernel: the same on the tensor cores (bf16 mode, head sizes that tile), 64 query rows per CTA
//   attn_window_decode_kernel:  one CTA = one single-token request x one K/V head (all of its query heads share the K/V reads)
//                               x one slice of the visible keys, one key per lane; slices merged by attn_window_merge_kernel
#include "common.cuh"
#include "../../include/phi3_b200.h"
#include <cfloat>
#include <cstdlib>

namespace {
template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// element-wise output gate: sigmoid of the logit that belongs to output column `col` of batch row `row` (1 without such a gate)
__device__ __forceinline__ float elem_gate(const p3_attn_window_args& a, size_t row, size_t col) {
    return a.elem_gate ? 1.0f / (1.0f + expf(-a.elem_gate[row * a.ld_elem_gate + col])) : 1.f;
}

constexpr int BQ = 32, WARPS = 4, RPW = BQ / WARPS;          // prefill: query rows per CTA / per warp
constexpr int WIDE = 256;                                    // fp32 kernels: key numbers per chunk, value columns per CTA

// The pages a tile of queries visits: those of the kept first tokens that lie before the window's pages, then the pages from
// the first key inside the first row's window to the last row's own position.
struct PageWalk {
    int keep, n_keep, lo, n;
    __device__ PageWalk(const p3_attn_window_args& a, int first, int last) {
        keep = a.window > 0 ? a.keep_first : 0;              // without a window every earlier key is visible anyway
        lo = first / P3_PAGE;
        n_keep = min((keep + P3_PAGE - 1) / P3_PAGE, lo);
        n = n_keep + last / P3_PAGE - lo + 1;
    }
    __device__ __forceinline__ int page(int it) const { return it < n_keep ? it : lo + it - n_keep; }
};

template <typename AT, typename CT, int DVC>
__global__ void __launch_bounds__(WARPS * 32) attn_window_prefill_kernel(p3_attn_window_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ __align__(16) float sm[];
    // Rows of more than WIDE numbers: the scores are summed over key chunks of WIDE numbers (Q and K chunks restaged per page),
    // and the values are covered in column blocks of WIDE by blockIdx.z (each CTA forms the scores itself).
    const int d = a.dim, nchunk = (d + WIDE - 1) / WIDE, dp = (min(d, WIDE) + 3) & ~3;       // q rows padded to float4
    const int vc0 = blockIdx.z * WIDE, dv = min(a.vdim - vc0, WIDE);
    const int vld = a.v_ld > 0 ? a.v_ld : a.vdim;            // pitch of the value rows in a page
    float* Qs = sm;                                          // [BQ][dp]
    float* Ks = Qs + BQ * dp;                                // [64][dp + 1]
    float* Vs = Ks + P3_PAGE * (dp + 1);                     // [64][dv]
    float* Ss = Vs + P3_PAGE * dv;                           // [BQ][64 + 4]
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row0 = tile.x, nq = tile.y, slot = tile.z, pos0 = tile.w;
    const int h = blockIdx.y, g = h / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const AT* q = (const AT*)a.q;
    auto stage_q = [&](int c0, int dcur) {
        for (int i = tid; i < BQ * dp; i += blockDim.x) {
            const int r = i / dp, c = i % dp;
            Qs[i] = (r < nq && c < dcur) ? ldv(q + (size_t)(row0 + r) * a.ld_q + (size_t)h * d + c0 + c) * a.scale : 0.f;
        }
    };
    if (nchunk == 1) stage_q(0, d);
    const float sink = a.sink ? a.sink[h] : -FLT_MAX;
    float m[RPW], l[RPW], acc[RPW][DVC];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        m[r] = sink; l[r] = a.sink ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < DVC; j++) acc[r][j] = 0.f;
    }
    const int last = pos0 + nq - 1;
    const int first = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const float* pen = a.penalty ? a.penalty + (size_t)h * a.n_penalty : nullptr;
    const bool sig = a.sig_bias != nullptr;                  // sigmoid weights: no running maximum, no denominator
    const float sbias = sig ? a.sig_bias[h] : 0.f;
    const PageWalk walk(a, first, last);
    for (int it = 0; it < walk.n; it++) {
        const int pg = walk.page(it);
        const int page = bt[pg];
        const CT* kp = (const CT*)a.k_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * d;
        const CT* vp = (const CT*)a.v_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * vld + vc0;
        // scores: this warp's RPW rows x keys (lane, lane + 32)
        float s[RPW][2];
#pragma unroll
        for (int r = 0; r < RPW; r++) s[r][0] = s[r][1] = 0.f;
        for (int ck = 0; ck < nchunk; ck++) {
            const int c0 = ck * WIDE, dcur = min(WIDE, d - c0);
            __syncthreads();                                 // previous tile / chunk fully consumed (and Qs written, first time)
            if (nchunk > 1) stage_q(c0, dcur);
            for (int i = tid; i < P3_PAGE * dcur; i += blockDim.x) Ks[(i / dcur) * (dp + 1) + (i % dcur)] = ldv(kp + (size_t)(i / dcur) * d + c0 + (i % dcur));
            if (ck == 0)
                for (int i = tid; i < P3_PAGE * dv; i += blockDim.x) Vs[i] = ldv(vp + (size_t)(i / dv) * vld + (i % dv));
            __syncthreads();
            const float* k0 = Ks + lane * (dp + 1);
            const float* k1 = Ks + (lane + 32) * (dp + 1);
            for (int i = 0; i < dcur; i += 4) {
                float ka[4], kb[4];
#pragma unroll
                for (int e = 0; e < 4; e++) { const bool in = i + e < dcur; ka[e] = in ? k0[i + e] : 0.f; kb[e] = in ? k1[i + e] : 0.f; }
#pragma unroll
                for (int r = 0; r < RPW; r++) {
                    const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp * RPW + r) * dp + i);
                    s[r][0] = fmaf(qv.x, ka[0], s[r][0]); s[r][0] = fmaf(qv.y, ka[1], s[r][0]);
                    s[r][0] = fmaf(qv.z, ka[2], s[r][0]); s[r][0] = fmaf(qv.w, ka[3], s[r][0]);
                    s[r][1] = fmaf(qv.x, kb[0], s[r][1]); s[r][1] = fmaf(qv.y, kb[1], s[r][1]);
                    s[r][1] = fmaf(qv.z, kb[2], s[r][1]); s[r][1] = fmaf(qv.w, kb[3], s[r][1]);
                }
            }
        }
        // mask, penalty, online softmax; P goes to shared memory for the P.V pass
#pragma unroll
        for (int r = 0; r < RPW; r++) {
            const int qr = warp * RPW + r, qpos = pos0 + qr;
            float pv[2];
            float tmax = -FLT_MAX;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int kpos = pg * P3_PAGE + lane + 32 * e, dist = qpos - kpos;
                const bool vis = qr < nq && dist >= 0 && (a.window <= 0 || dist < a.window || kpos < walk.keep);
                float v = -FLT_MAX;
                if (vis) v = s[r][e] - (pen ? pen[min(dist, a.n_penalty - 1)] : 0.f);
                pv[e] = v;
                tmax = fmaxf(tmax, v);
            }
            if (sig) {
#pragma unroll
                for (int e = 0; e < 2; e++)
                    Ss[qr * (P3_PAGE + 4) + lane + 32 * e] = pv[e] > -FLT_MAX ? 1.0f / (1.0f + expf(-(pv[e] + sbias))) : 0.f;
                continue;
            }
            tmax = warp_max(tmax);
            const float mn = fmaxf(m[r], tmax);
            const float corr = expf(m[r] - mn);               // m is finite (sink) or -FLT_MAX; both give a finite difference or 0
            float ps = 0.f;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float p = pv[e] > -FLT_MAX ? expf(pv[e] - mn) : 0.f;
                Ss[qr * (P3_PAGE + 4) + lane + 32 * e] = p;
                ps += p;
            }
            ps = warp_sum(ps);
            l[r] = l[r] * corr + ps;
            m[r] = mn;
#pragma unroll
            for (int j = 0; j < DVC; j++) acc[r][j] *= corr;
        }
        __syncwarp();
        // P.V: lane owns value columns lane + 32 j
        for (int k = 0; k < P3_PAGE; k += 4) {
            float vv[4][DVC];
#pragma unroll
            for (int e = 0; e < 4; e++)
#pragma unroll
                for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; vv[e][j] = c < dv ? Vs[(k + e) * dv + c] : 0.f; }
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                const float4 p = *reinterpret_cast<const float4*>(Ss + (warp * RPW + r) * (P3_PAGE + 4) + k);
#pragma unroll
                for (int j = 0; j < DVC; j++) {
                    acc[r][j] = fmaf(p.x, vv[0][j], acc[r][j]); acc[r][j] = fmaf(p.y, vv[1][j], acc[r][j]);
                    acc[r][j] = fmaf(p.z, vv[2][j], acc[r][j]); acc[r][j] = fmaf(p.w, vv[3][j], acc[r][j]);
                }
            }
        }
    }
    AT* out = (AT*)a.out;
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const int qr = warp * RPW + r;
        if (qr >= nq) continue;
        const float gate = (a.gate ? a.gate[(size_t)(row0 + qr) * a.n_heads + h] : 1.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
        const float inv = sig ? gate : (l[r] > 0.f ? gate / l[r] : 0.f);
#pragma unroll
        for (int j = 0; j < DVC; j++) {
            const int c = lane + 32 * j;
            if (c < dv) {
                const size_t oc = (size_t)h * a.vdim + vc0 + c;
                stv(out + (size_t)(row0 + qr) * a.ld_out + oc, acc[r][j] * inv * elem_gate(a, row0 + qr, oc));
            }
        }
    }
}

// 2^x on the special-function unit (one instruction; -FLT_MAX and -inf give 0)
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 64 rows of a page (row-major, `chunks` 16-byte pieces per row) -> shared memory rows of pitch ld, by 128 threads: LPR lanes per
// row (chunks <= LPR), no division in the address arithmetic; src_ld = elements between the rows of the source
template <int LPR>
__device__ __forceinline__ void stage_rows(bf16* dst, int ld, const bf16* src, int chunks, int tid, int src_ld) {
    const int c = tid % LPR, r0 = tid / LPR;
    if (c < chunks) {
#pragma unroll
        for (int r = r0; r < P3_PAGE; r += 128 / LPR) cp_async16(smem_u32(dst + r * ld + c * 8), src + r * src_ld + c * 8);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// bf16 serving mode, head sizes that tile (dim % 16 == 0, vdim % 8 == 0, both <= 256): the two products run on the tensor cores
// (mma.sync m16n8k16, fp32 accumulators). One CTA = up to 64 query rows (4 warps x 16) x one head, key tile = one page. The K and
// V pages and the tile's penalties travel through a two-stage cp.async ring, so page j + 1 is in flight while page j is
// multiplied. Scores, mask, penalty (index row - col + 63 into the staged slice), sink and the online softmax stay fp32 in
// registers, in the base-2 domain (scale, penalty and sink carry the factor log2 e, so a weight is one subtraction and one
// ex2); the weights are rounded to bf16 only as the A operand of P.V, taken straight from the score accumulators. K fragments
// come by ldmatrix from the row-major page, V by ldmatrix.trans. A page that every row of the tile sees in full (behind the
// diagonal, inside the window) skips the visibility tests.
template <int DK, int DN, int MINB, bool SIG>
__global__ void __launch_bounds__(128, MINB) attn_window_prefill_mma_kernel(p3_attn_window_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr float LOG2E = 1.4426950408889634f;
    // blockIdx.z = a block of 8 DN value columns (values wider than that are covered by several CTAs that each form the scores)
    constexpr bool PARTS = DK > 8;                           // only the wide variant is launched with several column blocks
    const int vc0 = PARTS ? blockIdx.z * 8 * DN : 0, dv = PARTS ? min(a.vdim - vc0, 8 * DN) : a.vdim, dvs = PARTS ? min(a.vdim, 8 * DN) : a.vdim;
    const int d = a.dim, ldk = d + 8, ldv = dvs + 8, vld = a.v_ld > 0 ? a.v_ld : a.vdim;
    const bool v_in_k = a.v_pool == a.k_pool && vld == d && a.n_kv == 1;   // values = leading part of the key rows: staged once
    const int stage_elems = P3_PAGE * (ldk + ldv);           // bf16 elements of one stage: K [64][ldk] then V [64][ldv]
    bf16* kv_s = reinterpret_cast<bf16*>(smraw);
    float* pen_s = reinterpret_cast<float*>(kv_s + 2 * stage_elems);   // [2][128]
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row0 = tile.x, nq = tile.y, slot = tile.z, pos0 = tile.w;
    const int h = blockIdx.y, g = h / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int r0 = warp * 16 + gid, r1 = r0 + 8;             // this thread's two rows of the tile
    const int last = pos0 + nq - 1;
    const int first = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const float* pen = a.penalty ? a.penalty + (size_t)h * a.n_penalty : nullptr;
    const int kc = d / 8, vc = dv / 8;                       // 16-byte chunks per row
    const PageWalk walk(a, first, last);
    constexpr bool sig = SIG;                                // sigmoid weights (a.sig_bias): no running maximum, no denominator
    const float sbias2 = sig ? a.sig_bias[h] * LOG2E : 0.f;

    auto stage_page = [&](int pg, int st) {                  // all threads: issue the copies of page pg into stage st
        const int page = bt[pg];
        const bf16* kp = (const bf16*)a.k_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * d;
        const bf16* vp = (const bf16*)a.v_pool + ((size_t)page * a.n_kv + g) * P3_PAGE * vld + vc0;
        bf16* Ks = kv_s + st * stage_elems;
        bf16* Vs = Ks + P3_PAGE * ldk;
        stage_rows<2 * DK>(Ks, ldk, kp, kc, tid, d);
        if (!v_in_k) stage_rows<DN>(Vs, ldv, vp, vc, tid, vld);
        // penalty at distance (row - col + 63) + dmin, dmin = pos0 - (pg * 64 + 63); plain store, made visible by the barrier
        // that follows the wait for this stage
        const int dist = pos0 - (pg * P3_PAGE + 63) + tid;
        pen_s[st * 128 + tid] = (pen && dist >= 0) ? pen[min(dist, a.n_penalty - 1)] * LOG2E : 0.f;
    };
    stage_page(walk.page(0), 0);
    cp_async_commit();

    const bf16* q = (const bf16*)a.q + (size_t)h * d;
    uint32_t qf[DK][4];
#pragma unroll
    for (int t = 0; t < DK; t++) {
        qf[t][0] = qf[t][1] = qf[t][2] = qf[t][3] = 0u;
        if (t * 16 < d) {
            const int c = t * 16 + tig * 2;
            if (r0 < nq) { const bf16* p = q + (size_t)(row0 + r0) * a.ld_q + c; qf[t][0] = *reinterpret_cast<const uint32_t*>(p); qf[t][2] = *reinterpret_cast<const uint32_t*>(p + 8); }
            if (r1 < nq) { const bf16* p = q + (size_t)(row0 + r1) * a.ld_q + c; qf[t][1] = *reinterpret_cast<const uint32_t*>(p); qf[t][3] = *reinterpret_cast<const uint32_t*>(p + 8); }
        }
    }
    const float sink = a.sink ? a.sink[h] * LOG2E : -FLT_MAX;
    const float scale2 = a.scale * LOG2E;
    float m0 = sink, m1 = sink, l0 = (a.sink && tig == 0) ? 1.f : 0.f, l1 = l0;   // row sums are per-thread partials of a quad
    float o[DN][4];
#pragma unroll
    for (int n = 0; n < DN; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

    for (int it = 0; it < walk.n; it++) {
        const int pg = walk.page(it), st = it & 1;
        __syncthreads();                                     // every warp is done with the stage that is refilled now
        if (it + 1 < walk.n) stage_page(walk.page(it + 1), st ^ 1);
        cp_async_commit();
        cp_async_wait<1>();                                  // page pg has landed (this thread's copies) ...
        __syncthreads();                                     // ... and everyone else's
        const bf16* Ks = kv_s + st * stage_elems;
        const bf16* Vs = v_in_k ? Ks + vc0 : Ks + P3_PAGE * ldk;
        const int ldvs = v_in_k ? ldk : ldv;
        const float* ps = pen_s + st * 128;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        // K fragments: one ldmatrix.x4 = keys 16 jj .. 16 jj + 15 x dims 16 t .. 16 t + 15 (b0, b1 of key block 2 jj, then 2 jj + 1)
        const bf16* krow = Ks + ((lane & 7) + 8 * (lane >> 4)) * ldk + 8 * ((lane >> 3) & 1);
#pragma unroll
        for (int t = 0; t < DK; t++) {
            if (t * 16 < d) {
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(krow + jj * 16 * ldk + t * 16));
                    mma_bf16_16816(s[2 * jj], qf[t], b0, b1);
                    mma_bf16_16816(s[2 * jj + 1], qf[t], b2, b3);
                }
            }
        }
        float mx0 = -FLT_MAX, mx1 = -FLT_MAX;
        // every key of the page is visible to every row of the tile: behind the first row, and the last row's window reaches it
        const bool full = pg * P3_PAGE + 63 <= pos0 && (a.window <= 0 || pos0 + 63 - pg * P3_PAGE < a.window || pg * P3_PAGE + 63 < walk.keep);
        // the penalty depends on row - col only, and this thread's second row is its first plus 8: the penalties of (r1, key block
        // j) are those of (r0, key block j - 1), so 18 values serve the 32 scores
        float pq[9][2];
#pragma unroll
        for (int j = 0; j < 9; j++) {
            pq[j][0] = ps[r0 - ((j - 1) * 8 + tig * 2) + 63];
            pq[j][1] = ps[r0 - ((j - 1) * 8 + tig * 2 + 1) + 63];
        }
        if (full) {
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s[j][e] = fmaf(s[j][e], scale2, -pq[(e < 2) ? j + 1 : j][e & 1]);
                }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int row = (e < 2) ? r0 : r1, col = j * 8 + tig * 2 + (e & 1);
                    const int kpos = pg * P3_PAGE + col, dist = pos0 + row - kpos;
                    const bool vis = row < nq && dist >= 0 && (a.window <= 0 || dist < a.window || kpos < walk.keep);
                    s[j][e] = vis ? fmaf(s[j][e], scale2, -pq[(e < 2) ? j + 1 : j][e & 1]) : -FLT_MAX;
                }
        }
        if (sig) {                                           // weight = 1 / (1 + 2^-(score + bias)), 0 for a masked key
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = s[j][e];
                    s[j][e] = (full || v > -FLT_MAX) ? __frcp_rn(1.0f + ex2f(-(v + sbias2))) : 0.f;
                }
        } else {
        {   // row maxima by a tree (depth 4 instead of a chain of 16)
            float t0[8], t1[8];
#pragma unroll
            for (int j = 0; j < 8; j++) { t0[j] = fmaxf(s[j][0], s[j][1]); t1[j] = fmaxf(s[j][2], s[j][3]); }
#pragma unroll
            for (int w = 4; w > 0; w >>= 1)
#pragma unroll
                for (int j = 0; j < w; j++) { t0[j] = fmaxf(t0[j], t0[j + w]); t1[j] = fmaxf(t1[j], t1[j + w]); }
            mx0 = t0[0]; mx1 = t1[0];
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float c0 = ex2f(m0 - n0), c1 = ex2f(m1 - n1);     // m is finite (sink) or -FLT_MAX: the difference is finite or -inf
        m0 = n0; m1 = n1;
        float q0[4] = {0.f, 0.f, 0.f, 0.f}, q1[4] = {0.f, 0.f, 0.f, 0.f};   // four partial row sums each: short dependency chains
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float v = s[j][e];
                const float p = (full || v > -FLT_MAX) ? ex2f(v - ((e < 2) ? n0 : n1)) : 0.f;
                s[j][e] = p;
                if (e < 2) q0[(j & 1) * 2 + e] += p; else q1[(j & 1) * 2 + (e & 1)] += p;
            }
        const float ps0 = (q0[0] + q0[1]) + (q0[2] + q0[3]), ps1 = (q1[0] + q1[1]) + (q1[2] + q1[3]);
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {   // a maximum moved somewhere in the warp (a factor of exactly 1 changes nothing)
#pragma unroll
            for (int n = 0; n < DN; n++) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        }
        }
#pragma unroll
        for (int t = 0; t < 4; t++) {                        // 16 keys per step
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * t][0], s[2 * t][1]); pa[1] = pack_bf16(s[2 * t][2], s[2 * t][3]);
            pa[2] = pack_bf16(s[2 * t + 1][0], s[2 * t + 1][1]); pa[3] = pack_bf16(s[2 * t + 1][2], s[2 * t + 1][3]);
            const bf16* vrow = Vs + (t * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldvs + 8 * (lane >> 4);
#pragma unroll
            for (int n = 0; n < DN; n += 2) {
                if (n * 8 < dv) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(vrow + n * 8));
                    mma_bf16_16816(o[n], pa, b0, b1);
                    if (n + 1 < DN) mma_bf16_16816(o[n + 1], pa, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    bf16* out = (bf16*)a.out + (size_t)h * a.vdim + vc0;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int row = half ? r1 : r0;
        if (row >= nq) continue;
        const float l = half ? l1 : l0;
        const float gate = (a.gate ? a.gate[(size_t)(row0 + row) * a.n_heads + h] : 1.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
        const float inv = sig ? gate : (l > 0.f ? gate / l : 0.f);
#pragma unroll
        for (int n = 0; n < DN; n++) {
            const int c = n * 8 + tig * 2;
            if (c < dv) {
                const size_t oc = (size_t)h * a.vdim + vc0 + c;
                *reinterpret_cast<uint32_t*>(out + (size_t)(row0 + row) * a.ld_out + c) =
                    pack_bf16(o[n][half * 2] * inv * elem_gate(a, row0 + row, oc), o[n][half * 2 + 1] * inv * elem_gate(a, row0 + row, oc + 1));
            }
        }
    }
}

constexpr int DW = 4, RMAX = 8;                              // decode: warps per CTA, query heads per pass

template <typename CT> __device__ __forceinline__ void load8(const CT* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* f) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), e = unpack_bf16(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = e.x; f[7] = e.y;
}

// Decode: one CTA = one single-token request x one K/V head x one slice of the visible keys (grid.z = n_splits). A warp takes
// 32 keys at a time, ONE KEY PER LANE: the lane reads its key row in 16-byte pieces and forms the dot products with all query
// heads of the group (q broadcast from shared memory), so a score costs no cross-lane traffic; the softmax statistics take one
// warp reduction per 32 keys and head. For P.V the lanes switch to value columns and the weights travel by shuffle. Warps are
// merged through shared memory; with several slices the CTA writes its unnormalised (max, sum, vector) to the workspace and
// attn_window_merge_kernel combines them. The sink enters once, as the initial state of slice 0's first warp.
template <typename AT, typename CT, int DVC>
__global__ void __launch_bounds__(DW * 32) attn_window_decode_kernel(p3_attn_window_args a, int v_parts) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ __align__(16) float sm[];
    // blockIdx.y = K/V head x block of WIDE value columns (wider values: several CTAs that each form the scores)
    const int vc0 = (blockIdx.y % v_parts) * WIDE, dv = min(a.vdim - vc0, WIDE);
    const int d = a.dim, rep = a.n_heads / a.n_kv, G = a.n_kv, vld = a.v_ld > 0 ? a.v_ld : a.vdim;
    float* Qs = sm;                                          // [RMAX][d]
    float* Ms = Qs + RMAX * d;                               // [DW][RMAX]
    float* Ls = Ms + DW * RMAX;                              // [DW][RMAX]
    float* As = Ls + DW * RMAX;                              // [DW][RMAX][dv]
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row = tile.x, slot = tile.z, pos = tile.w;
    const int g = blockIdx.y / v_parts, split = blockIdx.z, n_splits = gridDim.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    // the visible keys in one running index: the kept first tokens that lie before the window, then the window
    const int n_keep = a.window > 0 ? min(a.keep_first, first) : 0, n_vis = n_keep + pos - first + 1;
    const int per = ((n_vis + n_splits - 1) / n_splits + 31) & ~31;
    const int k_lo = split * per, k_hi = min(n_vis, k_lo + per);
    auto key_at = [&](int c) { return c < n_keep ? c : first + c - n_keep; };
    const bool sig = a.sig_bias != nullptr;                  // sigmoid weights: the maximum is pinned at 0, the sum is not used
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const AT* q = (const AT*)a.q + (size_t)row * a.ld_q;
    const bool vec = (d % 8 == 0) && (((uintptr_t)a.k_pool & 15) == 0);
    for (int h0 = 0; h0 < rep; h0 += RMAX) {
        const int nr = min(RMAX, rep - h0), hb = g * rep + h0;
        __syncthreads();
        for (int i = tid; i < nr * d; i += blockDim.x) Qs[i] = ldv(q + (size_t)hb * d + i) * a.scale;
        __syncthreads();
        float m[RMAX], l[RMAX], acc[RMAX][DVC];
#pragma unroll
        for (int r = 0; r < RMAX; r++) {
            const bool s0 = split == 0 && warp == 0 && a.sink && r < nr;
            m[r] = s0 ? a.sink[hb + r] : -FLT_MAX; l[r] = (s0 && lane == 0) ? 1.f : 0.f;      // l: per-lane partial sums
#pragma unroll
            for (int j = 0; j < DVC; j++) acc[r][j] = 0.f;
        }
        for (int kb = k_lo + warp * 32; kb < k_hi; kb += DW * 32) {
            const bool valid = kb + lane < k_hi;
            const int kpos = key_at(kb + lane);
            float s[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; r++) s[r] = 0.f;
            if (valid) {
                const CT* kp = (const CT*)a.k_pool + (((size_t)bt[kpos / P3_PAGE] * G + g) * P3_PAGE + kpos % P3_PAGE) * d;
                if (vec) {
#pragma unroll 8
                    for (int i = 0; i < d; i += 8) {
                        float kf[8];
                        load8(kp + i, kf);
#pragma unroll
                        for (int r = 0; r < RMAX; r++) {
                            if (r >= nr) break;
                            const float4 qa = *reinterpret_cast<const float4*>(Qs + r * d + i), qb = *reinterpret_cast<const float4*>(Qs + r * d + i + 4);
                            s[r] = fmaf(qa.x, kf[0], s[r]); s[r] = fmaf(qa.y, kf[1], s[r]); s[r] = fmaf(qa.z, kf[2], s[r]); s[r] = fmaf(qa.w, kf[3], s[r]);
                            s[r] = fmaf(qb.x, kf[4], s[r]); s[r] = fmaf(qb.y, kf[5], s[r]); s[r] = fmaf(qb.z, kf[6], s[r]); s[r] = fmaf(qb.w, kf[7], s[r]);
                        }
                    }
                } else {
                    for (int i = 0; i < d; i++) {
                        const float kv = ldv(kp + i);
#pragma unroll
                        for (int r = 0; r < RMAX; r++) { if (r >= nr) break; s[r] = fmaf(Qs[r * d + i], kv, s[r]); }
                    }
                }
            }
            const int dist = pos - kpos;
            float p[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; r++) {
                p[r] = 0.f;
                if (r >= nr) continue;
                float sv = -FLT_MAX;
                if (valid) sv = s[r] - (a.penalty ? a.penalty[(size_t)(hb + r) * a.n_penalty + min(dist, a.n_penalty - 1)] : 0.f);
                if (sig) {
                    p[r] = valid ? 1.0f / (1.0f + expf(-(sv + a.sig_bias[hb + r]))) : 0.f;
                    l[r] += p[r];
                    m[r] = 0.f;
                    continue;
                }
                const float mn = fmaxf(m[r], warp_max(sv)), corr = expf(m[r] - mn);
                p[r] = valid ? expf(sv - mn) : 0.f;
                l[r] = l[r] * corr + p[r];
                m[r] = mn;
#pragma unroll
                for (int j = 0; j < DVC; j++) acc[r][j] *= corr;
            }
            const int nk = min(32, k_hi - kb);
            constexpr int VR = DVC <= 2 ? 16 : (DVC <= 4 ? 8 : 4);   // value rows in flight per step
            for (int k0 = 0; k0 < nk; k0 += VR) {
                float vr[VR][DVC];
#pragma unroll
                for (int u = 0; u < VR; u++) {
                    const int kp2 = key_at(min(kb + k0 + u, k_hi - 1));
                    const CT* vp = (const CT*)a.v_pool + (((size_t)bt[kp2 / P3_PAGE] * G + g) * P3_PAGE + kp2 % P3_PAGE) * vld + vc0;
#pragma unroll
                    for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; vr[u][j] = c < dv ? ldv(vp + c) : 0.f; }
                }
#pragma unroll
                for (int u = 0; u < VR; u++) {
#pragma unroll
                    for (int r = 0; r < RMAX; r++) {
                        if (r >= nr) break;
                        const float pk = __shfl_sync(0xffffffffu, p[r], (k0 + u) & 31);   // weight 0 beyond the slice's end
#pragma unroll
                        for (int j = 0; j < DVC; j++) acc[r][j] = fmaf(pk, vr[u][j], acc[r][j]);
                    }
                }
            }
        }
        // merge the warps' partial states
#pragma unroll
        for (int r = 0; r < RMAX; r++) {
            if (r >= nr) break;
            const float lt = warp_sum(l[r]);
            if (lane == 0) { Ms[warp * RMAX + r] = m[r]; Ls[warp * RMAX + r] = lt; }
#pragma unroll
            for (int j = 0; j < DVC; j++) { const int c = lane + 32 * j; if (c < dv) As[(size_t)(warp * RMAX + r) * dv + c] = acc[r][j]; }
        }
        __syncthreads();
        for (int i = tid; i < nr * dv; i += blockDim.x) {
            const int r = i / dv, c = i % dv;
            float M = -FLT_MAX;
            for (int w = 0; w < DW; w++) M = fmaxf(M, Ms[w * RMAX + r]);
            float L = 0.f, o = 0.f;
            for (int w = 0; w < DW; w++) {
                const float f = Ls[w * RMAX + r] > 0.f ? expf(Ms[w * RMAX + r] - M) : 0.f;
                L = fmaf(Ls[w * RMAX + r], f, L);
                o = fmaf(As[(size_t)(w * RMAX + r) * dv + c], f, o);
            }
            if (n_splits == 1) {
                const float gate = (a.gate ? a.gate[(size_t)row * a.n_heads + hb + r] : 1.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
                const size_t oc = (size_t)(hb + r) * a.vdim + vc0 + c;
                stv((AT*)a.out + (size_t)row * a.ld_out + oc, L > 0.f ? o * gate / (sig ? 1.f : L) * elem_gate(a, row, oc) : 0.f);
            } else {
                float* w = a.ws + (((size_t)blockIdx.x * a.n_heads + hb + r) * n_splits + split) * (a.vdim + 2);
                if (c == 0 && vc0 == 0) { w[0] = M; w[1] = L; }            // every column block forms the same maximum and sum
                w[2 + vc0 + c] = o;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Decode on the tensor cores (bf16 mode, head sizes that tile). One CTA = one single-token request x one K/V head x one slice of
// the visible PAGES; its K and V pages stream through a cp.async ring of 2 or 3 stages (whole pages, 16-byte copies; the launch
// takes as many stages as let two CTAs share an SM), so the kernel
// is a stream of the cache. The query heads of the group are the rows of one m16n8k16 tile (rows beyond the group are zero).
// Each warp takes 16 keys of the page: scores by mma.sync from ldmatrix K fragments, fp32 mask / penalty / online softmax in
// registers (base-2 domain), weights rounded to bf16 as the A operand of P.V against ldmatrix.trans V fragments. The warps keep
// separate softmax states and are merged through shared memory at the end; slices are merged by attn_window_merge_kernel.
// Keys of the last page beyond the query's position, and of the first page before the window, are masked; what those cache rows
// hold is finite (the pool is zero-initialised and only ever written with finite numbers), so a zero weight removes them.
constexpr int DEC_MAX_STAGES = 3;                          // a fourth stage measured slower on B200 (two CTAs no longer share an SM)

// wait until at most n of this thread's copy groups are pending (n is uniform over the CTA)
__device__ __forceinline__ void cp_async_wait_pending(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        default: cp_async_wait<4>(); break;
    }
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory");
}

// The loop holds no plain global load on its critical path: the penalties of a page's 64 distances travel with the page
// (4-byte async copies into the stage), and the block-table entry of the page issued next is read one iteration ahead.
template <int DK, int DN>
__global__ void __launch_bounds__(128, 2) attn_window_decode_mma_kernel(p3_attn_window_args a, int n_stages, int v_parts) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr float LOG2E = 1.4426950408889634f;
    // blockIdx.y = K/V head x block of 8 DN value columns (wider values: several CTAs that each form the scores)
    constexpr bool PARTS = DK > 8;                           // only the wide variant is launched with several column blocks
    if (!PARTS) v_parts = 1;
    const int vc0 = PARTS ? (blockIdx.y % v_parts) * 8 * DN : 0, dv = PARTS ? min(a.vdim - vc0, 8 * DN) : a.vdim, dvs = PARTS ? min(a.vdim, 8 * DN) : a.vdim;
    const int d = a.dim, ldk = d + 8, ldv = dvs + 8, rep = a.n_heads / a.n_kv, G = a.n_kv, vld = a.v_ld > 0 ? a.v_ld : a.vdim;
    const bool v_in_k = a.v_pool == a.k_pool && vld == d && G == 1;       // values = leading part of the key rows: staged once
    const int pr = min(rep, 16);                             // penalty rows per stage
    const int stage_bytes = P3_PAGE * (ldk + ldv) * 2 + pr * P3_PAGE * 4;   // K [64][ldk], V [64][ldv] (bf16), penalties [pr][64] (fp32)
    float* Ms = reinterpret_cast<float*>(smraw);             // after the stream: [4 warps][16 rows] maxima, sums, [4][16][dv] vectors
    float* Ls = Ms + 64;
    float* Os = Ls + 64;
    const int4 tile = reinterpret_cast<const int4*>(a.tiles)[blockIdx.x];
    const int row = tile.x, slot = tile.z, pos = tile.w;
    const int g = PARTS ? blockIdx.y / v_parts : blockIdx.y, split = blockIdx.z, n_splits = gridDim.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const PageWalk walk(a, first, pos);                      // the kept first pages, then the window's pages: one running index
    const int per = (walk.n + n_splits - 1) / n_splits;      // pages per slice, rounded up
    const int pg_lo = split * per;                           // first running index of this slice
    const int n_pg = max(0, min(walk.n, pg_lo + per) - pg_lo);
    const bool sig = a.sig_bias != nullptr;                  // sigmoid weights: the maximum is pinned at 0, the sum is not used
    const int32_t* bt = a.block_table + (size_t)slot * a.bt_stride;
    const int kc = d / 8, vc = dv / 8;
    const float scale2 = a.scale * LOG2E;

    for (int h0 = 0; h0 < rep; h0 += 16) {
        const int nr = min(16, rep - h0), hb = g * rep + h0;
        auto stage_page = [&](int pg, int page, int st) {
            const bf16* kp = (const bf16*)a.k_pool + ((size_t)page * G + g) * P3_PAGE * d;
            const bf16* vp = (const bf16*)a.v_pool + ((size_t)page * G + g) * P3_PAGE * vld + vc0;
            bf16* Ks = reinterpret_cast<bf16*>(smraw + (size_t)st * stage_bytes);
            bf16* Vs = Ks + P3_PAGE * ldk;
            stage_rows<2 * DK>(Ks, ldk, kp, kc, tid, d);
            if (!v_in_k) stage_rows<DN>(Vs, ldv, vp, vc, tid, vld);
            if (a.penalty) {
                float* Ps = reinterpret_cast<float*>(Vs + P3_PAGE * ldv);
                for (int i = tid; i < nr * P3_PAGE; i += 128) {
                    const int dist = pos - (pg * P3_PAGE + (i & 63));             // masked keys (dist < 0) read entry 0, unused
                    cp_async4(smem_u32(Ps + i), a.penalty + (size_t)(hb + (i >> 6)) * a.n_penalty + min(max(dist, 0), a.n_penalty - 1));
                }
            }
        };
        __syncthreads();                                     // the merge buffer of the previous pass is read
        for (int s = 0; s < n_stages - 1; s++) {
            if (s < n_pg) stage_page(walk.page(pg_lo + s), bt[walk.page(pg_lo + s)], s);
            cp_async_commit();
        }
        int next_page = (n_stages - 1 < n_pg) ? bt[walk.page(pg_lo + n_stages - 1)] : 0;
        const bf16* q = (const bf16*)a.q + (size_t)row * a.ld_q + (size_t)hb * d;
        uint32_t qf[DK][4];
#pragma unroll
        for (int t = 0; t < DK; t++) {
            qf[t][0] = qf[t][1] = qf[t][2] = qf[t][3] = 0u;
            if (t * 16 < d) {
                const int c = t * 16 + tig * 2;
                if (gid < nr) { const bf16* p = q + (size_t)gid * d + c; qf[t][0] = *reinterpret_cast<const uint32_t*>(p); qf[t][2] = *reinterpret_cast<const uint32_t*>(p + 8); }
                if (gid + 8 < nr) { const bf16* p = q + (size_t)(gid + 8) * d + c; qf[t][1] = *reinterpret_cast<const uint32_t*>(p); qf[t][3] = *reinterpret_cast<const uint32_t*>(p + 8); }
            }
        }
        // the sink enters once per head: as the initial state of slice 0's first warp
        const bool s0 = split == 0 && warp == 0 && a.sink;
        float m0 = sig ? 0.f : (s0 && gid < nr) ? a.sink[hb + gid] * LOG2E : -FLT_MAX;
        float m1 = sig ? 0.f : (s0 && gid + 8 < nr) ? a.sink[hb + gid + 8] * LOG2E : -FLT_MAX;
        const float sb0 = (sig && gid < nr) ? a.sig_bias[hb + gid] * LOG2E : 0.f, sb1 = (sig && gid + 8 < nr) ? a.sig_bias[hb + gid + 8] * LOG2E : 0.f;
        float l0 = (s0 && gid < nr && tig == 0) ? 1.f : 0.f, l1 = (s0 && gid + 8 < nr && tig == 0) ? 1.f : 0.f;
        const bool has_pen = a.penalty != nullptr;
        const int prow0 = min(gid, nr - 1) * P3_PAGE, prow1 = min(gid + 8, nr - 1) * P3_PAGE;
        float o[DN][4];
#pragma unroll
        for (int n = 0; n < DN; n++) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

        for (int i = 0; i < n_pg; i++) {
            cp_async_wait_pending(n_stages - 2);             // page i has landed (this thread's copies) ...
            __syncthreads();                                 // ... and everyone else's; the stage of page i - 1 is free
            const int ahead = i + n_stages - 1;
            if (ahead < n_pg) stage_page(walk.page(pg_lo + ahead), next_page, ahead % n_stages);
            cp_async_commit();
            if (ahead + 1 < n_pg) next_page = bt[walk.page(pg_lo + ahead + 1)];
            const int pg = walk.page(pg_lo + i);
            const bf16* Ks = reinterpret_cast<const bf16*>(smraw + (size_t)(i % n_stages) * stage_bytes);
            const bf16* Vs = Ks + P3_PAGE * ldk;
            const float* Ps = reinterpret_cast<const float*>(Vs + P3_PAGE * ldv);
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
            const bf16* krow = Ks + (warp * 16 + (lane & 7) + 8 * (lane >> 4)) * ldk + 8 * ((lane >> 3) & 1);
#pragma unroll
            for (int t = 0; t < DK; t++) {
                if (t * 16 < d) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(krow + t * 16));
                    mma_bf16_16816(s[0], qf[t], b0, b1);
                    mma_bf16_16816(s[1], qf[t], b2, b3);
                }
            }
            float mx0 = -FLT_MAX, mx1 = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int col = warp * 16 + j * 8 + tig * 2 + (e & 1);
                    const int kpos = pg * P3_PAGE + col, dist = pos - kpos;
                    const bool vis = (kpos >= first || kpos < walk.keep) && dist >= 0 && ((e < 2) ? gid : gid + 8) < nr;
                    float v = -FLT_MAX;
                    if (vis) v = fmaf(s[j][e], scale2, has_pen ? -LOG2E * Ps[((e < 2) ? prow0 : prow1) + col] : 0.f);
                    s[j][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = sig ? 0.f : fmaxf(m0, mx0), n1 = sig ? 0.f : fmaxf(m1, mx1);
            const float c0 = exp2f(m0 - n0), c1 = exp2f(m1 - n1);
            m0 = n0; m1 = n1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = s[j][e];
                    const float p = v <= -FLT_MAX ? 0.f : sig ? 1.0f / (1.0f + exp2f(-(v + ((e < 2) ? sb0 : sb1)))) : exp2f(v - ((e < 2) ? n0 : n1));
                    s[j][e] = p;
                    if (e < 2) ps0 += p; else ps1 += p;
                }
            l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
            if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
#pragma unroll
                for (int n = 0; n < DN; n++) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]); pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]); pa[3] = pack_bf16(s[1][2], s[1][3]);
            const bf16* vrow = v_in_k ? Ks + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldk + 8 * (lane >> 4) + vc0
                                      : Vs + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * ldv + 8 * (lane >> 4);
#pragma unroll
            for (int n = 0; n < DN; n += 2) {
                if (n * 8 < dv) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(vrow + n * 8));
                    mma_bf16_16816(o[n], pa, b0, b1);
                    if (n + 1 < DN) mma_bf16_16816(o[n + 1], pa, b2, b3);
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();                                     // the ring is drained and read: its memory becomes the merge buffer
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        if (tig == 0) {
            Ms[warp * 16 + gid] = m0; Ms[warp * 16 + gid + 8] = m1;
            Ls[warp * 16 + gid] = l0; Ls[warp * 16 + gid + 8] = l1;
        }
#pragma unroll
        for (int n = 0; n < DN; n++) {
            const int c = n * 8 + tig * 2;
            if (c < dv) {
                float* w0 = Os + (size_t)(warp * 16 + gid) * dv + c;
                float* w1 = Os + (size_t)(warp * 16 + gid + 8) * dv + c;
                w0[0] = o[n][0]; w0[1] = o[n][1]; w1[0] = o[n][2]; w1[1] = o[n][3];
            }
        }
        __syncthreads();
        for (int i = tid; i < nr * dv; i += 128) {
            const int r = i / dv, c = i % dv;
            float M = -FLT_MAX;
#pragma unroll
            for (int w = 0; w < 4; w++) M = fmaxf(M, Ms[w * 16 + r]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float f = Ls[w * 16 + r] > 0.f ? exp2f(Ms[w * 16 + r] - M) : 0.f;
                L = fmaf(Ls[w * 16 + r], f, L);
                acc = fmaf(Os[(size_t)(w * 16 + r) * dv + c], f, acc);
            }
            if (n_splits == 1) {
                const float gate = (a.gate ? a.gate[(size_t)row * a.n_heads + hb + r] : 1.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
                const size_t oc = (size_t)(hb + r) * a.vdim + vc0 + c;
                ((bf16*)a.out)[(size_t)row * a.ld_out + oc] = __float2bfloat16_rn(L > 0.f ? acc * gate / (sig ? 1.f : L) * elem_gate(a, row, oc) : 0.f);
            } else {
                float* w = a.ws + (((size_t)blockIdx.x * a.n_heads + hb + r) * n_splits + split) * (a.vdim + 2);
                if (c == 0 && vc0 == 0) { w[0] = M; w[1] = L; }            // every column block forms the same maximum and sum
                w[2 + vc0 + c] = acc;
            }
        }
    }
}

// combine the slices of one (request, head): out = gate * sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M)
// (base2: the slices' maxima are in the base-2 domain, as the tensor-core decode kernel keeps them)
template <typename AT>
__global__ void attn_window_merge_kernel(p3_attn_window_args a, int n_splits, int base2) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    auto ex = [base2](float x) { return base2 ? exp2f(x) : expf(x); };
    const int t = blockIdx.x / a.n_heads, h = blockIdx.x % a.n_heads, dv = a.vdim;
    const int row = reinterpret_cast<const int4*>(a.tiles)[t].x;
    const float* w = a.ws + ((size_t)t * a.n_heads + h) * n_splits * (dv + 2);
    const float gate = (a.gate ? a.gate[(size_t)row * a.n_heads + h] : 1.f) * (a.out_scale != 0.f ? a.out_scale : 1.f);
    const bool sig = a.sig_bias != nullptr;                  // sigmoid weights: the slices' vectors add up, nothing divides
    float M = -FLT_MAX;
#pragma unroll 4
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, w[(size_t)s * (dv + 2)]);
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float L = 0.f, o = 0.f;                              // every thread forms the denominator itself: the loads of all slices are independent
#pragma unroll 4
        for (int s = 0; s < n_splits; s++) {
            const float* ws = w + (size_t)s * (dv + 2);
            const float ms = ws[0], ls = ws[1], os = ws[2 + c];
            const float f = ls > 0.f ? ex(ms - M) : 0.f;
            L = fmaf(ls, f, L);
            o = fmaf(os, f, o);
        }
        const size_t oc = (size_t)h * dv + c;
        stv((AT*)a.out + (size_t)row * a.ld_out + oc, L > 0.f ? o * gate / (sig ? 1.f : L) * elem_gate(a, row, oc) : 0.f);
    }
}

int check_args(const p3_attn_window_args* a, const char* who) {
    P3_CHECK_ARG(a && a->q && a->k_pool && a->v_pool && a->block_table && a->out && a->tiles, "%s: null argument", who);
    P3_CHECK_ARG(a->n_heads >= 1 && a->n_kv >= 1 && a->n_heads % a->n_kv == 0, "%s: heads must be a multiple of kv heads", who);
    P3_CHECK_ARG(a->dim >= 1 && a->dim <= 4096 && a->vdim >= 1 && a->vdim <= 4096, "%s: head sizes must be in [1, 4096]", who);
    P3_CHECK_ARG(!a->penalty || a->n_penalty >= 1, "%s: empty penalty table", who);
    P3_CHECK_ARG(a->act_f32 == a->cache_f32, "%s: activations and cache must both be fp32 or both bf16", who);
    P3_CHECK_ARG(a->v_ld == 0 || a->v_ld >= a->vdim, "%s: the value row pitch must hold a value row", who);
    P3_CHECK_ARG(a->keep_first >= 0, "%s: keep_first must not be negative", who);
    P3_CHECK_ARG(!a->sig_bias || !a->sink, "%s: sigmoid weights have no denominator for a sink", who);
    return 0;
}

template <typename K>
int set_smem(K kernel, size_t bytes, const char* who) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        P3_CHECK_ARG(e == cudaSuccess, "%s: shared memory attribute: %s", who, cudaGetErrorString(e));
    }
    return 0;
}

template <typename AT, typename CT>
int launch_prefill(const p3_attn_window_args* a, cudaStream_t st) {
    const int dc = a->dim < WIDE ? a->dim : WIDE, dp = (dc + 3) & ~3, dvb = a->vdim < WIDE ? a->vdim : WIDE;
    const size_t bytes = sizeof(float) * ((size_t)BQ * dp + (size_t)P3_PAGE * (dp + 1) + (size_t)P3_PAGE * dvb + (size_t)BQ * (P3_PAGE + 4));
    const dim3 grid((unsigned)a->n_tiles, (unsigned)a->n_heads, (unsigned)((a->vdim + WIDE - 1) / WIDE));
    const int c = (dvb + 31) / 32;
#define GO(N)                                                                                              \
    do { if (set_smem(attn_window_prefill_kernel<AT, CT, N>, bytes, "attn_window_prefill")) return -1;      \
         p3_launch_pdl(attn_window_prefill_kernel<AT, CT, N>, dim3(grid), dim3(WARPS * 32), (size_t)(bytes), st, *a); } while (0)
    if (c <= 1) GO(1); else if (c <= 2) GO(2); else if (c <= 4) GO(4); else GO(8);
#undef GO
    return 0;
}

template <typename AT, typename CT>
int launch_decode(const p3_attn_window_args* a, cudaStream_t st) {
    const int dvb = a->vdim < WIDE ? a->vdim : WIDE, parts = (a->vdim + WIDE - 1) / WIDE;
    const size_t bytes = sizeof(float) * ((size_t)RMAX * a->dim + 2 * DW * RMAX + (size_t)DW * RMAX * dvb);
    const int ns = a->n_splits > 1 ? a->n_splits : 1;
    const dim3 grid((unsigned)a->n_tiles, (unsigned)(a->n_kv * parts), (unsigned)ns);
    const int cv = (dvb + 31) / 32;
#define GO(NV)                                                                                             \
    do { if (set_smem(attn_window_decode_kernel<AT, CT, NV>, bytes, "attn_window_decode")) return -1;       \
         p3_launch_pdl(attn_window_decode_kernel<AT, CT, NV>, dim3(grid), dim3(DW * 32), (size_t)(bytes), st, *a, parts); } while (0)
    if (cv <= 1) GO(1); else if (cv <= 2) GO(2); else if (cv <= 4) GO(4); else GO(8);
#undef GO
    if (ns > 1) p3_launch_pdl(attn_window_merge_kernel<AT>, dim3((unsigned)(a->n_tiles * a->n_heads)), dim3(64), (size_t)(0), st, *a, ns, 0);
    return 0;
}
}  // namespace

static bool prefill_mma_ok(const p3_attn_window_args* a) {
    static int off = -1;
    if (off < 0) { const char* e = getenv("P3_ATTN_WINDOW_MMA"); off = (e && e[0] == '0') ? 1 : 0; }
    return !off && !a->act_f32 && a->dim % 16 == 0 && a->vdim % 8 == 0 && a->dim <= 256 && a->vdim <= 256 &&
           a->ld_q % 2 == 0 && a->ld_out % 2 == 0 && ((uintptr_t)a->q & 3) == 0 && ((uintptr_t)a->out & 3) == 0 &&
           ((uintptr_t)a->k_pool & 15) == 0 && ((uintptr_t)a->v_pool & 15) == 0 && a->v_ld % 8 == 0;
}

static int launch_prefill_mma(const p3_attn_window_args* a, cudaStream_t st) {
    // key rows above 128 numbers: the <16, 16> variant, values in column blocks of 128 (grid.z), each CTA forms the scores itself
    const bool wide = a->dim > 128 || a->vdim > 128;
    const int vcols = wide ? 128 : (a->dim <= 64 && a->vdim <= 64 ? 64 : 128), dvs = a->vdim < vcols ? a->vdim : vcols;
    const size_t bytes = 2 * (sizeof(bf16) * P3_PAGE * (size_t)(a->dim + 8 + dvs + 8) + 128 * sizeof(float));   // two stages
    const dim3 grid((unsigned)a->n_tiles, (unsigned)a->n_heads, (unsigned)((a->vdim + vcols - 1) / vcols));
#define GO(DK, DN, MINB)                                                                                        \
    do { if (a->sig_bias) {                                                                                      \
             if (set_smem(attn_window_prefill_mma_kernel<DK, DN, MINB, true>, bytes, "attn_window_prefill")) return -1;       \
             p3_launch_pdl(attn_window_prefill_mma_kernel<DK, DN, MINB, true>, dim3(grid), dim3(128), (size_t)(bytes), st, *a);   \
         } else {                                                                                                \
             if (set_smem(attn_window_prefill_mma_kernel<DK, DN, MINB, false>, bytes, "attn_window_prefill")) return -1;      \
             p3_launch_pdl(attn_window_prefill_mma_kernel<DK, DN, MINB, false>, dim3(grid), dim3(128), (size_t)(bytes), st, *a);  \
         } } while (0)
    if (wide) GO(16, 16, 2);
    else if (a->dim <= 64 && a->vdim <= 64) GO(4, 8, 3);
    else GO(8, 16, 3);
#undef GO
    return 0;
}

static int launch_decode_mma(const p3_attn_window_args* a, cudaStream_t st) {
    const int rep = a->n_heads / a->n_kv, pr = rep < 16 ? rep : 16;
    const bool wide = a->dim > 128 || a->vdim > 128;
    const int vcols = wide ? 128 : (a->dim <= 64 && a->vdim <= 64 ? 64 : 128), dvs = a->vdim < vcols ? a->vdim : vcols;
    const int parts = (a->vdim + vcols - 1) / vcols;
    const size_t stage = sizeof(bf16) * P3_PAGE * (size_t)(a->dim + 8 + dvs + 8) + sizeof(float) * P3_PAGE * (size_t)pr;
    // as many stages as leave room for two CTAs per SM (227 KB, 1 KB reserved per CTA); the merge buffer fits two stages
    int nst = (int)((227 * 1024 / 2 - 1024) / stage);
    nst = nst < 2 ? 2 : (nst > DEC_MAX_STAGES ? DEC_MAX_STAGES : nst);
    const size_t bytes = nst * stage;
    const int ns = a->n_splits > 1 ? a->n_splits : 1;
    const dim3 grid((unsigned)a->n_tiles, (unsigned)(a->n_kv * parts), (unsigned)ns);
    if (wide) {
        if (set_smem(attn_window_decode_mma_kernel<16, 16>, bytes, "attn_window_decode")) return -1;
        p3_launch_pdl(attn_window_decode_mma_kernel<16, 16>, dim3(grid), dim3(128), (size_t)(bytes), st, *a, nst, parts);
    } else if (a->dim <= 64 && a->vdim <= 64) {
        if (set_smem(attn_window_decode_mma_kernel<4, 8>, bytes, "attn_window_decode")) return -1;
        p3_launch_pdl(attn_window_decode_mma_kernel<4, 8>, dim3(grid), dim3(128), (size_t)(bytes), st, *a, nst, parts);
    } else {
        if (set_smem(attn_window_decode_mma_kernel<8, 16>, bytes, "attn_window_decode")) return -1;
        p3_launch_pdl(attn_window_decode_mma_kernel<8, 16>, dim3(grid), dim3(128), (size_t)(bytes), st, *a, nst, parts);
    }
    if (ns > 1) p3_launch_pdl(attn_window_merge_kernel<bf16>, dim3((unsigned)(a->n_tiles * a->n_heads)), dim3(64), (size_t)(0), st, *a, ns, 1);
    return 0;
}

/* rows per tile the launch accepts: 64 on the tensor-core path, 32 otherwise */
extern "C" int p3_attn_window_tile_rows(const p3_attn_window_args* a) { return (a && prefill_mma_ok(a)) ? 64 : BQ; }

extern "C" int p3_attn_window_prefill(const p3_attn_window_args* a, cudaStream_t st) {
    if (check_args(a, "attn_window_prefill")) return -1;
    if (a->n_tiles == 0) return 0;
    const int rc = prefill_mma_ok(a) ? launch_prefill_mma(a, st)
                 : a->act_f32 ? launch_prefill<float, float>(a, st) : launch_prefill<bf16, bf16>(a, st);
    if (rc) return rc;
    P3_CHECK_LAUNCH("attn_window_prefill");
    return 0;
}

extern "C" int p3_attn_window_decode(const p3_attn_window_args* a, cudaStream_t st) {
    if (check_args(a, "attn_window_decode")) return -1;
    P3_CHECK_ARG(a->n_splits <= 1 || a->ws, "attn_window_decode: several key slices need the workspace");
    P3_CHECK_ARG(a->n_splits <= 65535, "attn_window_decode: too many key slices");
    if (a->n_tiles == 0) return 0;
    const int rc = prefill_mma_ok(a) ? launch_decode_mma(a, st)
                 : a->act_f32 ? launch_decode<float, float>(a, st) : launch_decode<bf16, bf16>(a, st);
    if (rc) return rc;
    P3_CHECK_LAUNCH("attn_window_decode");
    return 0;
}
