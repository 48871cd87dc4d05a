// Recurrent mixers that carry a state per sequence slot instead of a key/value cache.
//
// Matrix memory (the mLSTM cell of xLSTM: Beck et al., "xLSTM: Extended Long Short-Term Memory"). Per head a memory S [dim][vdim],
// a normaliser n [dim] and a stabiliser m (0 at the start of a sequence). With log gates a_t (input) and b_t (forget):
//     m_t = max(b_t + m_(t-1), a_t)
//     S_t = e^(b_t + m_(t-1) - m_t) S_(t-1) + e^(a_t - m_t) k_t v_t^T        n_t alike with k_t alone
//     y_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
// Both exponents are <= 0 by the choice of m_t. Everything here is fp32: the gates and their logarithms, the state and the sums.
//
//   matrix_memory_scan_kernel   token by token. One CTA = one sequence of the step x one head x a block of value columns. A thread of
//                               the four main warps owns one or two columns and a slice of the dim rows of S, in registers for the
//                               whole step; a warp is RS row slices x 32 / RS lanes, so a column's sum over the rows is one or two
//                               shuffles and no barrier separates two tokens. q, k, v of 32 tokens are staged in shared memory at
//                               a time by async copies, one round ahead of the arithmetic (k and q rows are read as 16-byte
//                               broadcasts). A fifth warp turns the gate pre-activations of the next round into log gates, walks
//                               the stabiliser through them (the only serial part: one add and one max per token) and leaves
//                               e^(b + m' - m), e^(a - m) and e^(-m) of every token in shared memory; in the CTA of the first
//                               column block a sixth warp carries the normaliser n and writes the denominators
//                               max(|n . q|, e^(-m)) + 1e-6. The main warps write numerators S^T q; headnorm_gate_kernel divides.
//                               The shape of a warp (row slices, columns per lane) trades parallelism against shared-memory
//                               traffic and is chosen per launch; the arithmetic of a token is the same for every choice and does
//                               not depend on how the sequence was cut into steps, so a prompt fed in portions, or token by token,
//                               leaves bit-identical states and outputs. State of a head: S [dim][vdim], n [dim], then one copy of
//                               m per 32 value columns: every CTA needs m at its start and the first CTA to finish must not
//                               overwrite what another still has to read, so a CTA reads the copy of its first 32 columns and
//                               rewrites those of all its columns.
//   headnorm_gate_kernel        y / rms(y over the head) * gain * sigmoid(gate logits) * scale -> activation type (the gate may also
//                               be silu, the gain one vector shared by the heads)
//
// Gated linear attention (Yang et al., "Gated Linear Attention Transformers with Hardware-Efficient Training"). Per head a state
// S [dim][vdim] that starts at zero, with one decay per key channel and token:
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        y_t = S_t^T q_t        a_t = sigmoid(z_t)^(1/tau) = exp(logsigmoid(z_t) / tau)
//   gla_decay_kernel            decay logits of all rows of the step -> decays, in place (one pass at memory speed)
//   gla_scan_kernel             the matrix-memory scan's layout (columns of S in registers, rounds of staged tokens, async copies one
//                               round ahead) with a staged row of decays beside every k and q row. There is no normaliser and no
//                               stabiliser (every factor is in (0, 1]), so all four warps own columns. As there, a token's
//                               arithmetic does not depend on how the sequence was cut into steps.
#include "common.cuh"
#include "../../include/phi3_b200.h"
#include <cfloat>

namespace {
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int MM_TB = 32;        // tokens staged per round (16 for rows above 256 numbers, so that two rounds fit shared memory)
constexpr int MM_MAIN = 4;       // warps that own columns of S; one more warp for the gates, one for the normaliser
constexpr int MM_WARPS = MM_MAIN + 2;

__host__ __device__ inline int mm_m_copies(int vdim) { return (vdim + 31) / 32; }
// floats of one head's state: S [dim][vdim], n [dim], m per 32 value columns
__host__ __device__ inline int64_t mm_head_floats(int dim, int vdim) { return (int64_t)dim * vdim + dim + mm_m_copies(vdim); }

__device__ __forceinline__ float log_sigmoid(float z) {       // -softplus(-z), without overflow on either side
    return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

// 4-byte async copy global -> shared; src_bytes 0 writes zeros
__device__ __forceinline__ void cp_async4z(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

template <int DS, int RS, int NC, int TB>
__global__ void __launch_bounds__(MM_WARPS * 32) matrix_memory_scan_kernel(p3_matrix_memory_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    // a warp = RS row slices x CW lanes, every lane with NC columns (CW apart); DP: dim rounded up; NR: n rows per lane
    constexpr int CW = 32 / RS, WCOLS = CW * NC, COLS = MM_MAIN * WCOLS, DP = DS * RS, NR = (DP + 31) / 32;
    constexpr int NT = MM_WARPS * 32;
    // a staged q / k row keeps its RS slices 4 floats apart (pitch DPP): the 16-byte reads of a warp's slices then fall into
    // different banks and one read serves all of them
    constexpr int DPP = DP + 4 * RS;
    constexpr int ROUND = TB * (2 * DPP + COLS + 3);      // floats of one staged round
    auto at_row = [](int c) { return c + 4 * (c / DS); };    // where number c of a row lives
    extern __shared__ __align__(16) float sm[];
    const int d = a.dim, dv = a.vdim, H = a.n_heads;
    // two rounds in flight: [q [TB][DP] (zeros beyond dim) | k alike | v [TB][COLS] | e^(a - m) | e^(b + m' - m) | e^(-m)]
    const int4 rec = reinterpret_cast<const int4*>(a.seqs)[blockIdx.x];
    const int row0 = rec.x, n_tok = rec.y, slot = rec.z, pos0 = rec.w;
    const int hd = blockIdx.y, vb = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool fresh = pos0 == 0, main = warp < MM_MAIN, gate_warp = warp == MM_MAIN, first_block = vb == 0;
    float* Sg = a.state + ((size_t)slot * H + hd) * mm_head_floats(d, dv);
    float* ng = Sg + (size_t)d * dv;
    float* mg = ng + d;
    const int col = vb * COLS + warp * WCOLS + lane % CW, d0 = (lane / CW) * DS;   // first of this lane's columns
    float S[NC][DS], nr[NR];
    float m = 0.f;
    if (main) {
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int j = 0; j < DS; j++)
                S[c][j] = (!fresh && col + c * CW < dv && d0 + j < d) ? Sg[(size_t)(d0 + j) * dv + col + c * CW] : 0.f;
    } else if (gate_warp) {
        if (!fresh) m = mg[vb * (COLS / 32)];
    } else {
#pragma unroll
        for (int r = 0; r < NR; r++) nr[r] = (!fresh && first_block && lane * NR + r < d) ? ng[lane * NR + r] : 0.f;
    }
    const float inv_cap = 1.0f / a.gate_cap;
    const bool vec = d % 4 == 0 && a.ld_proj % 4 == 0 && a.q_off % 4 == 0 && a.k_off % 4 == 0 && ((uintptr_t)a.proj & 15) == 0;

    // all threads: start the copies of the round that begins at token t0 into buffer `buf` (q, k, v as projected; q is scaled when
    // the sums are written)
    auto stage = [&](int t0, int buf) {
        const int nb = min(TB, n_tok - t0);
        float* qs = sm + buf * ROUND;
        float* ks = qs + TB * DPP;
        float* vs = ks + TB * DPP;
        if (vec) {
            for (int i = tid; i < nb * (DP / 4); i += NT) {
                const int tt = i / (DP / 4), c = (i - tt * (DP / 4)) * 4;
                const float* pr = a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + (size_t)hd * d + (c < d ? c : 0);
                cp_async16(smem_u32(qs + tt * DPP + at_row(c)), pr + a.q_off, c < d ? 16 : 0);
                cp_async16(smem_u32(ks + tt * DPP + at_row(c)), pr + a.k_off, c < d ? 16 : 0);
            }
        } else {
            for (int i = tid; i < nb * DP; i += NT) {
                const int tt = i / DP, c = i - tt * DP;
                const float* pr = a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + (size_t)hd * d + (c < d ? c : 0);
                cp_async4z(smem_u32(qs + tt * DPP + at_row(c)), pr + a.q_off, c < d ? 4 : 0);
                cp_async4z(smem_u32(ks + tt * DPP + at_row(c)), pr + a.k_off, c < d ? 4 : 0);
            }
        }
        for (int i = tid; i < nb * COLS; i += NT) {
            const int tt = i / COLS, c = vb * COLS + (i - tt * COLS);
            cp_async4z(smem_u32(vs + i), a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + a.v_off + (size_t)hd * dv + (c < dv ? c : 0), c < dv ? 4 : 0);
        }
    };
    // gate warp: the log gates of the round (one token per lane), the walk of the stabiliser through them (every lane walks, the
    // gates come by shuffle: one add and one max per token on the critical path), and the three factors of every token
    auto gates = [&](int t0, int buf) {
        const int nb = min(TB, n_tok - t0);
        float* ga = sm + buf * ROUND + TB * (2 * DPP + COLS);
        float* gb = ga + TB;
        float* gm = gb + TB;
        float at = 0.f, bt = 0.f;
        if (lane < nb) {
            const float* pr = a.proj + (size_t)(row0 + t0 + lane) * a.ld_proj + hd;
            at = a.gate_cap * tanhf((pr[a.i_off] + a.i_bias[hd]) * inv_cap);
            bt = log_sigmoid(a.gate_cap * tanhf((pr[a.f_off] + a.f_bias[hd]) * inv_cap));
        }
        float m_before = 0.f, m_after = 0.f;
#pragma unroll
        for (int tt = 0; tt < TB; tt++) {
            const float as = __shfl_sync(0xffffffffu, at, tt), bs = __shfl_sync(0xffffffffu, bt, tt);
            if (tt < nb) {
                const float mn = fmaxf(bs + m, as);
                if (lane == tt) { m_before = m; m_after = mn; }
                m = mn;
            }
        }
        if (lane < nb) {
            gb[lane] = expf(bt + m_before - m_after);
            ga[lane] = expf(at - m_after);
            gm[lane] = expf(-m_after);
        }
    };

    stage(0, 0);
    cp_async_commit();
    if (gate_warp) gates(0, 0);
    for (int t0 = 0, r = 0; t0 < n_tok; t0 += TB, r++) {
        const int nb = min(TB, n_tok - t0), buf = r & 1;
        cp_async_wait<0>();                                  // this thread's copies of round r have landed ...
        __syncthreads();                                     // ... and everyone's, with the round's factors; round r - 1 is consumed
        if (t0 + TB < n_tok) stage(t0 + TB, buf ^ 1);
        cp_async_commit();
        const float* qs = sm + buf * ROUND;
        const float* ks = qs + TB * DPP;
        const float* vs = ks + TB * DPP;
        const float* ga = vs + TB * COLS;
        const float* gb = ga + TB;
        const float* gm = gb + TB;
        if (main) {
#pragma unroll 2
            for (int tt = 0; tt < nb; tt++) {
                const float keep = gb[tt], take = ga[tt];
                float tv[NC], acc[NC][4];
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    tv[c] = take * vs[tt * COLS + warp * WCOLS + lane % CW + c * CW];
                    acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
                }
                const float4* kq = reinterpret_cast<const float4*>(ks + tt * DPP + at_row(d0));
                const float4* qq = reinterpret_cast<const float4*>(qs + tt * DPP + at_row(d0));
#pragma unroll
                for (int j = 0; j < DS; j += 4) {
                    const float4 kk = kq[j / 4], qv = qq[j / 4];
#pragma unroll
                    for (int c = 0; c < NC; c++) {
                        S[c][j] = fmaf(kk.x, tv[c], keep * S[c][j]);         acc[c][0] = fmaf(S[c][j], qv.x, acc[c][0]);
                        S[c][j + 1] = fmaf(kk.y, tv[c], keep * S[c][j + 1]); acc[c][1] = fmaf(S[c][j + 1], qv.y, acc[c][1]);
                        S[c][j + 2] = fmaf(kk.z, tv[c], keep * S[c][j + 2]); acc[c][2] = fmaf(S[c][j + 2], qv.z, acc[c][2]);
                        S[c][j + 3] = fmaf(kk.w, tv[c], keep * S[c][j + 3]); acc[c][3] = fmaf(S[c][j + 3], qv.w, acc[c][3]);
                    }
                }
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    float y = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
                    if (RS >= 2) y += __shfl_xor_sync(0xffffffffu, y, CW);
                    if (RS >= 4) y += __shfl_xor_sync(0xffffffffu, y, 2 * CW);
                    if (lane < CW && col + c * CW < dv)
                        a.out[(size_t)(row0 + t0 + tt) * a.ld_out + (size_t)hd * dv + col + c * CW] = y * a.q_scale;
                }
            }
        } else if (gate_warp) {
            if (t0 + TB < n_tok) gates(t0 + TB, buf ^ 1);      // the next round's factors, while the main warps work on this one
        } else {
            if (first_block) {
#pragma unroll 4
                for (int tt = 0; tt < nb; tt++) {
                    const float keep = gb[tt], take = ga[tt];
                    float nq = 0.f;
#pragma unroll
                    for (int rr = 0; rr < NR; rr++) {
                        if (lane * NR + rr < d) {
                            nr[rr] = fmaf(take, ks[tt * DPP + at_row(lane * NR + rr)], keep * nr[rr]);
                            nq = fmaf(nr[rr], qs[tt * DPP + at_row(lane * NR + rr)], nq);
                        }
                    }
                    nq = warp_sum(nq);
                    if (lane == 0) a.den[(size_t)(row0 + t0 + tt) * H + hd] = fmaxf(fabsf(nq * a.q_scale), gm[tt]) + 1e-6f;
                }
            }
        }
    }
    if (main) {
#pragma unroll
        for (int c = 0; c < NC; c++)
#pragma unroll
            for (int j = 0; j < DS; j++)
                if (col + c * CW < dv && d0 + j < d) Sg[(size_t)(d0 + j) * dv + col + c * CW] = S[c][j];
    } else if (gate_warp) {
        if (lane == 0)
            for (int c = vb * (COLS / 32); c < min((vb + 1) * (COLS / 32), mm_m_copies(dv)); c++) mg[c] = m;
    } else if (first_block) {
#pragma unroll
        for (int r = 0; r < NR; r++) if (lane * NR + r < d) ng[lane * NR + r] = nr[r];
    }
}

__host__ __device__ inline int64_t gla_head_floats(int dim, int vdim) { return (int64_t)dim * vdim; }

// decay logits -> decays, in place: z <- exp(logsigmoid(z + bias) * inv_tau), n numbers per row
__global__ void gla_decay_kernel(float* __restrict__ z, int64_t ld_z, const float* __restrict__ bias, int64_t T, int n, float inv_tau, int vec) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t step = (int64_t)gridDim.x * blockDim.x, me = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (vec) {
        const int nq = n / 4;
        for (int64_t i = me; i < T * nq; i += step) {
            const int64_t t = i / nq;
            const int c = (int)(i - t * nq) * 4;
            float4 v = *reinterpret_cast<float4*>(z + t * ld_z + c);
            const float4 b = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            v.x = expf(log_sigmoid(v.x + b.x) * inv_tau); v.y = expf(log_sigmoid(v.y + b.y) * inv_tau);
            v.z = expf(log_sigmoid(v.z + b.z) * inv_tau); v.w = expf(log_sigmoid(v.w + b.w) * inv_tau);
            *reinterpret_cast<float4*>(z + t * ld_z + c) = v;
        }
    } else {
        for (int64_t i = me; i < T * n; i += step) {
            const int64_t t = i / n;
            const int c = (int)(i - t * n);
            z[t * ld_z + c] = expf(log_sigmoid(z[t * ld_z + c] + (bias ? bias[c] : 0.f)) * inv_tau);
        }
    }
}

// the same with the logits formed on the way: z[t][c] = exp(logsigmoid(bias[c] + sum_r lr[t][r] a2[c][r]) * inv_tau). A thread owns
// one column with its a2 row in registers and walks the tokens of its CTA's chunk, whose low-rank vectors are staged in shared
// memory 32 tokens at a time (every thread reads the same number: a broadcast); the FMA chain runs in ascending r.
constexpr int GD_TOK = 32;
template <int RMAX>
__global__ void __launch_bounds__(256) gla_decay_lowrank_kernel(float* __restrict__ z, int64_t ld_z, const float* __restrict__ bias,
                                                                const float* __restrict__ lr, int64_t ld_lr, const float* __restrict__ a2,
                                                                int rank, int64_t T, int n, float inv_tau, int tok_per_cta) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ float lrs[GD_TOK][RMAX];
    const int c = blockIdx.x * 256 + threadIdx.x;
    float w[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; r++) w[r] = (c < n && r < rank) ? a2[(size_t)c * rank + r] : 0.f;
    const float b = (c < n && bias) ? bias[c] : 0.f;
    const int64_t t_end = min(T, (int64_t)(blockIdx.y + 1) * tok_per_cta);
    for (int64_t t0 = (int64_t)blockIdx.y * tok_per_cta; t0 < t_end; t0 += GD_TOK) {
        const int nb = (int)min((int64_t)GD_TOK, t_end - t0);
        __syncthreads();                                     // the round before is consumed
        for (int i = threadIdx.x; i < nb * RMAX; i += 256) {
            const int tt = i / RMAX, r = i - tt * RMAX;
            lrs[tt][r] = r < rank ? lr[(t0 + tt) * ld_lr + r] : 0.f;
        }
        __syncthreads();
        if (c < n) {
            for (int tt = 0; tt < nb; tt++) {
                float acc = b;
#pragma unroll
                for (int r = 0; r < RMAX; r++) acc = fmaf(lrs[tt][r], w[r], acc);
                z[(t0 + tt) * ld_z + c] = expf(log_sigmoid(acc) * inv_tau);
            }
        }
    }
}

constexpr int GLA_WARPS = 4;     // every warp owns columns of S

template <int DS, int RS, int NC, int TB>
__global__ void __launch_bounds__(GLA_WARPS * 32) gla_scan_kernel(p3_gla_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    // a warp = RS row slices x CW lanes, every lane with NC columns (CW apart); DP: dim rounded up
    constexpr int CW = 32 / RS, WCOLS = CW * NC, COLS = GLA_WARPS * WCOLS, DP = DS * RS;
    constexpr int NT = GLA_WARPS * 32;
    constexpr int DPP = DP + 4 * RS;                         // pitch of a staged row: its RS slices 4 floats apart (bank spread)
    constexpr int ROUND = TB * (3 * DPP + COLS);             // floats of one staged round
    auto at_row = [](int c) { return c + 4 * (c / DS); };    // where number c of a row lives
    extern __shared__ __align__(16) float sm[];
    const int d = a.dim, dv = a.vdim, H = a.n_heads;
    // two rounds in flight: [q [TB][DPP] (zeros beyond dim) | k alike | decays alike | v [TB][COLS]]
    const int4 rec = reinterpret_cast<const int4*>(a.seqs)[blockIdx.x];
    const int row0 = rec.x, n_tok = rec.y, slot = rec.z, pos0 = rec.w;
    const int hd = blockIdx.y, vb = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool fresh = pos0 == 0;
    float* Sg = a.state + ((size_t)slot * H + hd) * gla_head_floats(d, dv);
    const int col = vb * COLS + warp * WCOLS + lane % CW, d0 = (lane / CW) * DS;   // first of this lane's columns
    float S[NC][DS];
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int j = 0; j < DS; j++)
            S[c][j] = (!fresh && col + c * CW < dv && d0 + j < d) ? Sg[(size_t)(d0 + j) * dv + col + c * CW] : 0.f;
    const bool vec = d % 4 == 0 && a.ld_proj % 4 == 0 && a.q_off % 4 == 0 && a.k_off % 4 == 0 && ((uintptr_t)a.proj & 15) == 0 &&
                     a.ld_z % 4 == 0 && ((uintptr_t)a.z & 15) == 0;

    // all threads: start the copies of the round that begins at token t0 into buffer `buf` (q is scaled when the sums are written)
    auto stage = [&](int t0, int buf) {
        const int nb = min(TB, n_tok - t0);
        float* qs = sm + buf * ROUND;
        float* ks = qs + TB * DPP;
        float* as = ks + TB * DPP;
        float* vs = as + TB * DPP;
        if (vec) {
            for (int i = tid; i < nb * (DP / 4); i += NT) {
                const int tt = i / (DP / 4), c = (i - tt * (DP / 4)) * 4;
                const float* pr = a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + (size_t)hd * d + (c < d ? c : 0);
                cp_async16(smem_u32(qs + tt * DPP + at_row(c)), pr + a.q_off, c < d ? 16 : 0);
                cp_async16(smem_u32(ks + tt * DPP + at_row(c)), pr + a.k_off, c < d ? 16 : 0);
                cp_async16(smem_u32(as + tt * DPP + at_row(c)), a.z + (size_t)(row0 + t0 + tt) * a.ld_z + (size_t)hd * d + (c < d ? c : 0), c < d ? 16 : 0);
            }
        } else {
            for (int i = tid; i < nb * DP; i += NT) {
                const int tt = i / DP, c = i - tt * DP;
                const float* pr = a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + (size_t)hd * d + (c < d ? c : 0);
                cp_async4z(smem_u32(qs + tt * DPP + at_row(c)), pr + a.q_off, c < d ? 4 : 0);
                cp_async4z(smem_u32(ks + tt * DPP + at_row(c)), pr + a.k_off, c < d ? 4 : 0);
                cp_async4z(smem_u32(as + tt * DPP + at_row(c)), a.z + (size_t)(row0 + t0 + tt) * a.ld_z + (size_t)hd * d + (c < d ? c : 0), c < d ? 4 : 0);
            }
        }
        for (int i = tid; i < nb * COLS; i += NT) {
            const int tt = i / COLS, c = vb * COLS + (i - tt * COLS);
            cp_async4z(smem_u32(vs + i), a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + a.v_off + (size_t)hd * dv + (c < dv ? c : 0), c < dv ? 4 : 0);
        }
    };

    stage(0, 0);
    cp_async_commit();
    for (int t0 = 0, r = 0; t0 < n_tok; t0 += TB, r++) {
        const int nb = min(TB, n_tok - t0), buf = r & 1;
        cp_async_wait<0>();                                  // this thread's copies of round r have landed ...
        __syncthreads();                                     // ... and everyone's; round r - 1 is consumed
        if (t0 + TB < n_tok) stage(t0 + TB, buf ^ 1);
        cp_async_commit();
        const float* qs = sm + buf * ROUND;
        const float* ks = qs + TB * DPP;
        const float* as = ks + TB * DPP;
        const float* vs = as + TB * DPP;
#pragma unroll(DS >= 128 ? 1 : 2)
        for (int tt = 0; tt < nb; tt++) {
            float tv[NC], acc[NC][4];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                tv[c] = vs[tt * COLS + warp * WCOLS + lane % CW + c * CW];
                acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
            }
            const float4* kq = reinterpret_cast<const float4*>(ks + tt * DPP + at_row(d0));
            const float4* qq = reinterpret_cast<const float4*>(qs + tt * DPP + at_row(d0));
            const float4* aq = reinterpret_cast<const float4*>(as + tt * DPP + at_row(d0));
#pragma unroll
            for (int j = 0; j < DS; j += 4) {
                const float4 kk = kq[j / 4], qv = qq[j / 4], al = aq[j / 4];
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    S[c][j] = fmaf(kk.x, tv[c], al.x * S[c][j]);         acc[c][0] = fmaf(S[c][j], qv.x, acc[c][0]);
                    S[c][j + 1] = fmaf(kk.y, tv[c], al.y * S[c][j + 1]); acc[c][1] = fmaf(S[c][j + 1], qv.y, acc[c][1]);
                    S[c][j + 2] = fmaf(kk.z, tv[c], al.z * S[c][j + 2]); acc[c][2] = fmaf(S[c][j + 2], qv.z, acc[c][2]);
                    S[c][j + 3] = fmaf(kk.w, tv[c], al.w * S[c][j + 3]); acc[c][3] = fmaf(S[c][j + 3], qv.w, acc[c][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < NC; c++) {
                float y = (acc[c][0] + acc[c][1]) + (acc[c][2] + acc[c][3]);
                if (RS >= 2) y += __shfl_xor_sync(0xffffffffu, y, CW);
                if (RS >= 4) y += __shfl_xor_sync(0xffffffffu, y, 2 * CW);
                if (lane < CW && col + c * CW < dv)
                    a.out[(size_t)(row0 + t0 + tt) * a.ld_out + (size_t)hd * dv + col + c * CW] = y * a.q_scale;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < NC; c++)
#pragma unroll
        for (int j = 0; j < DS; j++)
            if (col + c * CW < dv && d0 + j < d) Sg[(size_t)(d0 + j) * dv + col + c * CW] = S[c][j];
}

// one warp per (token, head)
template <typename AT>
__global__ void headnorm_gate_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ den, int H, int dv,
                                     const float* __restrict__ gain, int gain_shared,
                                     const float* __restrict__ gate, int64_t ld_gate, int gate_silu, float scale, float eps,
                                     AT* __restrict__ out, int64_t ldo, int64_t T) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int lane = threadIdx.x & 31;
    const int64_t job = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (job >= T * H) return;
    const int64_t t = job / H;
    const int h = (int)(job - t * H);
    const float* yr = y + t * ldy + (size_t)h * dv;
    const float dn = den ? den[t * H + h] : 1.f;             // the read-out's denominator, when the producer left numerators
    // up to 8 numbers per lane stay in registers between the statistic and the write (heads of up to 256 numbers)
    float v[8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) { const int i = lane + 32 * k; v[k] = i < dv ? yr[i] / dn : 0.f; ss = fmaf(v[k], v[k], ss); }
    for (int i = lane + 256; i < dv; i += 32) { const float u = yr[i] / dn; ss = fmaf(u, u, ss); }
    ss = warp_sum(ss);
    const float r = scale / sqrtf(ss / (float)dv + eps);
    auto gated = [&](int c) {                                // the gate of output column c: sigmoid(g), or silu(g) = g sigmoid(g)
        if (!gate) return 1.f;
        const float g = gate[t * ld_gate + c], sg = 1.0f / (1.0f + expf(-g));
        return gate_silu ? g * sg : sg;
    };
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int i = lane + 32 * k, c = h * dv + i;
        if (i < dv) stv(out + t * ldo + c, v[k] * r * gain[gain_shared ? i : c] * gated(c));
    }
    for (int i = lane + 256; i < dv; i += 32) {
        const int c = h * dv + i;
        stv(out + t * ldo + c, yr[i] / dn * r * gain[gain_shared ? i : c] * gated(c));
    }
}
template <typename K>
int set_smem_attr(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        P3_CHECK_ARG(e == cudaSuccess, "matrix_memory_scan: shared memory attribute: %s", cudaGetErrorString(e));
    }
    return 0;
}
}  // namespace

extern "C" int64_t p3_matrix_memory_state_floats(int n_heads, int dim, int vdim) { return (int64_t)n_heads * mm_head_floats(dim, vdim); }

extern "C" int p3_matrix_memory_scan(const p3_matrix_memory_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->proj && a->i_bias && a->f_bias && a->state && a->seqs && a->out && a->den, "matrix_memory_scan: null argument");
    P3_CHECK_ARG(a->n_heads >= 1 && a->dim >= 1 && a->dim <= 512 && a->vdim >= 1, "matrix_memory_scan: need heads >= 1, 1 <= dim <= 512, vdim >= 1");
    P3_CHECK_ARG(a->gate_cap > 0.f, "matrix_memory_scan: the gate cap must be positive");
    P3_CHECK_ARG(((uintptr_t)a->seqs & 15) == 0, "matrix_memory_scan: the sequence records must be 16-byte aligned");
    if (a->n_seqs == 0) return 0;
    // A warp is four row slices x eight lanes; a lane owns two columns (each k / q read from shared memory, the limit of this
    // kernel, then serves two columns) when that still leaves a CTA for every SM, else one. rs_force (tests): 2 or 4 row slices
    // with one column per lane, 8 = four slices with two columns.
    int rs = 4, nc = (int64_t)a->n_seqs * a->n_heads * ((a->vdim + 63) / 64) >= 148 ? 2 : 1;
    if (a->rs_force == 2 || a->rs_force == 4) { rs = a->rs_force; nc = 1; }
    if (a->rs_force == 8) { rs = 4; nc = 2; }
    if (a->dim > 256) { rs = 4; nc = 1; }                    // 128 rows per thread, 16 tokens per round
    const int per = (a->dim + rs - 1) / rs, ds = per <= 16 ? 16 : per <= 32 ? 32 : per <= 64 ? 64 : 128;
    const int cols = MM_MAIN * 32 / rs * nc, tb = a->dim > 256 ? 16 : MM_TB;
    const dim3 grid((unsigned)a->n_seqs, (unsigned)a->n_heads, (unsigned)((a->vdim + cols - 1) / cols));
    const size_t bytes = sizeof(float) * (size_t)2 * tb * (2 * (ds * rs + 4 * rs) + cols + 3);   // two staged rounds
#define GO(DS, RS, NC)                                                                                              \
    do { if (set_smem_attr(matrix_memory_scan_kernel<DS, RS, NC, MM_TB>, bytes)) return -1;                           \
         p3_launch_pdl(matrix_memory_scan_kernel<DS, RS, NC, MM_TB>, dim3(grid), dim3(MM_WARPS * 32), (size_t)(bytes), st, *a); } while (0)
    if (a->dim > 256) {
        if (set_smem_attr(matrix_memory_scan_kernel<128, 4, 1, 16>, bytes)) return -1;
        p3_launch_pdl(matrix_memory_scan_kernel<128, 4, 1, 16>, dim3(grid), dim3(MM_WARPS * 32), (size_t)(bytes), st, *a);
    } else if (rs == 2) { if (ds == 16) GO(16, 2, 1); else if (ds == 32) GO(32, 2, 1); else if (ds == 64) GO(64, 2, 1); else GO(128, 2, 1); }
    else if (nc == 1) { if (ds == 16) GO(16, 4, 1); else if (ds == 32) GO(32, 4, 1); else GO(64, 4, 1); }
    else { if (ds == 16) GO(16, 4, 2); else if (ds == 32) GO(32, 4, 2); else GO(64, 4, 2); }
#undef GO
    P3_CHECK_LAUNCH("matrix_memory_scan");
    return 0;
}

extern "C" int p3_headnorm_gate_x(const float* y, int64_t ldy, const float* den, int n_heads, int vdim, const float* gain, int gain_shared,
                                  const float* gate, int64_t ld_gate, int gate_silu, float scale, float eps, void* out, int64_t ldo,
                                  int out_f32, int64_t T, cudaStream_t st) {
    P3_CHECK_ARG(y && gain && out && n_heads >= 1 && vdim >= 1, "headnorm_gate: null argument");
    if (T == 0) return 0;
    const int64_t jobs = T * n_heads;
    const unsigned grid = (unsigned)((jobs + 3) / 4);
    if (out_f32) p3_launch_pdl(headnorm_gate_kernel<float>, dim3(grid), dim3(128), (size_t)(0), st, y, ldy, den, n_heads, vdim, gain, gain_shared, gate, ld_gate, gate_silu, scale, eps, (float*)out, ldo, T);
    else p3_launch_pdl(headnorm_gate_kernel<bf16>, dim3(grid), dim3(128), (size_t)(0), st, y, ldy, den, n_heads, vdim, gain, gain_shared, gate, ld_gate, gate_silu, scale, eps, (bf16*)out, ldo, T);
    P3_CHECK_LAUNCH("headnorm_gate");
    return 0;
}

extern "C" int p3_headnorm_gate(const float* y, int64_t ldy, const float* den, int n_heads, int vdim, const float* gain, const float* gate,
                                int64_t ld_gate, float scale, float eps, void* out, int64_t ldo, int out_f32, int64_t T, cudaStream_t st) {
    return p3_headnorm_gate_x(y, ldy, den, n_heads, vdim, gain, 0, gate, ld_gate, 0, scale, eps, out, ldo, out_f32, T, st);
}

extern "C" int64_t p3_gla_state_floats(int n_heads, int dim, int vdim) { return (int64_t)n_heads * gla_head_floats(dim, vdim); }

extern "C" int p3_gla_scan(const p3_gla_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->proj && a->z && a->state && a->seqs && a->out, "gla_scan: null argument");
    P3_CHECK_ARG(a->n_heads >= 1 && a->dim >= 1 && a->dim <= 512 && a->vdim >= 1, "gla_scan: need heads >= 1, 1 <= dim <= 512, vdim >= 1");
    P3_CHECK_ARG(((uintptr_t)a->seqs & 15) == 0, "gla_scan: the sequence records must be 16-byte aligned");
    P3_CHECK_ARG(a->n_rows >= 0, "gla_scan: the number of rows must not be negative");
    if (a->n_seqs == 0 || a->n_rows == 0) return 0;
    P3_CHECK_ARG(!a->lr || (a->a2 && a->rank >= 1 && a->rank <= 64), "gla_scan: the low-rank decay projection needs a2 and 1 <= rank <= 64");
    if (a->lr) {   // decays first, over all rows of the step at once, logits formed on the way: the scan then stages them like k and q
        const int n = a->n_heads * a->dim;
        const unsigned gx = (unsigned)((n + 255) / 256);
        // enough CTAs for four per SM, at least one staged round of tokens each
        int64_t per = (a->n_rows + (148 * 4 / gx)) / (148 * 4 / gx + 1);
        per = (per + GD_TOK - 1) / GD_TOK * GD_TOK;
        if (per < GD_TOK) per = GD_TOK;
        const dim3 dgrid(gx, (unsigned)((a->n_rows + per - 1) / per));
#define GD(R) p3_launch_pdl(gla_decay_lowrank_kernel<R>, dim3(dgrid), dim3(256), (size_t)(0), st, a->z, a->ld_z, a->z_bias, a->lr, a->ld_lr, \
                            a->a2, a->rank, (int64_t)a->n_rows, n, a->inv_tau, (int)per)
        if (a->rank <= 16) GD(16); else if (a->rank <= 32) GD(32); else GD(64);
#undef GD
    } else {       // decays first, over all rows of the step at once and in place
        const int n = a->n_heads * a->dim;
        const int vec = n % 4 == 0 && a->ld_z % 4 == 0 && ((uintptr_t)a->z & 15) == 0 && (!a->z_bias || ((uintptr_t)a->z_bias & 15) == 0);
        const int64_t work = (int64_t)a->n_rows * (vec ? n / 4 : n);
        const unsigned blocks = (unsigned)(work + 255) / 256 < 148u * 8 ? (unsigned)((work + 255) / 256) : 148u * 8;
        p3_launch_pdl(gla_decay_kernel, dim3(blocks ? blocks : 1), dim3(256), (size_t)(0), st, a->z, a->ld_z, a->z_bias, (int64_t)a->n_rows, n, a->inv_tau, vec);
    }
    // A warp is four row slices x eight lanes. Two columns per lane halve the shared-memory reads per FMA, which is what bounds
    // this kernel (three staged rows per token against two of the matrix memory): a CTA then takes 1.14 times as long for twice
    // the columns, so that shape wins as soon as one column per lane would need more CTAs than there are SMs.
    int rs = 4, nc = (int64_t)a->n_seqs * a->n_heads * ((a->vdim + 31) / 32) > 148 ? 2 : 1;
    if (a->rs_force == 2 || a->rs_force == 4) { rs = a->rs_force; nc = 1; }
    if (a->rs_force == 8) { rs = 4; nc = 2; }
    if (a->dim > 256) { rs = 4; nc = 1; }                    // 128 rows per thread, 16 tokens per round
    const int per = (a->dim + rs - 1) / rs, ds = per <= 16 ? 16 : per <= 32 ? 32 : per <= 64 ? 64 : 128;
    const int cols = GLA_WARPS * 32 / rs * nc, tb = a->dim > 256 ? 16 : MM_TB;
    const dim3 grid((unsigned)a->n_seqs, (unsigned)a->n_heads, (unsigned)((a->vdim + cols - 1) / cols));
    const size_t bytes = sizeof(float) * (size_t)2 * tb * (3 * (ds * rs + 4 * rs) + cols);   // two staged rounds
#define GO(DS, RS, NC)                                                                                              \
    do { if (set_smem_attr(gla_scan_kernel<DS, RS, NC, MM_TB>, bytes)) return -1;                                     \
         p3_launch_pdl(gla_scan_kernel<DS, RS, NC, MM_TB>, dim3(grid), dim3(GLA_WARPS * 32), (size_t)(bytes), st, *a); } while (0)
    if (a->dim > 256) {
        if (set_smem_attr(gla_scan_kernel<128, 4, 1, 16>, bytes)) return -1;
        p3_launch_pdl(gla_scan_kernel<128, 4, 1, 16>, dim3(grid), dim3(GLA_WARPS * 32), (size_t)(bytes), st, *a);
    } else if (rs == 2) { if (ds == 16) GO(16, 2, 1); else if (ds == 32) GO(32, 2, 1); else if (ds == 64) GO(64, 2, 1); else GO(128, 2, 1); }
    else if (nc == 1) { if (ds == 16) GO(16, 4, 1); else if (ds == 32) GO(32, 4, 1); else GO(64, 4, 1); }
    else { if (ds == 16) GO(16, 4, 2); else if (ds == 32) GO(32, 4, 2); else GO(64, 4, 2); }
#undef GO
    P3_CHECK_LAUNCH("gla_scan");
    return 0;
}
