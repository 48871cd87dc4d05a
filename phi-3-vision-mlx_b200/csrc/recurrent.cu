// Recurrent mixers that carry a state per sequence slot instead of a key/value cache.
//
// Matrix memory (the mLSTM cell of xLSTM: Beck et al., "xLSTM: Extended Long Short-Term Memory"). Per head a memory S [dim][vdim],
// a normaliser n [dim] and a stabiliser m (0 at the start of a sequence). With log gates a_t (input) and b_t (forget):
//     m_t = max(b_t + m_(t-1), a_t)
//     S_t = e^(b_t + m_(t-1) - m_t) S_(t-1) + e^(a_t - m_t) k_t v_t^T        n_t alike with k_t alone
//     y_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)
// Both exponents are <= 0 by the choice of m_t. Everything here is fp32: the gates and their logarithms, the state and the sums.
//
//   matrix_memory_scan_kernel   token by token. One CTA = one sequence of the step x one head x 32 value columns; its four warps
//                               split the dim rows of S, every thread keeps its part of one column in registers for the whole
//                               step. q, k, v and the gates of 16 tokens are staged in shared memory at a time. The arithmetic
//                               of a token does not depend on how the sequence was cut into steps, so a prompt fed in portions,
//                               or token by token, leaves bit-identical states and outputs.
//                               A CTA owns its state outright: the columns of S it covers and a private copy of n and m (every
//                               column block needs them, and a shared copy would be overwritten by the first CTA to finish
//                               while another still has to read it).
//   headnorm_gate_kernel        y / rms(y over the head) * gain * sigmoid(gate logits) * scale -> activation type
#include "common.cuh"
#include "../../include/phi3_b200.h"
#include <cfloat>

namespace {
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int MM_COLS = 32;      // value columns per CTA
constexpr int MM_WARPS = 4;      // slices of the dim rows
constexpr int MM_TB = 16;        // tokens staged per round

__host__ __device__ inline int mm_col_blocks(int vdim) { return (vdim + MM_COLS - 1) / MM_COLS; }
// floats of one head's state: S [dim][vdim], then per column block n [dim] and m
__host__ __device__ inline int64_t mm_head_floats(int dim, int vdim) { return (int64_t)dim * vdim + (int64_t)mm_col_blocks(vdim) * (dim + 1); }

__device__ __forceinline__ float log_sigmoid(float z) {       // -softplus(-z), without overflow on either side
    return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z));
}

template <int DS>
__global__ void __launch_bounds__(MM_WARPS * 32) matrix_memory_scan_kernel(p3_matrix_memory_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ __align__(16) float sm[];
    const int d = a.dim, dv = a.vdim, H = a.n_heads;
    float* qs = sm;                                          // [MM_TB][d]
    float* ks = qs + MM_TB * d;                              // [MM_TB][d]
    float* vs = ks + MM_TB * d;                              // [MM_TB][MM_COLS]
    float* ga = vs + MM_TB * MM_COLS;                        // [MM_TB] log input gates
    float* gb = ga + MM_TB;                                  // [MM_TB] log forget gates
    float* part = gb + MM_TB;                                // [2][MM_WARPS][MM_COLS] column sums of the warps' row slices
    float* npart = part + 2 * MM_WARPS * MM_COLS;            // [2][MM_WARPS] partial n . q
    const int4 rec = reinterpret_cast<const int4*>(a.seqs)[blockIdx.x];
    const int row0 = rec.x, n_tok = rec.y, slot = rec.z, pos0 = rec.w;
    const int hd = blockIdx.y, vb = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = vb * MM_COLS + lane, d0 = warp * DS;
    const bool colok = col < dv, fresh = pos0 == 0;
    float* Sg = a.state + (size_t)slot * H * mm_head_floats(d, dv) + (size_t)hd * mm_head_floats(d, dv);
    float* ng = Sg + (size_t)d * dv + (size_t)vb * (d + 1);
    float* mg = ng + d;
    float S[DS], nr[2];
#pragma unroll
    for (int j = 0; j < DS; j++) S[j] = (!fresh && colok && d0 + j < d) ? Sg[(size_t)(d0 + j) * dv + col] : 0.f;
#pragma unroll
    for (int r = 0; r < 2; r++) { const int i = tid + r * MM_WARPS * 32; nr[r] = (!fresh && i < d) ? ng[i] : 0.f; }
    float m = fresh ? 0.f : *mg;
    const float inv_cap = 1.0f / a.gate_cap;
    for (int t0 = 0; t0 < n_tok; t0 += MM_TB) {
        const int nb = min(MM_TB, n_tok - t0);
        __syncthreads();                                     // the round before is consumed
        for (int i = tid; i < nb * d; i += MM_WARPS * 32) {
            const int tt = i / d, c = i - tt * d;
            const float* pr = a.proj + (size_t)(row0 + t0 + tt) * a.ld_proj + (size_t)hd * d + c;
            qs[i] = pr[a.q_off] * a.q_scale;
            ks[i] = pr[a.k_off];
        }
        for (int i = tid; i < nb * MM_COLS; i += MM_WARPS * 32) {
            const int tt = i / MM_COLS, c = vb * MM_COLS + (i % MM_COLS);
            vs[i] = c < dv ? a.proj[(size_t)(row0 + t0 + tt) * a.ld_proj + a.v_off + (size_t)hd * dv + c] : 0.f;
        }
        if (tid < nb) {
            const float* pr = a.proj + (size_t)(row0 + t0 + tid) * a.ld_proj + hd;
            ga[tid] = a.gate_cap * tanhf((pr[a.i_off] + a.i_bias[hd]) * inv_cap);
            gb[tid] = log_sigmoid(a.gate_cap * tanhf((pr[a.f_off] + a.f_bias[hd]) * inv_cap));
        }
        __syncthreads();
        for (int tt = 0; tt < nb; tt++) {
            const float at = ga[tt], bt = gb[tt];
            const float mn = fmaxf(bt + m, at);
            const float keep = expf(bt + m - mn), take = expf(at - mn);
            m = mn;
            const float* qt = qs + tt * d;
            const float* kt = ks + tt * d;
            const float tv = take * vs[tt * MM_COLS + lane];
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < DS; j++) {
                if (d0 + j < d) {
                    S[j] = fmaf(kt[d0 + j], tv, keep * S[j]);
                    acc = fmaf(S[j], qt[d0 + j], acc);
                }
            }
            float nq = 0.f;
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const int i = tid + r * MM_WARPS * 32;
                if (i < d) { nr[r] = fmaf(take, kt[i], keep * nr[r]); nq = fmaf(nr[r], qt[i], nq); }
            }
            nq = warp_sum(nq);
            float* pp = part + (tt & 1) * MM_WARPS * MM_COLS;
            float* np = npart + (tt & 1) * MM_WARPS;
            pp[warp * MM_COLS + lane] = acc;
            if (lane == 0) np[warp] = nq;
            __syncthreads();                                 // the buffers alternate, so one barrier per token is enough
            if (warp == 0 && colok) {
                const float y = (pp[lane] + pp[MM_COLS + lane]) + (pp[2 * MM_COLS + lane] + pp[3 * MM_COLS + lane]);
                const float den = fmaxf(fabsf((np[0] + np[1]) + (np[2] + np[3])), expf(-m)) + 1e-6f;
                a.out[(size_t)(row0 + t0 + tt) * a.ld_out + (size_t)hd * dv + col] = y / den;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < DS; j++) if (colok && d0 + j < d) Sg[(size_t)(d0 + j) * dv + col] = S[j];
#pragma unroll
    for (int r = 0; r < 2; r++) { const int i = tid + r * MM_WARPS * 32; if (i < d) ng[i] = nr[r]; }
    if (tid == 0) *mg = m;
}

// one warp per (token, head)
template <typename AT>
__global__ void headnorm_gate_kernel(const float* __restrict__ y, int64_t ldy, int H, int dv, const float* __restrict__ gain,
                                     const float* __restrict__ gate, int64_t ld_gate, float scale, float eps, AT* __restrict__ out,
                                     int64_t ldo, int64_t T) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int lane = threadIdx.x & 31;
    const int64_t job = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (job >= T * H) return;
    const int64_t t = job / H;
    const int h = (int)(job - t * H);
    const float* yr = y + t * ldy + (size_t)h * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(yr[i], yr[i], ss);
    ss = warp_sum(ss);
    const float r = scale / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const int c = h * dv + i;
        const float g = gate ? 1.0f / (1.0f + expf(-gate[t * ld_gate + c])) : 1.f;
        stv(out + t * ldo + c, yr[i] * r * gain[c] * g);
    }
}
}  // namespace

extern "C" int64_t p3_matrix_memory_state_floats(int n_heads, int dim, int vdim) { return (int64_t)n_heads * mm_head_floats(dim, vdim); }

extern "C" int p3_matrix_memory_scan(const p3_matrix_memory_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->proj && a->i_bias && a->f_bias && a->state && a->seqs && a->out, "matrix_memory_scan: null argument");
    P3_CHECK_ARG(a->n_heads >= 1 && a->dim >= 1 && a->dim <= 256 && a->vdim >= 1, "matrix_memory_scan: need heads >= 1, 1 <= dim <= 256, vdim >= 1");
    P3_CHECK_ARG(a->gate_cap > 0.f, "matrix_memory_scan: the gate cap must be positive");
    P3_CHECK_ARG(((uintptr_t)a->seqs & 15) == 0, "matrix_memory_scan: the sequence records must be 16-byte aligned");
    if (a->n_seqs == 0) return 0;
    const dim3 grid((unsigned)a->n_seqs, (unsigned)a->n_heads, (unsigned)mm_col_blocks(a->vdim));
    const size_t bytes = sizeof(float) * ((size_t)2 * MM_TB * a->dim + MM_TB * MM_COLS + 2 * MM_TB + 2 * MM_WARPS * MM_COLS + 2 * MM_WARPS);
    if (a->dim <= 64) p3_launch_pdl(matrix_memory_scan_kernel<16>, dim3(grid), dim3(MM_WARPS * 32), (size_t)(bytes), st, *a);
    else if (a->dim <= 128) p3_launch_pdl(matrix_memory_scan_kernel<32>, dim3(grid), dim3(MM_WARPS * 32), (size_t)(bytes), st, *a);
    else p3_launch_pdl(matrix_memory_scan_kernel<64>, dim3(grid), dim3(MM_WARPS * 32), (size_t)(bytes), st, *a);
    P3_CHECK_LAUNCH("matrix_memory_scan");
    return 0;
}

extern "C" int p3_headnorm_gate(const float* y, int64_t ldy, int n_heads, int vdim, const float* gain, const float* gate, int64_t ld_gate,
                                float scale, float eps, void* out, int64_t ldo, int out_f32, int64_t T, cudaStream_t st) {
    P3_CHECK_ARG(y && gain && out && n_heads >= 1 && vdim >= 1, "headnorm_gate: null argument");
    if (T == 0) return 0;
    const int64_t jobs = T * n_heads;
    const unsigned grid = (unsigned)((jobs + 3) / 4);
    if (out_f32) p3_launch_pdl(headnorm_gate_kernel<float>, dim3(grid), dim3(128), (size_t)(0), st, y, ldy, n_heads, vdim, gain, gate, ld_gate, scale, eps, (float*)out, ldo, T);
    else p3_launch_pdl(headnorm_gate_kernel<bf16>, dim3(grid), dim3(128), (size_t)(0), st, y, ldy, n_heads, vdim, gain, gate, ld_gate, scale, eps, (bf16*)out, ldo, T);
    P3_CHECK_LAUNCH("headnorm_gate");
    return 0;
}
