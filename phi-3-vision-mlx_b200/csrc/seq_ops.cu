// Row kernels of decoders that keep the residual stream in fp32 and run a ragged token batch (several sequences, each with its
// own number of new tokens) against a paged cache: embedding into fp32, RMS norm of a sublayer's OUTPUT fused with the residual
// add, per-head query/key RMS norm fused with value mixing, the output-gate sigmoid and the paged K/V write, the clamped
// gated-linear activation, the mixture-of-experts router (logits, top-k, softmax over the chosen), the expert sort and the
// weighted combine, the distance tables of the biased attention (logarithmic and linear), and the embedding that adds the row of
// a hashed (previous, current) token pair, with the previous token kept per sequence slot. Everything here is fp32 arithmetic; only the
// storage type of activations ("act": bf16 or fp32) and of the cache differs between the serving mode and the all-fp32 mode.
#include "common.cuh"
#include "../../include/phi3_b200.h"

namespace {
template <typename T> __device__ __forceinline__ float ldv(const T* p);
template <> __device__ __forceinline__ float ldv<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldv<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stv(T* p, float v);
template <> __device__ __forceinline__ void stv<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stv<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// sum over a CTA of up to 1024 threads; every thread gets the total. The order of the additions is fixed by the thread
// layout alone, so a row's statistic does not depend on the batch it is in.
__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += sh[i];
    return t;
}

// ---------------------------------------------------------------- embedding -> fp32 residual (+ activation copy)
// Row kernels below keep up to RPT elements per thread in registers: all loads of a pass are issued before the first use, so a
// row of a small batch costs a few memory round trips instead of one per loop iteration.
constexpr int RPT = 8;

template <typename AT>
__global__ void embed_rows_kernel(const bf16* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ x,
                                  AT* __restrict__ xa, int W, int vocab, float scale, int64_t ldxa) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const bf16* src = table + (size_t)id * W;
    for (int i0 = threadIdx.x; i0 < W; i0 += RPT * blockDim.x) {
        float v[RPT];
#pragma unroll
        for (int k = 0; k < RPT; k++) { const int i = i0 + k * blockDim.x; v[k] = i < W ? __bfloat162float(src[i]) * scale : 0.f; }
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            const int i = i0 + k * blockDim.x;
            if (i < W) { x[(size_t)t * W + i] = v[k]; if (xa) stv(xa + (size_t)t * ldxa + i, v[k]); }
        }
    }
}

// ---------------------------------------------------------------- x += rms_norm(y) * gain ; activation copy of the new x
template <typename AT>
__global__ void postnorm_residual_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ ybias,
                                         const float* __restrict__ gain, float* x, AT* __restrict__ xa, int W, float eps) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ float sh[32];
    const int64_t t = blockIdx.x;
    const float* yr = y + (size_t)t * ldy;
    float* xr = x + (size_t)t * W;
    const int nt = blockDim.x;
    float v[RPT];                                            // the first RPT * nt elements of the row stay in registers
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; v[k] = i < W ? yr[i] + (ybias ? ybias[i] : 0.f) : 0.f; }
#pragma unroll
    for (int k = 0; k < RPT; k++) ss = fmaf(v[k], v[k], ss);
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) { const float u = yr[i] + (ybias ? ybias[i] : 0.f); ss = fmaf(u, u, ss); }
    float xv[RPT], gv[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; xv[k] = i < W ? xr[i] : 0.f; gv[k] = i < W ? gain[i] : 0.f; }
    ss = block_sum(ss, sh);
    const float r = 1.0f / sqrtf(ss / (float)W + eps);
#pragma unroll
    for (int k = 0; k < RPT; k++) {
        const int i = threadIdx.x + k * nt;
        if (i < W) { const float u = xv[k] + v[k] * r * gv[k]; xr[i] = u; if (xa) stv(xa + (size_t)t * W + i, u); }
    }
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) {
        const float u = xr[i] + (yr[i] + (ybias ? ybias[i] : 0.f)) * r * gain[i];
        xr[i] = u;
        if (xa) stv(xa + (size_t)t * W + i, u);
    }
}

// ---------------------------------------------------------------- out[r] = rms_norm(x[rows[r]]) * gain   (final norm of chosen rows)
template <typename AT>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ gain,
                                    AT* __restrict__ out, int W, float eps) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ float sh[32];
    const int64_t r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * W;
    const int nt = blockDim.x;
    float v[RPT], gv[RPT];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; v[k] = i < W ? xr[i] : 0.f; gv[k] = i < W ? gain[i] : 0.f; }
#pragma unroll
    for (int k = 0; k < RPT; k++) ss = fmaf(v[k], v[k], ss);
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) { const float u = xr[i]; ss = fmaf(u, u, ss); }
    ss = block_sum(ss, sh);
    const float s = 1.0f / sqrtf(ss / (float)W + eps);
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; if (i < W) stv(out + (size_t)r * W + i, v[k] * s * gv[k]); }
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) stv(out + (size_t)r * W + i, xr[i] * s * gain[i]);
}

// ---------------------------------------------------------------- per-head q/k norm + value mixing + gate + paged K/V write
// Grid (token, job group): one warp per head job (H query heads, G key heads, G value heads); group 0 also turns the H gate
// logits into gates. A head's numbers stay in registers between the statistic and the write (head sizes <= 256: 8 per lane).
template <typename AT, typename CT>
__global__ void qk_norm_kv_write_kernel(p3_qkv_post_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* pr = a.proj + (size_t)t * a.ld_proj;
    const int slot = a.tok_slot[t], pos = a.tok_pos[t];
    const int page = a.block_table[(size_t)slot * a.bt_stride + pos / P3_PAGE], off = pos % P3_PAGE;
    const int H = a.n_heads, G = a.n_kv, d = a.dim, dv = a.vdim;
    for (int job = blockIdx.y * nw + warp; job < H + 2 * G; job += gridDim.y * nw) {
        if (job < H + G) {                                   // query or key head: RMS norm over its d numbers, shared gain
            const bool isq = job < H;
            const int h = isq ? job : job - H;
            const int c0 = (isq ? a.q_off : a.k_off) + h * d;
            const float* src = pr + c0;
            const float* gain = isq ? a.q_gain : a.k_gain;
            float sv[8], gv[8];
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = lane + 32 * k;
                sv[k] = i < d ? src[i] + (a.bias ? a.bias[c0 + i] : 0.f) : 0.f;
                gv[k] = i < d ? gain[i] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 8; k++) ss = fmaf(sv[k], sv[k], ss);
            ss = warp_sum(ss);
            float r = 1.0f / sqrtf(ss / (float)d + a.eps);
            // query temperature: a factor that grows with the logarithm of the position counted in steps of q_temp_every
            if (isq && a.q_temp_every > 0) r *= 1.0f + a.q_temp_coef * logf((float)((pos + 1) / a.q_temp_every) + 1.0f);
            if (isq) {
                AT* dst = (AT*)a.q_out + (size_t)t * a.ld_q + (size_t)h * d;
#pragma unroll
                for (int k = 0; k < 8; k++) { const int i = lane + 32 * k; if (i < d) stv(dst + i, sv[k] * r * gv[k]); }
            } else {
                CT* dst = (CT*)a.k_pool + (((size_t)page * G + h) * P3_PAGE + off) * d;
#pragma unroll
                for (int k = 0; k < 8; k++) { const int i = lane + 32 * k; if (i < d) stv(dst + i, sv[k] * r * gv[k]); }
            }
        } else {                                             // value head: v, or (1 - lam) v + lam v_first; the mixed v is cached
            const int h = job - H - G;
            const int c0 = a.v_off + h * dv;
            const float* src = pr + c0;
            float* vf = a.v_first ? a.v_first + (size_t)t * G * dv + (size_t)h * dv : nullptr;
            CT* dst = (CT*)a.v_pool + (((size_t)page * G + h) * P3_PAGE + off) * dv;
            float sv[8], fv[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = lane + 32 * k;
                sv[k] = i < dv ? src[i] + (a.bias ? a.bias[c0 + i] : 0.f) : 0.f;
                fv[k] = (i < dv && a.v_mode == 2) ? vf[i] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int i = lane + 32 * k;
                if (i >= dv) continue;
                float v = sv[k];
                if (a.v_mode == 1) vf[i] = v;
                else if (a.v_mode == 2) v = (1.0f - a.v_lambda) * v + a.v_lambda * fv[k];
                stv(dst + i, v);
            }
        }
    }
    if (a.gate_out && blockIdx.y == 0)
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            a.gate_out[(size_t)t * H + h] = 1.0f / (1.0f + expf(-pr[a.g_off + h]));
}

// ---------------------------------------------------------------- y = g' * sigmoid(alpha g') * (u' + 1), g' = min(g, lim), u' = clamp(u)
template <typename AT>
__global__ void glu_clamped_kernel(const float* __restrict__ gu, int64_t ld, AT* __restrict__ out, int64_t ldo, int64_t R, int F,
                                   float limit, float alpha, const float* __restrict__ bias) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t n = R * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F; const int c = (int)(i % F);
        const float g = fminf(gu[(size_t)r * ld + c] + (bias ? bias[c] : 0.f), limit);
        const float u = fminf(fmaxf(gu[(size_t)r * ld + F + c] + (bias ? bias[F + c] : 0.f), -limit), limit);
        stv(out + (size_t)r * ldo + c, g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f));
    }
}

// four columns per thread (F, both row pitches and the pointers are multiples of four elements): 16-byte loads
template <typename AT>
__global__ void glu_clamped_vec4_kernel(const float* __restrict__ gu, int64_t ld, AT* __restrict__ out, int64_t ldo, int64_t R, int F,
                                        float limit, float alpha, const float* __restrict__ bias) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int F4 = F / 4;
    const int64_t n = R * F4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F4; const int c = (int)(i % F4) * 4;
        float4 g = *reinterpret_cast<const float4*>(gu + (size_t)r * ld + c);
        float4 u = *reinterpret_cast<const float4*>(gu + (size_t)r * ld + F + c);
        if (bias) {
            const float4 bg = *reinterpret_cast<const float4*>(bias + c), bu = *reinterpret_cast<const float4*>(bias + F + c);
            g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w; u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
        }
        float y[4];
        const float gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float a = fminf(gg[k], limit), b = fminf(fmaxf(uu[k], -limit), limit);
            y[k] = a * (1.0f / (1.0f + expf(-alpha * a))) * (b + 1.0f);
        }
        AT* o = out + (size_t)r * ldo + c;
        if constexpr (sizeof(AT) == 4) *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
        else *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
    }
}

// ---------------------------------------------------------------- router: fp32 logits, top-k (ties: lower index), softmax over the chosen
// One CTA per token: the threads split the token's activations, eight experts per pass; partial sums are reduced in an order
// fixed by the thread layout (lanes, then warps in ascending order), so a token's logits do not depend on the batch.
template <typename AT>
__global__ void router_topk_kernel(const AT* __restrict__ x, int64_t ldx, const float* __restrict__ Wr, const float* __restrict__ br,
                                   int T, int W, int E, int top, int32_t* __restrict__ ids, float* __restrict__ wts) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ float z[];                             // [E] logits, then [warps][8] partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int t = blockIdx.x;
    float* part = z + E;
    const AT* xr = x + (size_t)t * ldx;
    for (int e0 = 0; e0 < E; e0 += 8) {                      // eight experts per pass over the token's activations
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const int ne = min(8, E - e0);
#pragma unroll 2
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const float xv = ldv(xr + i);
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) wv[j] = j < ne ? Wr[(size_t)(e0 + j) * W + i] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) s[j] = fmaf(xv, wv[j], s[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float v = warp_sum(s[j]);
            if (lane == 0) part[warp * 8 + j] = v;
        }
        __syncthreads();
        if (threadIdx.x < ne) {
            float v = 0.f;
            for (int w = 0; w < nw; w++) v += part[w * 8 + threadIdx.x];
            z[e0 + threadIdx.x] = v + br[e0 + threadIdx.x];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float zmax = 0.f, den = 0.f;
        for (int j = 0; j < top; j++) {
            int best = -1; float bv = 0.f;
            for (int e = 0; e < E; e++) {
                bool taken = false;
                for (int q = 0; q < j; q++) taken |= ids[(size_t)t * top + q] == e;
                if (!taken && (best < 0 || z[e] > bv)) { best = e; bv = z[e]; }
            }
            ids[(size_t)t * top + j] = best;
            if (j == 0) zmax = bv;
            const float w = expf(bv - zmax);
            wts[(size_t)t * top + j] = w;
            den += w;
        }
        for (int j = 0; j < top; j++) wts[(size_t)t * top + j] /= den;
    }
}

// ---------------------------------------------------------------- expert sort: CTA e lists the (token, choice) pairs routed to expert e, in
// token order, behind those of the experts before it. seg[e] = first sorted row of expert e, seg[E] = n; order[r] = token * top +
// choice of sorted row r; where[token * top + choice] = r.
__global__ void moe_sort_kernel(const int32_t* __restrict__ ids, int n, int E, int32_t* __restrict__ seg,
                                int32_t* __restrict__ order, int32_t* __restrict__ where) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ int sh_w[33];
    __shared__ int sh_base;
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    int below = 0;
    for (int i = tid; i < n; i += blockDim.x) below += ids[i] < e;
    // block total of `below`
    for (int o = 16; o > 0; o >>= 1) below += __shfl_xor_sync(0xffffffffu, below, o);
    if (lane == 0) sh_w[warp] = below;
    __syncthreads();
    if (tid == 0) { int s = 0; for (int i = 0; i < nw; i++) s += sh_w[i]; sh_base = s; seg[e] = s; }
    __syncthreads();
    int base = sh_base;
    for (int i0 = 0; i0 < n; i0 += blockDim.x) {
        const int i = i0 + tid;
        const bool mine = i < n && ids[i] == e;
        const unsigned bal = __ballot_sync(0xffffffffu, mine);
        const int in_warp = __popc(bal & ((1u << lane) - 1));
        __syncthreads();
        if (lane == 0) sh_w[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < nw; w++) { const int c = sh_w[w]; if (w < warp) before += c; total += c; }
        if (mine) { const int r = base + before + in_warp; order[r] = i; where[i] = r; }
        base += total;
    }
    if (e == E - 1 && tid == 0) seg[E] = n;
}

// ---------------------------------------------------------------- out[r] = x[rows[r] / div]: rows of the activations in expert order
template <typename AT>
__global__ void gather_rows_kernel(const AT* __restrict__ x, int64_t ldx, const int32_t* __restrict__ rows, int div,
                                   AT* __restrict__ out, int W) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t r = blockIdx.x;
    const AT* src = x + (size_t)(rows[r] / div) * ldx;
    for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)r * W + i] = src[i];
}

// ---------------------------------------------------------------- out[t] = sum_j w[t][j] * y[where[t * top + j]]   (j ascending)
__global__ void moe_combine_kernel(const float* __restrict__ y, int64_t ldy, const int32_t* __restrict__ where,
                                   const float* __restrict__ wts, int top, float* __restrict__ out, int W) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ float cw[];                            // [top] weights, then [top] sorted rows
    int* rows = reinterpret_cast<int*>(cw + top);
    const int64_t t = blockIdx.x;
    for (int j = threadIdx.x; j < top; j += blockDim.x) { cw[j] = wts[t * top + j]; rows[j] = where[t * top + j]; }
    __syncthreads();
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float s = 0.f;
#pragma unroll 4
        for (int j = 0; j < top; j++) s = fmaf(cw[j], y[(size_t)rows[j] * ldy + i], s);
        out[(size_t)t * W + i] = s;
    }
}

// ---------------------------------------------------------------- pen[h][dist] = r1_h * ln(1 + r2_h * dist)
__global__ void distance_penalty_kernel(const float* __restrict__ r1, const float* __restrict__ r2, float* __restrict__ pen, int H, int n) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int h = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        pen[(size_t)h * n + i] = r1[h] * log1pf(r2[h] * (float)i);
}

// ---------------------------------------------------------------- v = x + add1 + add2 ; x <- v ; activation copy ; layer norm of v
// One CTA per row. Mean and variance are two passes over the row's fp32 sums (the variance is the mean squared deviation, not
// E[v^2] - mean^2). The first RPT * blockDim elements stay in registers; longer rows are formed again from memory in each pass
// (x is written only in the last one).
template <typename AT>
__global__ void residual_layernorm_kernel(float* x, const float* __restrict__ a1, int64_t ld1, const float* __restrict__ a2, int64_t ld2,
                                          const int32_t* __restrict__ rows, const float* __restrict__ gain, const float* __restrict__ bias,
                                          AT* __restrict__ xa, int64_t ldxa, AT* __restrict__ ho, int64_t ldh, int W, float eps) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ float sh[32];
    const int64_t r = blockIdx.x, t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * W;
    const float* p1 = a1 ? a1 + (size_t)t * ld1 : nullptr;
    const float* p2 = a2 ? a2 + (size_t)t * ld2 : nullptr;
    const int nt = blockDim.x;
    auto val = [&](int i) { float u = xr[i]; if (p1) u += p1[i]; if (p2) u += p2[i]; return u; };
    float v[RPT];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; v[k] = i < W ? val(i) : 0.f; s += v[k]; }
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) s += val(i);
    const bool store_x = !rows && (p1 || p2);
    float mean = 0.f, rstd = 0.f;
    if (ho) {
        mean = block_sum(s, sh) / (float)W;
        float q = 0.f;
#pragma unroll
        for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; const float dlt = v[k] - mean; if (i < W) q = fmaf(dlt, dlt, q); }
        for (int i = threadIdx.x + RPT * nt; i < W; i += nt) { const float dlt = val(i) - mean; q = fmaf(dlt, dlt, q); }
        rstd = 1.0f / sqrtf(block_sum(q, sh) / (float)W + eps);
    }
#pragma unroll
    for (int k = 0; k < RPT; k++) {
        const int i = threadIdx.x + k * nt;
        if (i >= W) continue;
        if (store_x) xr[i] = v[k];
        if (xa) stv(xa + (size_t)r * ldxa + i, v[k]);
        if (ho) stv(ho + (size_t)r * ldh + i, (v[k] - mean) * rstd * gain[i] + bias[i]);
    }
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) {
        const float u = val(i);
        if (store_x) xr[i] = u;
        if (xa) stv(xa + (size_t)r * ldxa + i, u);
        if (ho) stv(ho + (size_t)r * ldh + i, (u - mean) * rstd * gain[i] + bias[i]);
    }
}

// ---------------------------------------------------------------- latent attention: what follows the fused input projection
// Grid (token, job group). Jobs of a token: 0 = the latent vector (RMS norm -> cache) with the shared turning key part
// (rotation -> cache), 1 .. H = the query heads (plain part -> q_plain, turning part rotated -> q_lat); one warp per job. The
// gated unit's columns are then split over all threads of the token's CTAs, four columns per thread where the pitches allow.
__device__ __forceinline__ void turn_pair(float u, float v, float ang, float mag, float& ou, float& ov) {
    float sn, cs;
    sincosf(ang, &sn, &cs);
    sn *= mag; cs *= mag;
    ou = u * cs - v * sn;
    ov = v * cs + u * sn;
}

template <typename AT, typename CT>
__global__ void latent_post_kernel(p3_latent_post_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* pr = a.proj + (size_t)t * a.ld_proj;
    const int slot = a.tok_slot[t], pos = a.tok_pos[t];
    const int page = a.block_table[(size_t)slot * a.bt_stride + pos / P3_PAGE], off = pos % P3_PAGE;
    const int H = a.n_heads, d = a.dim, dr = a.rot_dim, R = a.kv_rank, half = a.rot_n / 2;
    const float fpos = (float)pos;
    // where the two numbers of rotation pair i live in a turning part
    const int pa = a.pair_mode ? 2 : 1, pb = a.pair_mode ? 1 : half;
    if (a.q_rank > 0 && blockIdx.y == 0) {
        // the query's low-rank vector: RMS norm -> input of the query up-projection. It is the longest row of the kernel, so the
        // whole CTA shares it (up to RPT numbers per thread stay in registers between the statistic and the write)
        __shared__ float sh[32];
        const float* c = pr + a.cq_off;
        AT* dst = (AT*)a.cq_out + (size_t)t * a.ld_cq;
        const int nt = blockDim.x;
        float v[RPT], gv[RPT];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            const int i = threadIdx.x + k * nt;
            v[k] = i < a.q_rank ? c[i] : 0.f;
            gv[k] = i < a.q_rank ? a.cq_gain[i] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < RPT; k++) ss = fmaf(v[k], v[k], ss);
        for (int i = threadIdx.x + RPT * nt; i < a.q_rank; i += nt) ss = fmaf(c[i], c[i], ss);
        ss = block_sum(ss, sh);
        const float rs = 1.0f / sqrtf(ss / (float)a.q_rank + a.eps);
#pragma unroll
        for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; if (i < a.q_rank) stv(dst + i, v[k] * rs * gv[k]); }
        for (int i = threadIdx.x + RPT * nt; i < a.q_rank; i += nt) stv(dst + i, c[i] * rs * a.cq_gain[i]);
    }
    for (int job = blockIdx.y * nw + warp; job < 1 + H; job += gridDim.y * nw) {
        if (job == 0) {
            if (!a.cache) continue;
            const float* c = pr + a.c_off;
            CT* dst = (CT*)a.cache + ((size_t)page * P3_PAGE + off) * (R + dr);
            float ss = 0.f;
            for (int i = lane; i < R; i += 32) ss = fmaf(c[i], c[i], ss);
            ss = warp_sum(ss);
            const float rs = 1.0f / sqrtf(ss / (float)R + a.eps);
            for (int i = lane; i < R; i += 32) stv(dst + i, c[i] * rs * a.c_gain[i]);
            const float* kr = c + R;
            for (int i = lane; i < half; i += 32) {
                float ou, ov;
                turn_pair(kr[pa * i], kr[pa * i + pb], fpos * a.freq[i], a.rot_mag, ou, ov);
                stv(dst + R + pa * i, ou); stv(dst + R + pa * i + pb, ov);
            }
            for (int i = a.rot_n + lane; i < dr; i += 32) stv(dst + R + i, kr[i]);
        } else {
            const int h = job - 1;
            const float* q = (a.q_src ? a.q_src + (size_t)t * a.ld_qsrc : pr + a.q_off) + (size_t)h * (d + dr);
            AT* qp = (AT*)a.q_plain + (size_t)t * a.ld_qp + (size_t)h * d;
            for (int i = lane; i < d; i += 32) stv(qp + i, q[i]);
            if (dr > 0) {
                const float* qr = q + d;
                AT* ql = (AT*)a.q_lat + (size_t)t * a.ld_ql + (size_t)h * (R + dr) + R;
                for (int i = lane; i < half; i += 32) {
                    float ou, ov;
                    turn_pair(qr[pa * i], qr[pa * i + pb], fpos * a.freq[i], a.rot_mag, ou, ov);
                    stv(ql + pa * i, ou); stv(ql + pa * i + pb, ov);
                }
                for (int i = a.rot_n + lane; i < dr; i += 32) stv(ql + i, qr[i]);
            }
        }
    }
    if (a.n_ff > 0) {
        const float* g = pr + a.gate_off;
        const float* u = pr + a.up_off;
        AT* hd = (AT*)a.hid + (size_t)t * a.ld_hid + a.hid_off;
        const int n_thr = blockDim.x * gridDim.y, me = blockIdx.y * blockDim.x + threadIdx.x;
        const bool vec = (a.n_ff % 4 == 0) && (a.gate_off % 4 == 0) && (a.up_off % 4 == 0) && (a.ld_proj % 4 == 0) &&
                         (a.hid_off % 4 == 0) && (a.ld_hid % 4 == 0) && (((uintptr_t)a.proj & 15) == 0) && (((uintptr_t)a.hid & 15) == 0);
        if (vec) {
            for (int i = me * 4; i < a.n_ff; i += n_thr * 4) {
                const float4 gv = *reinterpret_cast<const float4*>(g + i), uv = *reinterpret_cast<const float4*>(u + i);
                const float y0 = gv.x / (1.0f + expf(-gv.x)) * uv.x, y1 = gv.y / (1.0f + expf(-gv.y)) * uv.y;
                const float y2 = gv.z / (1.0f + expf(-gv.z)) * uv.z, y3 = gv.w / (1.0f + expf(-gv.w)) * uv.w;
                if constexpr (sizeof(AT) == 4) *reinterpret_cast<float4*>(hd + i) = make_float4(y0, y1, y2, y3);
                else *reinterpret_cast<uint2*>(hd + i) = make_uint2(pack_bf16(y0, y1), pack_bf16(y2, y3));
            }
        } else {
            for (int i = me; i < a.n_ff; i += n_thr) { const float gv = g[i]; stv(hd + i, gv / (1.0f + expf(-gv)) * u[i]); }
        }
    }
}

// ---------------------------------------------------------------- y = silu(g) * u
template <typename AT>
__global__ void glu_silu_kernel(const float* __restrict__ g, const float* __restrict__ u, int64_t ld, AT* __restrict__ out, int64_t ldo,
                                int64_t R, int F) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t n = R * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F; const int c = (int)(i % F);
        const float gv = g[(size_t)r * ld + c], uv = u[(size_t)r * ld + c];
        stv(out + (size_t)r * ldo + c, gv / (1.0f + expf(-gv)) * uv);
    }
}

// four columns per thread (F, the row pitches and the pointers are multiples of four elements): 16-byte loads
template <typename AT>
__global__ void glu_silu_vec4_kernel(const float* __restrict__ g, const float* __restrict__ u, int64_t ld, AT* __restrict__ out,
                                     int64_t ldo, int64_t R, int F) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int F4 = F / 4;
    const int64_t n = R * F4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F4; const int c = (int)(i % F4) * 4;
        const float4 gv = *reinterpret_cast<const float4*>(g + (size_t)r * ld + c), uv = *reinterpret_cast<const float4*>(u + (size_t)r * ld + c);
        const float y0 = gv.x / (1.0f + expf(-gv.x)) * uv.x, y1 = gv.y / (1.0f + expf(-gv.y)) * uv.y;
        const float y2 = gv.z / (1.0f + expf(-gv.z)) * uv.z, y3 = gv.w / (1.0f + expf(-gv.w)) * uv.w;
        AT* o = out + (size_t)r * ldo + c;
        if constexpr (sizeof(AT) == 4) *reinterpret_cast<float4*>(o) = make_float4(y0, y1, y2, y3);
        else *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(y0, y1), pack_bf16(y2, y3));
    }
}

// ---------------------------------------------------------------- router with sigmoid scores, a choice correction and expert groups
// One CTA per token; the logits are formed as in router_topk_kernel (eight experts per pass, fixed summation order). Warp 0 then
// selects: group scores (sum of the two largest choice scores of a group), the `keep` best groups, the `top` best experts of
// those; every maximum is an arg-max over the warp with ties going to the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

template <typename AT>
__global__ void router_sigmoid_groups_kernel(const AT* __restrict__ x, int64_t ldx, const float* __restrict__ Wr,
                                             const float* __restrict__ corr, const float* __restrict__ logits, int64_t ld_logits,
                                             int W, int E, int top, int n_groups, int keep,
                                             float scale, int mode, int32_t* __restrict__ ids, float* __restrict__ wts) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ float z[];                             // [E] scores s, [E] choice scores, [groups] group scores, [warps][8] partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int t = blockIdx.x, NG = n_groups > 1 ? n_groups : 1, gs = E / NG;
    float* ch = z + E;
    float* gsc = ch + E;
    float* part = gsc + NG;
    const AT* xr = x + (size_t)t * ldx;
    if (logits) {                                            // the logits came out of an earlier product (fp32 accumulation)
        for (int e = threadIdx.x; e < E; e += blockDim.x) z[e] = logits[(size_t)t * ld_logits + e];
        __syncthreads();
    } else
    for (int e0 = 0; e0 < E; e0 += 8) {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const int ne = min(8, E - e0);
#pragma unroll 2
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const float xv = ldv(xr + i);
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; j++) wv[j] = j < ne ? Wr[(size_t)(e0 + j) * W + i] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) s[j] = fmaf(xv, wv[j], s[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float v = warp_sum(s[j]);
            if (lane == 0) part[warp * 8 + j] = v;
        }
        __syncthreads();
        if (threadIdx.x < ne) {
            float v = 0.f;
            for (int w = 0; w < nw; w++) v += part[w * 8 + threadIdx.x];
            z[e0 + threadIdx.x] = v;
        }
        __syncthreads();
    }
    if (warp != 0) return;
    // logits -> scores: sigmoid of each, or (mode bit 0) softmax over all outputs with sums in a fixed order
    float zmax = -INFINITY, zsum = 0.f;
    if (mode & 1) {
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        for (int e = lane; e < E; e += 32) zsum += expf(z[e] - zmax);
        zsum = warp_sum(zsum);
    }
    for (int e = lane; e < E; e += 32) {
        const float sc = (mode & 1) ? expf(z[e] - zmax) / zsum : 1.0f / (1.0f + expf(-z[e]));
        z[e] = sc;
        ch[e] = sc + (corr ? corr[e] : 0.f);
    }
    __syncwarp();
    if (NG > 1) {
        for (int g = lane; g < NG; g += 32) {                // a group's score: its two largest choice scores
            float b1 = -INFINITY, b2 = -INFINITY;
            for (int e = g * gs; e < (g + 1) * gs; e++) { const float c = ch[e]; if (c > b1) { b2 = b1; b1 = c; } else if (c > b2) b2 = c; }
            gsc[g] = (gs > 1 && !(mode & 2)) ? b1 + b2 : b1;
        }
        __syncwarp();
        for (int k = 0; k < keep; k++) {                     // mark the kept groups by +inf, one arg-max per kept group
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < NG; g += 32) { const float c = gsc[g]; if (c != INFINITY && (c > bv || (c == bv && g < bi))) { bv = c; bi = g; } }
            warp_argmax(bv, bi);
            if (lane == 0 && bi < NG) gsc[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) if (gsc[e / gs] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    float den = 0.f;
    for (int j = 0; j < top; j++) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { const float c = ch[e]; if (!isnan(c) && (c > bv || (c == bv && e < bi))) { bv = c; bi = e; } }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;                                  // fewer selectable experts than `top`: cannot happen with valid configs
        if (lane == 0) { ids[(size_t)t * top + j] = bi; wts[(size_t)t * top + j] = z[bi]; ch[bi] = NAN; }
        den += z[bi];
        __syncwarp();
    }
    if (mode & 4) return;                                    // the chosen scores are the weights as they are
    const float f = scale / (den + 1e-20f);
    for (int j = lane; j < top; j += 32) wts[(size_t)t * top + j] *= f;
}

// ---------------------------------------------------------------- logits <- cap * tanh(logits * scale / cap)
__global__ void logit_softcap_kernel(float* __restrict__ lg, int64_t n, float scale, float cap) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = lg[i] * scale;
        lg[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

// ---------------------------------------------------------------- norm after a sublayer, residual add, norm before the next one
// x += rms_norm(y + bias) * gain_post, then h = rms_norm(x) * gain_pre: two row statistics in one pass over the row, which stays in
// registers in between (up to RPT elements per thread; longer rows go through the row of x itself).
template <typename AT>
__global__ void postnorm_prenorm_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ ybias,
                                        const float* __restrict__ gpost, float* x, const float* __restrict__ gpre,
                                        float* __restrict__ h32, AT* __restrict__ ha, int W, float eps) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    __shared__ float sh[32];
    const int64_t t = blockIdx.x;
    float* xr = x + (size_t)t * W;
    const int nt = blockDim.x;
    float xv[RPT];
#pragma unroll
    for (int k = 0; k < RPT; k++) { const int i = threadIdx.x + k * nt; xv[k] = i < W ? xr[i] : 0.f; }
    if (y) {
        const float* yr = y + (size_t)t * ldy;
        float v[RPT], gv[RPT];
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            const int i = threadIdx.x + k * nt;
            v[k] = i < W ? yr[i] + (ybias ? ybias[i] : 0.f) : 0.f;
            gv[k] = i < W ? gpost[i] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < RPT; k++) ss = fmaf(v[k], v[k], ss);
        for (int i = threadIdx.x + RPT * nt; i < W; i += nt) { const float u = yr[i] + (ybias ? ybias[i] : 0.f); ss = fmaf(u, u, ss); }
        ss = block_sum(ss, sh);
        const float r = 1.0f / sqrtf(ss / (float)W + eps);
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            const int i = threadIdx.x + k * nt;
            if (i < W) { xv[k] = xv[k] + v[k] * r * gv[k]; xr[i] = xv[k]; }
        }
        for (int i = threadIdx.x + RPT * nt; i < W; i += nt) xr[i] = xr[i] + (yr[i] + (ybias ? ybias[i] : 0.f)) * r * gpost[i];
    }
    if (!gpre) return;
    float s2 = 0.f;
#pragma unroll
    for (int k = 0; k < RPT; k++) s2 = fmaf(xv[k], xv[k], s2);
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) { const float u = xr[i]; s2 = fmaf(u, u, s2); }   // this thread's own writes
    s2 = block_sum(s2, sh);
    const float r2 = 1.0f / sqrtf(s2 / (float)W + eps);
#pragma unroll
    for (int k = 0; k < RPT; k++) {
        const int i = threadIdx.x + k * nt;
        if (i < W) { const float u = xv[k] * r2 * gpre[i]; if (h32) h32[(size_t)t * W + i] = u; if (ha) stv(ha + (size_t)t * W + i, u); }
    }
    for (int i = threadIdx.x + RPT * nt; i < W; i += nt) {
        const float u = xr[i] * r2 * gpre[i];
        if (h32) h32[(size_t)t * W + i] = u;
        if (ha) stv(ha + (size_t)t * W + i, u);
    }
}

// ---------------------------------------------------------------- token shift: a row is blended with the row of the token before it
// One CTA per row. The CTA of a sequence's first row reads the slot's saved row and then replaces it by the sequence's last
// row of this step (same thread, same element: read before write), so no other CTA touches the slot's state.
template <typename AT>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ shift, float* state,
                                   const int32_t* __restrict__ seqs, const int32_t* __restrict__ slot_seq,
                                   const int32_t* __restrict__ tok_slot, AT* __restrict__ out, int W) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t t = blockIdx.x;
    const int slot = tok_slot[t];
    const int4 rec = reinterpret_cast<const int4*>(seqs)[slot_seq[slot]];   // {first row, rows, slot, first position}
    const bool first = t == rec.x;
    float* sv = state + (size_t)slot * W;
    const float* hr = h + (size_t)t * W;
    const float* prev = first ? (rec.w > 0 ? sv : nullptr) : hr - W;
    const float* lastr = h + (size_t)(rec.x + rec.y - 1) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float hv = hr[i], pv = prev ? prev[i] : 0.f;
        stv(out + (size_t)t * W + i, hv + (pv - hv) * shift[i]);
        if (first) sv[i] = lastr[i];
    }
}

// ---------------------------------------------------------------- rotation of q and k + paged K/V write (+ projection biases)
// Grid (token, job group): one warp per head job (H query heads, G key heads, G value heads when there is a value projection).
// The lane that owns number i < rot_n / 2 of a head also owns its partner i + rot_n / 2; angles are position * frequency in fp32
// with the full-range sincosf. Without a value projection the key head is written twice: rotated to the K pool, as projected to
// the V pool.
template <typename AT, typename CT>
__global__ void qkv_rope_kv_write_kernel(p3_qkv_rope_post_args a) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float* pr = a.proj + (size_t)t * a.ld_proj;
    const int slot = a.tok_slot[t], pos = a.tok_pos[t];
    const int page = a.block_table[(size_t)slot * a.bt_stride + pos / P3_PAGE], off = pos % P3_PAGE;
    const int H = a.n_heads, G = a.n_kv, d = a.dim, dv = a.vdim, half = a.rot_n / 2;
    const bool v_is_k = a.v_off < 0;
    const int jobs = H + G + (v_is_k ? 0 : G);
    for (int job = blockIdx.y * nw + warp; job < jobs; job += gridDim.y * nw) {
        if (job < H + G) {
            const bool isq = job < H;
            const int h = isq ? job : job - H;
            const int col0 = (isq ? a.q_off : a.k_off) + h * d;
            const float* src = pr + col0;
            const float* b = a.bias ? a.bias + col0 : nullptr;
            AT* dq = isq ? (AT*)a.q_out + (size_t)t * a.ld_q + (size_t)h * d : nullptr;
            CT* dk = isq ? nullptr : (CT*)a.k_pool + (((size_t)page * G + h) * P3_PAGE + off) * d;
            CT* dvv = (!isq && v_is_k) ? (CT*)a.v_pool + (((size_t)page * G + h) * P3_PAGE + off) * dv : nullptr;
            for (int i = lane; i < d; i += 32) {
                if (i >= half && i < a.rot_n) continue;      // the partner of a turning pair: written by the pair's owner
                const float u = src[i] + (b ? b[i] : 0.f);
                if (i < half) {
                    const float w = src[i + half] + (b ? b[i + half] : 0.f);
                    float sn, cs;
                    sincosf((float)pos * a.freq[i], &sn, &cs);
                    const float r0 = u * cs - w * sn, r1 = w * cs + u * sn;
                    if (isq) { stv(dq + i, r0); stv(dq + i + half, r1); }
                    else { stv(dk + i, r0); stv(dk + i + half, r1); if (dvv) { stv(dvv + i, u); stv(dvv + i + half, w); } }
                } else {
                    if (isq) stv(dq + i, u);
                    else { stv(dk + i, u); if (dvv) stv(dvv + i, u); }
                }
            }
        } else {
            const int h = job - H - G, col0 = a.v_off + h * dv;
            CT* dst = (CT*)a.v_pool + (((size_t)page * G + h) * P3_PAGE + off) * dv;
            for (int i = lane; i < dv; i += 32) stv(dst + i, pr[col0 + i] + (a.bias ? a.bias[col0 + i] : 0.f));
        }
    }
}

// ---------------------------------------------------------------- out = max(u, 0)^2 (* sigmoid of a per-row gate logit)
template <typename AT>
__global__ void relu2_kernel(const float* __restrict__ u, int64_t ld, const float* __restrict__ row_gate, int64_t ld_gate,
                             AT* __restrict__ out, int64_t ldo, int64_t R, int F) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t n = R * F;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F;
        const int c = (int)(i - r * F);
        const float v = fmaxf(u[r * ld + c], 0.f);
        const float g = row_gate ? 1.0f / (1.0f + expf(-row_gate[r * ld_gate])) : 1.f;
        stv(out + r * ldo + c, v * v * g);
    }
}

// four columns per thread (F, the row pitches and the pointers are multiples of four elements): 16-byte loads
template <typename AT>
__global__ void relu2_vec4_kernel(const float* __restrict__ u, int64_t ld, const float* __restrict__ row_gate, int64_t ld_gate,
                                  AT* __restrict__ out, int64_t ldo, int64_t R, int F) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int F4 = F / 4;
    const int64_t n = R * F4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F4; const int c = (int)(i % F4) * 4;
        const float4 v = *reinterpret_cast<const float4*>(u + (size_t)r * ld + c);
        const float g = row_gate ? 1.0f / (1.0f + expf(-row_gate[r * ld_gate])) : 1.f;
        const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), e = fmaxf(v.z, 0.f), f = fmaxf(v.w, 0.f);
        AT* o = out + (size_t)r * ldo + c;
        if constexpr (sizeof(AT) == 4) *reinterpret_cast<float4*>(o) = make_float4(a * a * g, b * b * g, e * e * g, f * f * g);
        else *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(a * a * g, b * b * g), pack_bf16(e * e * g, f * f * g));
    }
}

// token shift, four channels per thread (W a multiple of four, 16-byte aligned rows)
template <typename AT>
__global__ void token_shift_vec4_kernel(const float* __restrict__ h, const float* __restrict__ shift, float* state,
                                        const int32_t* __restrict__ seqs, const int32_t* __restrict__ slot_seq,
                                        const int32_t* __restrict__ tok_slot, AT* __restrict__ out, int W) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t t = blockIdx.x;
    const int slot = tok_slot[t];
    const int4 rec = reinterpret_cast<const int4*>(seqs)[slot_seq[slot]];   // {first row, rows, slot, first position}
    const bool first = t == rec.x;
    float* sv = state + (size_t)slot * W;
    const float* hr = h + (size_t)t * W;
    const float* prev = first ? (rec.w > 0 ? sv : nullptr) : hr - W;
    const float* lastr = h + (size_t)(rec.x + rec.y - 1) * W;
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
        const float4 hv = *reinterpret_cast<const float4*>(hr + i), sh = *reinterpret_cast<const float4*>(shift + i);
        const float4 pv = prev ? *reinterpret_cast<const float4*>(prev + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float y0 = hv.x + (pv.x - hv.x) * sh.x, y1 = hv.y + (pv.y - hv.y) * sh.y;
        const float y2 = hv.z + (pv.z - hv.z) * sh.z, y3 = hv.w + (pv.w - hv.w) * sh.w;
        AT* o = out + (size_t)t * W + i;
        if constexpr (sizeof(AT) == 4) *reinterpret_cast<float4*>(o) = make_float4(y0, y1, y2, y3);
        else *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(y0, y1), pack_bf16(y2, y3));
        if (first) *reinterpret_cast<float4*>(sv + i) = *reinterpret_cast<const float4*>(lastr + i);
    }
}

// ---------------------------------------------------------------- weighted sum of the chosen experts, identity experts and an addend
__global__ void moe_combine_identity_kernel(const float* __restrict__ y, int64_t ldy, const int32_t* __restrict__ where,
                                            const int32_t* __restrict__ ids, const float* __restrict__ wts, int top, int n_real,
                                            const float* __restrict__ h, const float* __restrict__ add, int64_t ld_add,
                                            float* __restrict__ out, int W) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    extern __shared__ float cw[];                            // [top] weights, then [top] sorted rows (-1: identity expert)
    int* rows = reinterpret_cast<int*>(cw + top);
    const int64_t t = blockIdx.x;
    for (int j = threadIdx.x; j < top; j += blockDim.x) {
        cw[j] = wts[t * top + j];
        rows[j] = ids[t * top + j] < n_real ? where[t * top + j] : -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float s = 0.f;
        const float hv = h ? h[(size_t)t * W + i] : 0.f;
#pragma unroll 4
        for (int j = 0; j < top; j++) s = fmaf(cw[j], rows[j] >= 0 ? y[(size_t)rows[j] * ldy + i] : hv, s);
        out[(size_t)t * W + i] = s + (add ? add[(size_t)t * ld_add + i] : 0.f);
    }
}
// ---------------------------------------------------------------- embedding plus the row of a hashed (previous, current) token pair
// One CTA per row. The token before a row is the row above it inside a sequence's run of rows, else the token the slot saved at
// the end of the sequence's last step. The CTA of a sequence's first row reads the saved token and then replaces it by the
// sequence's last token of this step (read, barrier, write), so no other CTA touches the slot's state.
__global__ void embed_pair_rows_kernel(const bf16* __restrict__ table, const bf16* __restrict__ pair_table, const int32_t* __restrict__ ids,
                                       const int32_t* __restrict__ seqs, const int32_t* __restrict__ slot_seq,
                                       const int32_t* __restrict__ tok_slot, int32_t* prev_state, int64_t state_stride,
                                       float* __restrict__ x, int W, int vocab, float scale, long long buckets, long long mul_prev,
                                       long long mul_cur) {
    pdl_trigger();                                           // the next kernel may set up while this one runs ...
    pdl_wait();                                              // ... and this one touches memory only after its predecessors are done
    const int64_t t = blockIdx.x;
    int id = ids[t];
    const int slot = tok_slot[t];
    const int4 rec = reinterpret_cast<const int4*>(seqs)[slot_seq[slot]];   // {first row, rows, slot, first position}
    const bool first = t == rec.x;
    const long long prev = first ? (rec.w > 0 ? prev_state[(size_t)slot * state_stride] : -1) : ids[t - 1];
    if (first) {
        __syncthreads();                                     // every thread has read the saved token
        if (threadIdx.x == 0) prev_state[(size_t)slot * state_stride] = ids[rec.x + rec.y - 1];
    }
    long long pr = buckets;                                  // a sequence's first token: the table's last row
    if (prev >= 0) { pr = (prev * mul_prev + (long long)id * mul_cur) % buckets; if (pr < 0) pr += buckets; }
    if (id < 0 || id >= vocab) id = 0;
    const bf16* src = table + (size_t)id * W;
    const bf16* ps = pair_table ? pair_table + (size_t)pr * W : nullptr;
    if (W % 8 == 0 && (((uintptr_t)table | (uintptr_t)pair_table | (uintptr_t)x) & 15) == 0) {   // eight numbers per thread and pass
        for (int i = threadIdx.x * 8; i < W; i += 8 * blockDim.x) {
            const uint4 a = *reinterpret_cast<const uint4*>(src + i);
            const uint4 b = ps ? *reinterpret_cast<const uint4*>(ps + i) : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
            float o[8];
#pragma unroll
            for (int k = 0; k < 4; k++) {                    // a bf16 is the upper half of its fp32
                o[2 * k] = __uint_as_float(aw[k] << 16) * scale + __uint_as_float(bw[k] << 16);
                o[2 * k + 1] = __uint_as_float(aw[k] & 0xffff0000u) * scale + __uint_as_float(bw[k] & 0xffff0000u);
            }
            float4* dst = reinterpret_cast<float4*>(x + (size_t)t * W + i);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
        return;
    }
    for (int i0 = threadIdx.x; i0 < W; i0 += RPT * blockDim.x) {
        float v[RPT], u[RPT];
#pragma unroll
        for (int k = 0; k < RPT; k++) {
            const int i = i0 + k * blockDim.x;
            v[k] = i < W ? __bfloat162float(src[i]) : 0.f;
            u[k] = (ps && i < W) ? __bfloat162float(ps[i]) : 0.f;
        }
#pragma unroll
        for (int k = 0; k < RPT; k++) { const int i = i0 + k * blockDim.x; if (i < W) x[(size_t)t * W + i] = v[k] * scale + u[k]; }
    }
}

__global__ void distance_linear_kernel(const float* __restrict__ slope, float* __restrict__ pen, int H, int n) {
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= (int64_t)H * n) return;
    const int h = (int)(i / n);
    pen[i] = slope[h] * (float)(i - (int64_t)h * n);
}
}  // namespace

extern "C" int p3_embed_rows_f32(const void* table, const int32_t* ids, float* x, void* x_act, int act_f32, int64_t T, int W, int vocab,
                                 float scale, int64_t ld_act, cudaStream_t st) {
    if (T == 0) return 0;
    if (ld_act <= 0) ld_act = W;
    if (act_f32) p3_launch_pdl(embed_rows_kernel<float>, dim3((unsigned)T), dim3(128), (size_t)(0), st, (const bf16*)table, ids, x, (float*)x_act, W, vocab, scale, ld_act);
    else p3_launch_pdl(embed_rows_kernel<bf16>, dim3((unsigned)T), dim3(128), (size_t)(0), st, (const bf16*)table, ids, x, (bf16*)x_act, W, vocab, scale, ld_act);
    P3_CHECK_LAUNCH("embed_rows_f32");
    return 0;
}

extern "C" int p3_postnorm_residual(const float* y, int64_t ldy, const float* y_bias, const float* gain, float* x, void* x_act, int act_f32,
                                    int64_t T, int W, float eps, cudaStream_t st) {
    if (T == 0) return 0;
    const int th = W > 4096 ? 1024 : W > 2048 ? 512 : W >= 1024 ? 256 : 128;     // the row fits the threads' registers up to W = 8192
    if (act_f32) p3_launch_pdl(postnorm_residual_kernel<float>, dim3((unsigned)T), dim3(th), (size_t)(0), st, y, ldy, y_bias, gain, x, (float*)x_act, W, eps);
    else p3_launch_pdl(postnorm_residual_kernel<bf16>, dim3((unsigned)T), dim3(th), (size_t)(0), st, y, ldy, y_bias, gain, x, (bf16*)x_act, W, eps);
    P3_CHECK_LAUNCH("postnorm_residual");
    return 0;
}

extern "C" int p3_rmsnorm_rows_f32(const float* x, const int32_t* rows, const float* gain, void* out, int out_f32, int64_t R, int W,
                                   float eps, cudaStream_t st) {
    if (R == 0) return 0;
    const int th = W > 4096 ? 1024 : W > 2048 ? 512 : W >= 1024 ? 256 : 128;
    if (out_f32) p3_launch_pdl(rmsnorm_rows_kernel<float>, dim3((unsigned)R), dim3(th), (size_t)(0), st, x, rows, gain, (float*)out, W, eps);
    else p3_launch_pdl(rmsnorm_rows_kernel<bf16>, dim3((unsigned)R), dim3(th), (size_t)(0), st, x, rows, gain, (bf16*)out, W, eps);
    P3_CHECK_LAUNCH("rmsnorm_rows_f32");
    return 0;
}

extern "C" int p3_qkv_post(const p3_qkv_post_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->proj && a->q_out && a->k_pool && a->v_pool && a->block_table && a->tok_slot && a->tok_pos, "qkv_post: null argument");
    P3_CHECK_ARG(a->v_mode == 0 || a->v_first, "qkv_post: value mixing needs the v_first buffer");
    if (a->T == 0) return 0;
    P3_CHECK_ARG(a->dim <= 256 && a->vdim <= 256, "qkv_post: head sizes must be <= 256");
    const int jobs = a->n_heads + 2 * a->n_kv, th = 128;
    // few tokens: one warp per job; many tokens: each CTA walks all jobs of its token (the grid is large enough already; spreading
    // the jobs over more CTAs measured no faster)
    const int groups = a->T >= 1024 ? 1 : (jobs + 3) / 4;
    const dim3 grid((unsigned)a->T, (unsigned)groups);
    if (a->act_f32 && a->cache_f32) p3_launch_pdl(qk_norm_kv_write_kernel<float, float>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else if (!a->act_f32 && !a->cache_f32) p3_launch_pdl(qk_norm_kv_write_kernel<bf16, bf16>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else P3_CHECK_ARG(false, "qkv_post: activations and cache must both be fp32 or both bf16");
    P3_CHECK_LAUNCH("qkv_post");
    return 0;
}

extern "C" int p3_glu_clamped(const float* gu, int64_t ld, void* out, int64_t ldo, int out_f32, int64_t R, int F, float limit, float alpha,
                              const float* bias, cudaStream_t st) {
    if (R == 0) return 0;
    const bool vec = F % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                     (!bias || ((uintptr_t)bias & 15) == 0);
    const int64_t n = vec ? R * (F / 4) : R * F;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (vec) {
        if (out_f32) p3_launch_pdl(glu_clamped_vec4_kernel<float>, dim3(grid), dim3(256), (size_t)(0), st, gu, ld, (float*)out, ldo, R, F, limit, alpha, bias);
        else p3_launch_pdl(glu_clamped_vec4_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), st, gu, ld, (bf16*)out, ldo, R, F, limit, alpha, bias);
    } else if (out_f32) p3_launch_pdl(glu_clamped_kernel<float>, dim3(grid), dim3(256), (size_t)(0), st, gu, ld, (float*)out, ldo, R, F, limit, alpha, bias);
    else p3_launch_pdl(glu_clamped_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), st, gu, ld, (bf16*)out, ldo, R, F, limit, alpha, bias);
    P3_CHECK_LAUNCH("glu_clamped");
    return 0;
}

extern "C" int p3_router_topk(const void* x, int64_t ldx, int x_f32, const float* Wr, const float* br, int T, int W, int E, int top,
                              int32_t* ids, float* wts, cudaStream_t st) {
    P3_CHECK_ARG(top >= 1 && top <= E && E <= 1024, "router_topk: need 1 <= top <= experts <= 1024");
    if (T == 0) return 0;
    const int nw = W >= 1024 ? 8 : 4;
    const size_t sm = ((size_t)E + nw * 8) * sizeof(float);
    if (x_f32) p3_launch_pdl(router_topk_kernel<float>, dim3((unsigned)T), dim3(nw * 32), (size_t)(sm), st, (const float*)x, ldx, Wr, br, T, W, E, top, ids, wts);
    else p3_launch_pdl(router_topk_kernel<bf16>, dim3((unsigned)T), dim3(nw * 32), (size_t)(sm), st, (const bf16*)x, ldx, Wr, br, T, W, E, top, ids, wts);
    P3_CHECK_LAUNCH("router_topk");
    return 0;
}

extern "C" int p3_moe_sort(const int32_t* ids, int n, int E, int32_t* seg, int32_t* order, int32_t* where, cudaStream_t st) {
    P3_CHECK_ARG(n >= 1 && E >= 1, "moe_sort: empty");
    p3_launch_pdl(moe_sort_kernel, dim3(E), dim3(1024), (size_t)(0), st, ids, n, E, seg, order, where);
    P3_CHECK_LAUNCH("moe_sort");
    return 0;
}

extern "C" int p3_gather_rows(const void* x, int64_t ldx, int x_f32, const int32_t* rows, int div, void* out, int64_t R, int W,
                              cudaStream_t st) {
    P3_CHECK_ARG(div >= 1 && rows, "gather_rows: need an index list and div >= 1");
    if (R == 0) return 0;
    if (x_f32) p3_launch_pdl(gather_rows_kernel<float>, dim3((unsigned)R), dim3(128), (size_t)(0), st, (const float*)x, ldx, rows, div, (float*)out, W);
    else p3_launch_pdl(gather_rows_kernel<bf16>, dim3((unsigned)R), dim3(128), (size_t)(0), st, (const bf16*)x, ldx, rows, div, (bf16*)out, W);
    P3_CHECK_LAUNCH("gather_rows");
    return 0;
}

extern "C" int p3_moe_combine(const float* y, int64_t ldy, const int32_t* where, const float* wts, int top, float* out, int64_t T, int W,
                              cudaStream_t st) {
    if (T == 0) return 0;
    p3_launch_pdl(moe_combine_kernel, dim3((unsigned)T), dim3(W >= 1024 ? 256 : 128), (size_t)((size_t)top * 8), st, y, ldy, where, wts, top, out, W);
    P3_CHECK_LAUNCH("moe_combine");
    return 0;
}

extern "C" int p3_distance_penalty_table(const float* r1, const float* r2, float* pen, int H, int n, cudaStream_t st) {
    P3_CHECK_ARG(H >= 1 && n >= 1, "distance_penalty_table: empty");
    p3_launch_pdl(distance_penalty_kernel, dim3(dim3((unsigned)((n + 255) / 256), (unsigned)H)), dim3(256), (size_t)(0), st, r1, r2, pen, H, n);
    P3_CHECK_LAUNCH("distance_penalty_table");
    return 0;
}

extern "C" int p3_residual_layernorm(float* x, const float* add1, int64_t ld1, const float* add2, int64_t ld2, const int32_t* rows,
                                     const float* gain, const float* bias, void* x_act, int64_t ld_xact, void* h_out, int64_t ld_h,
                                     int act_f32, int64_t R, int W, float eps, cudaStream_t st) {
    P3_CHECK_ARG(x && W >= 1, "residual_layernorm: null argument");
    P3_CHECK_ARG(!h_out || (gain && bias), "residual_layernorm: the norm needs weight and bias");
    if (R == 0) return 0;
    const int th = W > 4096 ? 1024 : W > 2048 ? 512 : W >= 1024 ? 256 : 128;
    if (act_f32) p3_launch_pdl(residual_layernorm_kernel<float>, dim3((unsigned)R), dim3(th), (size_t)(0), st, x, add1, ld1, add2, ld2, rows, gain, bias,
                               (float*)x_act, ld_xact, (float*)h_out, ld_h, W, eps);
    else p3_launch_pdl(residual_layernorm_kernel<bf16>, dim3((unsigned)R), dim3(th), (size_t)(0), st, x, add1, ld1, add2, ld2, rows, gain, bias,
                       (bf16*)x_act, ld_xact, (bf16*)h_out, ld_h, W, eps);
    P3_CHECK_LAUNCH("residual_layernorm");
    return 0;
}

extern "C" int p3_latent_post(const p3_latent_post_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->block_table && a->tok_slot && a->tok_pos, "latent_post: null argument");
    P3_CHECK_ARG(a->n_heads == 0 || ((a->proj || a->q_src) && a->q_plain), "latent_post: the query part needs its source and q_plain");
    P3_CHECK_ARG(!a->cache || (a->proj && a->c_gain), "latent_post: the latent part needs proj and its gain");
    P3_CHECK_ARG(a->q_rank <= 0 || (a->proj && a->cq_gain && a->cq_out), "latent_post: the query's low-rank vector needs proj, its gain and its output");
    P3_CHECK_ARG(a->n_ff == 0 || a->proj, "latent_post: the gated unit reads proj");
    P3_CHECK_ARG(a->rot_dim == 0 || a->rot_n == 0 || (a->freq && (a->n_heads == 0 || a->q_lat)), "latent_post: a turning part needs q_lat and the frequencies");
    P3_CHECK_ARG(a->rot_n >= 0 && a->rot_n <= a->rot_dim && a->rot_n % 2 == 0, "latent_post: rot_n must be even and <= rot_dim");
    P3_CHECK_ARG(a->n_ff == 0 || a->hid, "latent_post: the gated unit needs its output");
    if (a->T == 0) return 0;
    const int jobs = 1 + a->n_heads, th = 128;
    // few tokens: one warp per job and enough CTAs for the gated unit's columns; many tokens: one CTA per token
    int groups = a->T >= 1024 ? 1 : (jobs + 3) / 4;
    if (a->T < 1024 && groups < (a->n_ff + 2047) / 2048) groups = (a->n_ff + 2047) / 2048;
    const dim3 grid((unsigned)a->T, (unsigned)groups);
    if (a->act_f32 && a->cache_f32) p3_launch_pdl(latent_post_kernel<float, float>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else if (!a->act_f32 && !a->cache_f32) p3_launch_pdl(latent_post_kernel<bf16, bf16>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else P3_CHECK_ARG(false, "latent_post: activations and cache must both be fp32 or both bf16");
    P3_CHECK_LAUNCH("latent_post");
    return 0;
}

extern "C" int p3_glu_silu(const float* g, const float* u, int64_t ld, void* out, int64_t ldo, int out_f32, int64_t R, int F,
                           cudaStream_t st) {
    if (R == 0 || F == 0) return 0;
    const bool vec = F % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)g & 15) == 0 && ((uintptr_t)u & 15) == 0 &&
                     ((uintptr_t)out & 15) == 0;
    const int64_t n = vec ? R * (F / 4) : R * F;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (vec) {
        if (out_f32) p3_launch_pdl(glu_silu_vec4_kernel<float>, dim3(grid), dim3(256), (size_t)(0), st, g, u, ld, (float*)out, ldo, R, F);
        else p3_launch_pdl(glu_silu_vec4_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), st, g, u, ld, (bf16*)out, ldo, R, F);
    } else if (out_f32) p3_launch_pdl(glu_silu_kernel<float>, dim3(grid), dim3(256), (size_t)(0), st, g, u, ld, (float*)out, ldo, R, F);
    else p3_launch_pdl(glu_silu_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), st, g, u, ld, (bf16*)out, ldo, R, F);
    P3_CHECK_LAUNCH("glu_silu");
    return 0;
}

extern "C" int p3_router_sigmoid_groups(const void* x, int64_t ldx, int x_f32, const float* Wr, const float* correction,
                                        const float* logits, int64_t ld_logits, int T, int W, int E, int top, int n_groups, int keep,
                                        float scale, int32_t* ids, float* wts, cudaStream_t st) {
    P3_CHECK_ARG(logits || (x && Wr), "router_sigmoid_groups: needs the logits, or the activations and the router matrix");
    P3_CHECK_ARG(top >= 1 && top <= E && E <= 1024, "router_sigmoid_groups: need 1 <= top <= experts <= 1024");
    const int NG = n_groups > 1 ? n_groups : 1;
    P3_CHECK_ARG(E % NG == 0 && (NG == 1 || (keep >= 1 && keep <= NG && keep * (E / NG) >= top)),
                 "router_sigmoid_groups: groups must divide the experts and the kept groups must hold `top` experts");
    if (T == 0) return 0;
    const int nw = logits ? 1 : (W >= 1024 ? 8 : 4);         // with ready logits one warp per token does everything
    const size_t sm = ((size_t)2 * E + NG + nw * 8) * sizeof(float);
    if (x_f32) p3_launch_pdl(router_sigmoid_groups_kernel<float>, dim3((unsigned)T), dim3(nw * 32), (size_t)(sm), st, (const float*)x, ldx, Wr, correction, logits, ld_logits, W, E, top, NG, keep, scale, 0, ids, wts);
    else p3_launch_pdl(router_sigmoid_groups_kernel<bf16>, dim3((unsigned)T), dim3(nw * 32), (size_t)(sm), st, (const bf16*)x, ldx, Wr, correction, logits, ld_logits, W, E, top, NG, keep, scale, 0, ids, wts);
    P3_CHECK_LAUNCH("router_sigmoid_groups");
    return 0;
}

extern "C" int p3_logit_softcap(float* logits, int64_t n, float scale, float cap, cudaStream_t st) {
    if (n == 0) return 0;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    p3_launch_pdl(logit_softcap_kernel, dim3(grid), dim3(256), (size_t)(0), st, logits, n, scale, cap);
    P3_CHECK_LAUNCH("logit_softcap");
    return 0;
}

extern "C" int p3_router_groups(const float* logits, int64_t ld_logits, const float* correction, int T, int E, int top, int n_groups,
                                int keep, float scale, int mode, int32_t* ids, float* wts, cudaStream_t st) {
    P3_CHECK_ARG(logits && ids && wts, "router_groups: null argument");
    P3_CHECK_ARG(top >= 1 && top <= E && E <= 1024, "router_groups: need 1 <= top <= outputs <= 1024");
    const int NG = n_groups > 1 ? n_groups : 1;
    P3_CHECK_ARG(E % NG == 0 && (NG == 1 || (keep >= 1 && keep <= NG && keep * (E / NG) >= top)),
                 "router_groups: groups must divide the outputs and the kept groups must hold `top` of them");
    if (T == 0) return 0;
    const size_t sm = ((size_t)2 * E + NG + 8) * sizeof(float);
    p3_launch_pdl(router_sigmoid_groups_kernel<float>, dim3((unsigned)T), dim3(32), (size_t)(sm), st, (const float*)nullptr, (int64_t)0,
                  (const float*)nullptr, correction, logits, ld_logits, 0, E, top, NG, keep, scale, mode, ids, wts);
    P3_CHECK_LAUNCH("router_groups");
    return 0;
}

extern "C" int p3_postnorm_prenorm(const float* y, int64_t ldy, const float* y_bias, const float* gain_post, float* x,
                                   const float* gain_pre, float* h32, void* h_act, int act_f32, int64_t T, int W, float eps,
                                   cudaStream_t st) {
    P3_CHECK_ARG(x && (!y || gain_post), "postnorm_prenorm: null argument");
    if (T == 0) return 0;
    const int th = W > 4096 ? 1024 : W > 2048 ? 512 : W >= 1024 ? 256 : 128;
    if (act_f32) p3_launch_pdl(postnorm_prenorm_kernel<float>, dim3((unsigned)T), dim3(th), (size_t)(0), st, y, ldy, y_bias, gain_post, x, gain_pre, h32, (float*)h_act, W, eps);
    else p3_launch_pdl(postnorm_prenorm_kernel<bf16>, dim3((unsigned)T), dim3(th), (size_t)(0), st, y, ldy, y_bias, gain_post, x, gain_pre, h32, (bf16*)h_act, W, eps);
    P3_CHECK_LAUNCH("postnorm_prenorm");
    return 0;
}

extern "C" int p3_token_shift(const float* h, const float* shift, float* state, const int32_t* seqs, const int32_t* slot_seq,
                              const int32_t* tok_slot, void* out, int out_f32, int64_t T, int W, cudaStream_t st) {
    P3_CHECK_ARG(h && shift && state && seqs && slot_seq && tok_slot && out, "token_shift: null argument");
    P3_CHECK_ARG(((uintptr_t)seqs & 15) == 0, "token_shift: the sequence records must be 16-byte aligned");
    if (T == 0) return 0;
    const int th = W >= 2048 ? 256 : 128;
    if (W % 4 == 0 && (((uintptr_t)h | (uintptr_t)shift | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
        if (out_f32) p3_launch_pdl(token_shift_vec4_kernel<float>, dim3((unsigned)T), dim3(th), (size_t)(0), st, h, shift, state, seqs, slot_seq, tok_slot, (float*)out, W);
        else p3_launch_pdl(token_shift_vec4_kernel<bf16>, dim3((unsigned)T), dim3(th), (size_t)(0), st, h, shift, state, seqs, slot_seq, tok_slot, (bf16*)out, W);
        P3_CHECK_LAUNCH("token_shift");
        return 0;
    }
    if (out_f32) p3_launch_pdl(token_shift_kernel<float>, dim3((unsigned)T), dim3(th), (size_t)(0), st, h, shift, state, seqs, slot_seq, tok_slot, (float*)out, W);
    else p3_launch_pdl(token_shift_kernel<bf16>, dim3((unsigned)T), dim3(th), (size_t)(0), st, h, shift, state, seqs, slot_seq, tok_slot, (bf16*)out, W);
    P3_CHECK_LAUNCH("token_shift");
    return 0;
}

extern "C" int p3_qkv_rope_post(const p3_qkv_rope_post_args* a, cudaStream_t st) {
    P3_CHECK_ARG(a && a->proj && a->q_out && a->k_pool && a->v_pool && a->block_table && a->tok_slot && a->tok_pos, "qkv_rope_post: null argument");
    P3_CHECK_ARG(a->rot_n >= 0 && a->rot_n % 2 == 0 && a->rot_n <= a->dim && (a->rot_n == 0 || a->freq), "qkv_rope_post: rot_n must be even and <= dim, with frequencies");
    P3_CHECK_ARG(a->v_off >= 0 || a->vdim == a->dim, "qkv_rope_post: keys that double as values need vdim == dim");
    if (a->T == 0) return 0;
    const int jobs = a->n_heads + a->n_kv + (a->v_off < 0 ? 0 : a->n_kv), th = 128;
    const int groups = a->T >= 1024 ? 1 : (jobs + 3) / 4;
    const dim3 grid((unsigned)a->T, (unsigned)groups);
    if (a->act_f32 && a->cache_f32) p3_launch_pdl(qkv_rope_kv_write_kernel<float, float>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else if (!a->act_f32 && !a->cache_f32) p3_launch_pdl(qkv_rope_kv_write_kernel<bf16, bf16>, dim3(grid), dim3(th), (size_t)(0), st, *a);
    else P3_CHECK_ARG(false, "qkv_rope_post: activations and cache must both be fp32 or both bf16");
    P3_CHECK_LAUNCH("qkv_rope_post");
    return 0;
}

extern "C" int p3_relu2(const float* u, int64_t ld, const float* row_gate, int64_t ld_gate, void* out, int64_t ldo, int out_f32,
                        int64_t R, int F, cudaStream_t st) {
    if (R == 0 || F == 0) return 0;
    if (F % 4 == 0 && ld % 4 == 0 && ldo % 4 == 0 && (((uintptr_t)u | (uintptr_t)out) & 15) == 0) {
        const int64_t n4 = R * (F / 4);
        const unsigned g4 = (unsigned)((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
        if (out_f32) p3_launch_pdl(relu2_vec4_kernel<float>, dim3(g4), dim3(256), (size_t)(0), st, u, ld, row_gate, ld_gate, (float*)out, ldo, R, F);
        else p3_launch_pdl(relu2_vec4_kernel<bf16>, dim3(g4), dim3(256), (size_t)(0), st, u, ld, row_gate, ld_gate, (bf16*)out, ldo, R, F);
        P3_CHECK_LAUNCH("relu2");
        return 0;
    }
    const int64_t n = R * F;
    const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (out_f32) p3_launch_pdl(relu2_kernel<float>, dim3(grid), dim3(256), (size_t)(0), st, u, ld, row_gate, ld_gate, (float*)out, ldo, R, F);
    else p3_launch_pdl(relu2_kernel<bf16>, dim3(grid), dim3(256), (size_t)(0), st, u, ld, row_gate, ld_gate, (bf16*)out, ldo, R, F);
    P3_CHECK_LAUNCH("relu2");
    return 0;
}

extern "C" int p3_moe_combine_identity(const float* y, int64_t ldy, const int32_t* where, const int32_t* ids, const float* wts, int top,
                                       int n_real, const float* h, const float* add, int64_t ld_add, float* out, int64_t T, int W,
                                       cudaStream_t st) {
    P3_CHECK_ARG(y && where && ids && wts && out, "moe_combine_identity: null argument");
    if (T == 0) return 0;
    p3_launch_pdl(moe_combine_identity_kernel, dim3((unsigned)T), dim3(W >= 1024 ? 256 : 128), (size_t)(2 * top * sizeof(float)), st,
                  y, ldy, where, ids, wts, top, n_real, h, add, ld_add, out, W);
    P3_CHECK_LAUNCH("moe_combine_identity");
    return 0;
}

extern "C" int p3_embed_pair_rows_f32(const void* table, const void* pair_table, const int32_t* ids, const int32_t* seqs,
                                      const int32_t* slot_seq, const int32_t* tok_slot, int32_t* prev_state, int64_t state_stride,
                                      float* x, int64_t T, int W, int vocab, float scale, int64_t buckets, int64_t mul_prev,
                                      int64_t mul_cur, cudaStream_t st) {
    P3_CHECK_ARG(table && ids && seqs && slot_seq && tok_slot && prev_state && x, "embed_pair_rows_f32: null argument");
    P3_CHECK_ARG(((uintptr_t)seqs & 15) == 0, "embed_pair_rows_f32: the sequence records must be 16-byte aligned");
    P3_CHECK_ARG(!pair_table || buckets >= 1, "embed_pair_rows_f32: the pair table needs at least one bucket");
    if (T == 0) return 0;
    if (!pair_table) buckets = 1;
    p3_launch_pdl(embed_pair_rows_kernel, dim3((unsigned)T), dim3(128), (size_t)(0), st, (const bf16*)table, (const bf16*)pair_table, ids, seqs,
                  slot_seq, tok_slot, prev_state, state_stride, x, W, vocab, scale, (long long)buckets, (long long)mul_prev, (long long)mul_cur);
    P3_CHECK_LAUNCH("embed_pair_rows_f32");
    return 0;
}

extern "C" int p3_distance_linear_table(const float* slope, float* pen, int H, int n, cudaStream_t st) {
    P3_CHECK_ARG(slope && pen && H >= 1 && n >= 1, "distance_linear_table: bad argument");
    const int64_t tot = (int64_t)H * n;
    distance_linear_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(slope, pen, H, n);
    P3_CHECK_LAUNCH("distance_linear_table");
    return 0;
}
