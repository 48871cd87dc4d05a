/* phi3_b200.h — C ABI of libphi3b200.so (sm_100a only).
 *
 * The reference (JosefAlbers/Phi-3-Vision-MLX) has no FFI/plugin layer: its hot path calls
 * mlx==0.15 ops from Python. Each entry below replaces one of those MLX call
 * sites; the cited lines are in /root/reference/phi.py (phi:) and
 * /root/reference/phi_3_vision_mlx.py (pv:). INTEGRATION.md shows the ctypes binding a
 * maintainer of the reference would add.
 *
 * Conventions: plain device pointers + sizes, caller-owned memory and workspaces, no
 * allocation and no host synchronisation inside, stream-ordered and CUDA-graph capturable.
 * Every function returns 0 on success, <0 on error; p3_last_error() gives the message
 * (thread-local). bf16 = __nv_bfloat16 storage. "Rows" are tokens (B*L flattened).
 */
#ifndef PHI3_B200_H
#define PHI3_B200_H
#include <stdint.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GEMM epilogues (p3_gemm, p3_gemm_skinny) */
#define P3_EPI_NONE 0       /* out bf16 = acc (+bias) */
#define P3_EPI_QGELU 1      /* bias + x*sigmoid(1.702x)         nn.gelu_fast_approx, phi:154 */
#define P3_EPI_GELU 2       /* bias + exact erf GELU            nn.GELU(), phi:391 */
#define P3_EPI_RESIDUAL 3   /* out = resid + bf16(acc+bias)     phi:170-171, 483, 485 */
#define P3_EPI_SWIGLU 4     /* out[:, N/2] = silu(gate)*up      phi:470-471, interleaved W (see p3_gemm) */
#define P3_EPI_F32 5        /* out fp32 = acc (+bias)           lm_head logits, phi:608 */
#define P3_EPI_RESIDUAL_F32 6 /* out fp32 = resid fp32 + acc+bias  CLIP residual stream (fp32 in the reference) */

#define P3_PAGE_TOKENS 64   /* tokens per KV page */

const char* p3_last_error(void);
int p3_version(void);
/* Diagnostics (tools/chain_trace.py), not part of the reference interface: with a device buffer of n_slots x 1024 x 8 uint64 set,
 * every decode-path launch (skinny GEMMs, decode attention) takes the next slot and its CTAs store globaltimer stamps
 * {start, dependency resolved, first operands ready, main loop done, exit, smid, kind, grid}. p3_trace_set(NULL, 0) turns it off. */
int p3_trace_set(void* buf, int n_slots);
int p3_trace_count(void);

/* nn.Embedding phi:568,577 — ids<0 (image placeholders, phi:270) read row 0. ss_out (fp32 [T], may be
 * NULL) receives each row's sum of squares for the RMSNorm fused into the next p3_gemm_skinny. */
int p3_embed_gather(const void* table, const int32_t* ids, void* out, int64_t T, int H, int vocab, float* ss_out,
                    cudaStream_t st);

/* nn.RMSNorm / mx.fast.rms_norm phi:478-479,571 */
int p3_rmsnorm(const void* x, const void* w, void* y, int64_t T, int H, float eps, cudaStream_t st);

/* nn.LayerNorm / mx.fast.layer_norm phi:165,167,212. x fp32 (CLIP residual stream);
 * y bf16 (out_f32 = 0, feeds a GEMM) or fp32 (out_f32 = 1, pre_layrnorm phi:218). */
int p3_layernorm(const float* x, const void* w, const void* b, void* y, int64_t T, int H, float eps, int out_f32,
                 cudaStream_t st);

/* _rotate_half + SuRoPE table + KVCache slice-assign: phi:418-423, 487-507, 542-548.
 * qkv [B*L, (n_heads+2*n_kv)*hd] bf16 roped in place; cos/sin fp32 [Bt, L_all, hd/2];
 * tab_bstride = 0 for a shared table, else elements between table rows; row b uses
 * table/cache row b/row_div (row_div = n_beam, phi:447-450). pool = this layer's page pool
 * [page][2][n_kv][64][hd]; block_table int32 [n_seq, bt_stride]. past_dev (device int32, may be
 * NULL) overrides `past` at run time so a captured CUDA graph can be replayed every step. */
int p3_rope_kvwrite(void* qkv, const float* cosT, const float* sinT, int64_t tab_bstride, int B, int L, int n_heads,
                    int n_kv, int hd, int past, int row_div, void* pool, const int32_t* block_table, int bt_stride,
                    int write_cache, const int32_t* past_dev, cudaStream_t st);

/* mx.argmax pv:386,392,506,559; nn.log_softmax + gathers pv:476,541-547,571-573;
 * mx.argpartition top-n pv:507 — one pass per logits row. Any output pointer may be NULL. */
int p3_row_stats(const float* logits, int64_t R, int64_t ld, int V, int32_t* argmax_out, float* max_out,
                 float* lse_out, int n_top, int32_t* topk_ids, float* topk_lp, int n_gather,
                 const int32_t* gather_ids, float* gather_lp, cudaStream_t st);

/* Nucleus (top-p) sampling — extension: the reference decodes greedily only (pv:386,392).
 * tau = largest probability v with sum_{p_i>=v} p_i >= top_p (exact bisection, no sort); token drawn by
 * inverse CDF in index order over {p_i >= tau} with the caller's uniform u[R] in [0,1). tau_out may be NULL.
 * step_dev (device int32, may be NULL): u is a table and row *step_dev * u_stride is used (graph replay). */
int p3_top_p_sample(const float* logits, int64_t R, int64_t ld, int V, float top_p, float temperature, const float* u,
                    int32_t* out, float* tau_out, const int32_t* step_dev, int64_t u_stride, cudaStream_t st);

/* Greedy-loop bookkeeping on the device (pv:390-398 without the two host syncs per token):
 * history[b][*step] = tok[b]; eos_seen[b] |= (tok[b]==32007); ++*step; ++*past (past may be NULL). */
int p3_decode_advance(const int32_t* tok, int32_t* history, int64_t ld, int B, int32_t* step, int32_t* past,
                      int32_t* eos_seen, cudaStream_t st);

/* nn.Linear at decode (M<=16 tokens): phi:437-438,465-466,604. Optional fused RMSNorm prologue
 * (norm_w != NULL: X is the raw hidden state). epi in {NONE, RESIDUAL, SWIGLU, F32}.
 * ss_in (fp32 [n_ss_in][16], may be NULL): per-token partial sums of squares of X written by the
 * kernel that produced X (p3_embed_gather / a RESIDUAL p3_gemm_skinny via ss_out, which writes
 * [ceil(N/16)][16]); without it the RMSNorm statistic is recomputed from X.
 * l2_prefetch (may be NULL): the NEXT kernel's weights; every CTA pulls a slice into L2 before it waits on its
 * predecessor, so HBM keeps streaming across the kernel boundary (own weights are loaded L2::evict_first). */
int p3_gemm_skinny(const void* X, int64_t ldx, const void* norm_w, float eps, const void* W, void* out, int64_t ldo,
                   const void* resid, int M, int N, int K, int epi, const float* ss_in, int n_ss_in, float* ss_out,
                   const void* l2_prefetch, int64_t l2_prefetch_bytes, cudaStream_t st);

/* Decode-time qkv_proj + _rotate_half/SuRoPE + KVCache write in ONE launch (phi:442-453): each CTA owns
 * 16 rotary pairs (column c and c + hd/2 of one head) so the rotation fuses into the epilogue. */
int p3_gemm_skinny_qkv_rope(const void* X, int64_t ldx, const void* norm_w, float eps, const void* Wqkv, void* qkv,
                            const float* ss_in, int n_ss_in, const float* cosT, const float* sinT, int64_t tab_bstride,
                            int B, int L, int n_heads, int n_kv, int hd, int K, int past, const int32_t* past_dev,
                            int row_div, void* pool, const int32_t* block_table, int bt_stride, int write_cache,
                            const void* l2_prefetch, int64_t l2_prefetch_bytes, cudaStream_t st);

/* quantize_model=True (pv:264,291-305: nn.quantize(model, group_size=64, bits=4) -> QuantizedLinear): the two decode-time
 * entries above over the 4-bit image of W. Wq uint8 [N][K/2] and Wmeta bf16 [N][K/64][2] = (scale, bias) in the lane order
 * written by phi3_b200/quant.py::pack_w4g64; y = sum_k x_k (scale_g q_k + bias_g) accumulated in fp32 (codes and a
 * matrix of ones go through the tensor cores per 64-wide group, the affine map is applied to the group sums). K % 128 == 0.
 * Prefill / ViT GEMMs of a quantised model run p3_gemm on the bf16 dequantised image. */
int p3_gemm_skinny_w4(const void* X, int64_t ldx, const void* norm_w, float eps, const void* Wq, const void* Wmeta, void* out,
                      int64_t ldo, const void* resid, int M, int N, int K, int epi, const float* ss_in, int n_ss_in,
                      float* ss_out, const void* l2_prefetch, int64_t l2_prefetch_bytes, cudaStream_t st);
int p3_gemm_skinny_qkv_rope_w4(const void* X, int64_t ldx, const void* norm_w, float eps, const void* Wq, const void* Wmeta,
                               void* qkv, const float* ss_in, int n_ss_in, const float* cosT, const float* sinT,
                               int64_t tab_bstride, int B, int L, int n_heads, int n_kv, int hd, int K, int past,
                               const int32_t* past_dev, int row_div, void* pool, const int32_t* block_table, int bt_stride,
                               int write_cache, const void* l2_prefetch, int64_t l2_prefetch_bytes, cudaStream_t st);

/* nn.Linear for prefill / ViT / projector (phi:140-143,155-156,391,437-438,465-466,604) and the
 * patch-embed conv as GEMM (phi:186-192): out[M,N] = X[M,K] . W[N,K]^T on tcgen05 tensor cores
 * (TMA -> smem -> tcgen05.mma -> TMEM -> epilogue). bias bf16 [N] or NULL. row_map int32 [M] or
 * NULL scatters output rows (image-feature splice, phi:412-415). For P3_EPI_SWIGLU W must be in
 * the interleaved layout (per 256 rows: 128 gate rows then the matching 128 up rows) and out is
 * [M, N/2]. impl: 0 = tcgen05 (product path), 1 = mma.sync cross-check kernel (tests only). */
int p3_gemm(const void* X, int64_t ldx, const void* W, int64_t ldw, const void* bias, void* out, int64_t ldo,
            const void* resid, const int32_t* row_map, int64_t M, int N, int K, int epi, int impl, cudaStream_t st);

/* Prefill / ViT flash attention: phi:454-457 (causal + left-pad predicate instead of Mask4D
 * phi:550-563) and mx.fast.scaled_dot_product_attention phi:148 (causal=0).
 * q/k/v point into the (roped) qkv buffer; row strides in elements; head h at +h*hd.
 * Keys [0,past) come from the paged pool (cache row b/row_div), keys [past,past+L) from k/v.
 * kv_start int32 [B] (left-pad length; NULL = 0). Pad queries produce zeros.
 * Runs the tcgen05 flash-attention kernel (S and P in TMEM, TMA operands) when past % 64 == 0, L >= 64 and
 * the pointers / strides are 16-byte aligned; otherwise (and with P3_ATTN_TC=0 in the environment, used by the
 * tests as a cross-check) the mma.sync kernel with the same contract. */
int p3_attention_prefill(const void* q, const void* k, const void* v, int64_t ldq, int64_t ldk, int64_t ldv, void* out,
                         int64_t ldo, int B, int L, int n_heads, int n_kv, int hd, float scale, int causal, int past,
                         const int32_t* kv_start, const void* pool, const int32_t* block_table, int bt_stride,
                         int row_div, cudaStream_t st);

/* Decode-time attention for L<=16 new tokens per row over a paged KV cache (split-KV):
 * phi:454-457 with KVCache reads phi:523-527 (n_beam shared prefix: row_div) / phi:548.
 * workspace: p3_attention_decode_workspace() bytes, MUST be zero-filled once before first use (it holds the
 * split-arrival counters, which the kernel resets itself); needed when n_splits > 1.
 * l2_prefetch (may be NULL): l2_prefetch_bytes of the NEXT kernel's weights (o_proj) that the CTAs pull into
 * L2 (prefetch.global.L2::evict_last) while the KV pages stream. */
/* Struct-argument form of p3_gemm_skinny / p3_gemm_skinny_w4 / p3_gemm_skinny_qkv_rope(_w4) with the RMSNorm split between
 * producer and consumer (decode over 4-bit weights, phi:478-485 with QuantizedLinear pv:264): a RESIDUAL launch with xg_out also
 * writes xg_out[m][n] = bf16(h[m][n] * xg_gain[n]) (xg_gain = weight of the NEXT RMSNorm); the consumer takes that as X with
 * norm_w = NULL and rs_epi = 1 and multiplies its reduced accumulators by rsqrt(sum(ss_in[.][m]) / K + eps). */
typedef struct {
    int32_t op;                          /* 0: out = epi(X W^T);  1: qkv projection + SuRoPE + paged KV write */
    const void* X; int64_t ldx;
    const void* norm_w; float eps;
    const void* W;                       /* bf16 [N][K], or NULL when Wq / Wmeta (4-bit g64 image) are given */
    const void* Wq; const void* Wmeta;
    void* out; int64_t ldo; const void* resid;
    int32_t M, N, K, epi;                /* op 1: N, M, ldo, epi are derived (M = B * L) */
    const float* ss_in; int32_t n_ss_in; float* ss_out;
    const void* l2_prefetch; int64_t l2_prefetch_bytes;
    const void* xg_gain; void* xg_out; int64_t ldxg; int32_t rs_epi;
    const float* cosT; const float* sinT; int64_t tab_bstride;          /* op 1, as p3_gemm_skinny_qkv_rope */
    int32_t B, L, n_heads, n_kv, hd, past, row_div, bt_stride, write_cache;
    const int32_t* past_dev; void* pool; const int32_t* block_table;
    int32_t packed;                      /* op 0, bf16 W, N % 16 == 0, N < 9472, not SwiGLU: W is given in stream order
                                          * [N/16 tiles][K/64 chunks][row half][k half][lane = 4 * (row % 8) + 16-byte quad][8 bf16]
                                          * (one contiguous 16 x K block per tile; phi3_b200.model.pack_rows16) */
} p3_skinny_args;
int p3_gemm_skinny_x(const p3_skinny_args* args, cudaStream_t st);
/* p3_embed_gather that also writes xg_out[t] = bf16(row * xg_gain) (input of the first rs_epi consumer) */
int p3_embed_gather_xg(const void* table, const int32_t* ids, void* out, int64_t T, int H, int vocab, float* ss_out,
                       const void* xg_gain, void* xg_out, cudaStream_t st);

int64_t p3_attention_decode_workspace(int B, int L, int n_heads, int hd, int n_splits);
int p3_attention_decode(const void* q, const void* k, const void* v, int64_t ldq, int64_t ldk, int64_t ldv, void* out,
                        int64_t ldo, int B, int L, int n_heads, int n_kv, int hd, float scale, int past,
                        const int32_t* kv_start, const void* pool, const int32_t* block_table, int bt_stride,
                        int row_div, int n_splits, void* workspace, const int32_t* past_dev, const void* l2_prefetch,
                        int64_t l2_prefetch_bytes, cudaStream_t st);

/* 4-bit g32 KV-cache quantisation (mx.quantize/dequantize, phi:532,536-537). Quantises the
 * first n_tokens positions of the bf16 pool pages of each cache row in place into a q4 pool
 * ([page][2][n_kv][64][hd/2 bytes] codes + [page][2][n_kv][64][hd/32][2] bf16 scale,bias). */
int p3_kv_quantize_q4g32(const void* pool, void* qcodes, void* qmeta, const int32_t* block_table, int bt_stride,
                         int n_seq, int n_tokens, int n_kv, int hd, cudaStream_t st);
int p3_attention_decode_q4(const void* q, const void* k, const void* v, int64_t ldq, int64_t ldk, int64_t ldv,
                           void* out, int64_t ldo, int B, int L, int n_heads, int n_kv, int hd, float scale, int past,
                           int n_quant, const int32_t* kv_start, const void* pool, const void* qcodes,
                           const void* qmeta, const int32_t* block_table, int bt_stride, int row_div, int n_splits,
                           void* workspace, const int32_t* past_dev, const void* l2_prefetch, int64_t l2_prefetch_bytes,
                           cudaStream_t st);

/* Vision front end. */
/* PIL BILINEAR resize (phi:299), white pad to x336 (phi:300-306), (x/255-mean)/std (phi:309):
 * src uint8 HWC with element strides (sx, sy) so a transposed view needs no copy (phi:295,308).
 * coefficient tables are built on the host exactly as Pillow's precompute_coeffs does. */
int p3_hd_resize_h(const uint8_t* src, int64_t sy, int64_t sx, int in_w, int in_h, uint8_t* tmp, int out_w,
                   const int32_t* bounds, const int32_t* kk, int ksize, cudaStream_t st);
/* vertical pass + white pad (pad_top rows above, to padded_h) + optional un-transpose; writes the
 * padded uint8 HWC image ([padded_h, tmp_w, 3], or [tmp_w, padded_h, 3] when transposed). */
int p3_hd_resize_v_pad(const uint8_t* tmp, int tmp_w, int tmp_h, int out_h, const int32_t* bounds, const int32_t* kk,
                       int ksize, int pad_top, int padded_h, int transposed, uint8_t* out_hwc, cudaStream_t st);
/* normalise through a 256x3 float64 LUT ((v/255-mean)/std, phi:309), sub-crop tiling (phi:322-326)
 * and the reference's 2-tap interpolate_336 global crop (phi:331-372, float64 accumulate) into
 * pixel_values [n_crops+1, 3, 336, 336] fp32 (crop 0 = global). idx/wgt tables are [336][2]. */
int p3_hd_tile_crops(const uint8_t* img_hwc, int H, int W, const double* lut, float* pixel_values,
                     const int32_t* h_idx, const float* h_wgt, const int32_t* w_idx, const float* w_wgt,
                     cudaStream_t st);
/* im2col for the 14x14/14 patch conv (phi:186-192,199): pixel_values [N,3,336,336] fp32 ->
 * A [N*576, Kpad] bf16, k = (ky*14+kx)*3 + c (NHWC weight order, pv:374), zero padded. */
int p3_patch_im2col(const float* pixel_values, void* A, int N, int Kpad, cudaStream_t st);
/* cat[class_emb, patches] + position_embedding (phi:202-205): patches fp32 [N*576, D] -> fp32 [N,577,D] */
int p3_clip_embed(const float* patches, const void* cls, const void* pos, float* out, int N, int D, cudaStream_t st);
/* drop CLS (phi:221) + 2x2 token merge + sub_GN/glb_GN separators (phi:403-407):
 * feats fp32 [n_crops+1, 577, C] (crop 0 = global) -> bf16 [(hc*wc+1)*144 + 1 + (hc+1)*12, 4*C] */
int p3_gn_assemble(const float* feats, const void* sub_GN, const void* glb_GN, void* out, int hc, int wc, int C,
                   cudaStream_t st);

/* ------------------------------------------------------------------------------------------------
 * Struct-argument GEMM entry with the fused prefill epilogues (north_star: "SuRoPE fused into the QKV epilogue",
 * "RMSNorm and residual fused with adjacent ops"); replaces nn.RMSNorm + nn.Linear + _rotate_half + KVCache slice-assign at
 * prefill: phi:442-453, 478-485.
 *   - ss_in / n_ss_in / eps: RMSNorm of the INPUT rows is applied as a per-row scale rsqrt(sum_c ss_in[row][c] / K + eps) on the
 *     accumulators; the gain must already be folded into W (W'[n][k] = W[n][k] * g[k]). ss_in rows hold partial sums of
 *     squares of X's rows (p3_row_sumsq, or the ss_out of the GEMM that produced X).
 *   - ss_out (P3_EPI_RESIDUAL): fp32 [M][N/32], sum of squares of every 32-column chunk written.
 *   - P3_EPI_ROPE_KV: out = qkv [M, N] bf16 with q,k rotated, K/V also written to the page pool (as p3_rope_kvwrite). The q
 *     and k rows of W must be permuted per head to [16j..16j+15 | half+16j..half+16j+15], j = 0..hd/32-1 (so a rotary pair
 *     meets in one 32-column chunk of the accumulator); v rows keep their order.
 *   - splitk_ws: see the field comment (deterministic split-K: partials are summed in slice order by the last CTA of a tile).
 *   - w_plan: NULL, or a P3_GEMM_WPLAN_BYTES blob filled once by p3_gemm_plan_weights for this W (skips re-encoding the
 *     weight tensor map on every call). */
#define P3_EPI_ROPE_KV 8
#define P3_GEMM_WPLAN_BYTES 320
typedef struct {
    const void* X; int64_t ldx;
    const void* W; int64_t ldw;
    const void* bias; void* out; int64_t ldo;
    const void* resid; const int32_t* row_map;
    int64_t M; int32_t N, K, epi, impl;
    const float* ss_in; int32_t n_ss_in; float eps;
    float* ss_out;
    const void* w_plan;
    /* P3_EPI_ROPE_KV (M = B*L rows, token i of row b at position past+i; table / cache row b/row_div) */
    const float* cosT; const float* sinT; int64_t tab_bstride;
    int32_t L, n_heads, n_kv, hd, past, row_div, write_cache, bt_stride;
    const int32_t* past_dev;
    void* pool; const int32_t* block_table;
    /* split-K for shapes with few output tiles (M <= 128 ...): NULL, or a caller-owned device workspace whose first 4 KB are
     * zero before the first use (per-tile arrival counters, left at zero by every launch) followed by room for the fp32
     * partial tiles (32 MB covers Phi-3.5 shapes). Without it such shapes run on as many SMs as they have tiles. */
    void* splitk_ws; int64_t splitk_ws_bytes;
} p3_gemm_args;
int p3_gemm_plan_weights(const void* W, int64_t ldw, int N, int K, void* plan);
int p3_gemm_fused(const p3_gemm_args* args, cudaStream_t st);
/* SuRoPE cos/sin table phi:487-507 on the device: cosT/sinT fp32 [Bt, L_all, half]; positions 0..L_all-1 (pids NULL) or per row
 * cat[pids[b, 0..Lp), pids[b, Lp-1] + 1 + arange] (phi:493-497); inv_freq fp32 [half] = 1 / (factor * theta^(2i/dim)). */
int p3_rope_table(const int32_t* pids, int64_t pid_stride, int Lp, const float* inv_freq, float* cosT, float* sinT, int Bt,
                  int L_all, int half, float scale, cudaStream_t st);
/* fp32 out[row] = sum of squares of bf16 x[row, 0..H) (feeds ss_in with n_ss_in = 1) */
int p3_row_sumsq(const void* x, int64_t ldx, float* out, int64_t T, int H, cudaStream_t st);

/* ------------------------------------------------------------------------------------------------
 * Persistent decode-layer kernel (decode_mega.cu): for M <= 8 decode rows, ONE launch of n_ctas (<= #SM,
 * co-resident) persistent CTAs runs up to 4 chained weight-stream phases with grid barriers in between,
 * e.g. o_proj(+residual) -> RMSNorm+gate_up(+SwiGLU) -> down_proj(+residual) -> RMSNorm+qkv_proj(+SuRoPE
 * +paged KV write) of the next layer, or ... -> RMSNorm+lm_head. Replaces nn.Linear / nn.RMSNorm /
 * _rotate_half / KVCache slice-assign at decode: phi:437-438, 442-453, 460, 465-471, 478-485, 604-608.
 * Arguments travel in a plain-old-data struct (device pointers + sizes), as SURVEY.md par. 8b asks. */
#define P3_MEGA_RESID 0     /* out[M,N] bf16 = bf16(out + bf16(x W^T)) in place; ss_out[tile][16] = sum of squares of the 16 new columns */
#define P3_MEGA_SWIGLU 1    /* W = [gate rows | up rows] (phi:470); out[M,N/2] bf16 = silu(gate) * up */
#define P3_MEGA_QKV_ROPE 2  /* out[M,N] bf16 = qkv with q,k rotated (phi:418-423) + K,V written to the page pool at `past` */
#define P3_MEGA_F32 3       /* out[M,N] fp32 logits */
#define P3_MEGA_MAX_PHASES 4

typedef struct {
    const void* wp;             /* weights in stream order (p3_mega_pack), N*K bf16 */
    int32_t kind, N, K;         /* N = rows of W (output features, SWIGLU: gate+up), K = input features */
    int32_t max_tiles_per_cta;  /* max over CTAs of the schedule below (checked against the smem partial buffer when K > 4096) */
    const void* x;              /* input activations bf16 [M, ldx] */
    int64_t ldx;
    const void* norm_w;         /* RMSNorm gain applied to x on load (bf16 [K]) or NULL */
    const float* ss_in;         /* per-row sum-of-squares partials of x: fp32 [n_ss_in][16]; NULL = recompute from x */
    int32_t n_ss_in, _pad;
    float* ss_out;              /* RESID: partials [N/16][16] of the rows written, or NULL */
    void* out;
    int64_t ldo;
    const int32_t* cta_off;     /* schedule: CTA c owns tile_ids[cta_off[c] .. cta_off[c+1]) of this phase (int32 [n_ctas+1]) */
    const int32_t* tile_ids;    /* tile = 16 (RESID) or 2x16 (other kinds) rows of W */
} p3_mega_phase;

typedef struct {
    p3_mega_phase ph[P3_MEGA_MAX_PHASES];
    int32_t n_phases, M;
    float eps;                  /* RMSNorm eps */
    int32_t n_ctas;             /* grid size the schedule was built for (<= #SM) */
    uint32_t* sync;             /* 2 words of device memory, zero before the first launch (grid barrier state) */
    /* P3_MEGA_QKV_ROPE: one new token per row at position *past_dev (or `past` when NULL) */
    const float* cosT;
    const float* sinT;          /* fp32 [Bt, L_all, hd/2]; row b uses table row b (tab_bstride elements apart, 0 = shared) */
    int64_t tab_bstride;
    int32_t n_heads, n_kv, hd, past;
    const int32_t* past_dev;
    void* pool;                 /* this layer's page pool [page][2][n_kv][64][hd] bf16 */
    const int32_t* block_table; /* int32 [M, bt_stride] */
    int32_t bt_stride, _pad2;
    long long* dbg;             /* NULL, or int64 [n_ctas][4][8]: per-CTA / per-phase SM-clock stamps (tools/mega_trace.py) */
} p3_mega_args;

/* W [N,K] bf16 (nn.Linear layout; SWIGLU: the checkpoint's [gate | up] row order) -> stream order for `kind` */
int p3_mega_pack(const void* W, void* out, int kind, int N, int K, int n_heads, int n_kv, int hd, cudaStream_t st);
/* number of SMs of the current device = the largest valid n_ctas */
int p3_decode_mega_ctas(void);
int p3_decode_mega(const p3_mega_args* args, cudaStream_t st);

/* ------------------------------------------------------------------------------------------------------------------------
 * Decoders with an fp32 residual stream, a ragged token batch and a page pool shared by all live sequences (Tagenex and any
 * design built from the same parts). "act" tensors are bf16, or fp32 in the all-fp32 serving mode (act_f32 / cache_f32 = 1);
 * norms, softmax, router and residual sums are fp32 in both. One K pool and one V pool per layer:
 * [page][kv head][P3_PAGE_TOKENS][dim | vdim]; block_table int32 [sequence slot][bt_stride] of page ids. */

/* out[M,N] = X[M,K] W[N,K]^T + bias for any sizes / strides / alignment; X and W both fp32 (FMA pipes, no TF32) or both bf16
 * (mma.sync when K, ldx, ldw are multiples of 8 and the bases 16-byte aligned, else FMA); fp32 accumulation in ascending k.
 * x_rows (may be NULL): row r reads X[x_rows[r] / x_row_div]. seg_offsets (device int32 [n_groups + 1], may be NULL): rows
 * [seg[g], seg[g+1]) multiply with W + g * w_group_stride and add bias + g * bias_group_stride (grouped expert product; M is
 * then the total row count = seg[n_groups]). bias fp32 or NULL.
 * n_batch > 1: that many independent products in one launch (per-head products of an attention mixer); product b reads X, W and
 * writes out at the element offsets b * x_batch_stride, b * w_batch_stride, b * out_batch_stride (column blocks of wider
 * matrices). gate (fp32 logits [M, ld_gate], may be NULL): out <- out * sigmoid(gate[m][b * out_batch_stride + n]). */
typedef struct {
    const void* X; int64_t ldx; int32_t x_f32; const int32_t* x_rows; int32_t x_row_div;
    const void* W; int64_t ldw; int32_t w_f32; int64_t w_group_stride;
    const float* bias; int64_t bias_group_stride;
    void* out; int64_t ldo; int32_t out_f32;
    int64_t M; int32_t N, K;
    const int32_t* seg_offsets; int32_t n_groups;
    int32_t force_fma;           /* tests: bf16 operands on the FMA kernel */
    int32_t n_batch; int64_t x_batch_stride, w_batch_stride, out_batch_stride;
    const float* gate; int64_t ld_gate;
} p3_gemm_any_args;
int p3_gemm_any(const p3_gemm_any_args* args, cudaStream_t st);

/* x fp32 [T,W] = table[ids] * scale (bf16 table); x_act (may be NULL; row pitch ld_act) receives the same rows in the activation
 * type */
int p3_embed_rows_f32(const void* table, const int32_t* ids, float* x, void* x_act, int act_f32, int64_t T, int W, int vocab,
                      float scale, int64_t ld_act, cudaStream_t st);
/* norm on a sublayer's OUTPUT: y' = y + y_bias (y_bias fp32 [W] or NULL: a bias the producing product left out);
 * x += y' / sqrt(mean(y'^2) + eps) * gain; x_act (may be NULL) = the new x in the activation type */
int p3_postnorm_residual(const float* y, int64_t ldy, const float* y_bias, const float* gain, float* x, void* x_act, int act_f32,
                         int64_t T, int W, float eps, cudaStream_t st);
/* out[r] = rms_norm(x[rows[r]]) * gain (rows NULL: r itself): the model's last norm, only for the rows whose logits are wanted */
int p3_rmsnorm_rows_f32(const float* x, const int32_t* rows, const float* gain, void* out, int out_f32, int64_t R, int W, float eps,
                        cudaStream_t st);

/* After the fused q|k|v|gate projection (proj fp32 [T, ld_proj], column offsets *_off): per-head RMS norm of q and k with gains
 * shared by all heads, q -> q_out (act), k -> K pool; v_mode 0: v -> V pool, 1: also kept in v_first (fp32 [T, n_kv * vdim]),
 * 2: v <- (1 - v_lambda) v + v_lambda v_first before it is cached; gate_out (may be NULL) fp32 [T, n_heads] = sigmoid(gate
 * logits). Token t of the batch belongs to sequence slot tok_slot[t] at position tok_pos[t]. */
typedef struct {
    const float* proj; int64_t ld_proj; int32_t q_off, k_off, v_off, g_off;
    int32_t n_heads, n_kv, dim, vdim;
    const float* q_gain; const float* k_gain; float eps;
    float* v_first; int32_t v_mode; float v_lambda;
    void* q_out; int64_t ld_q; float* gate_out;
    void* k_pool; void* v_pool; const int32_t* block_table; int32_t bt_stride;
    const int32_t* tok_slot; const int32_t* tok_pos; int32_t T;
    int32_t act_f32, cache_f32;
    const float* bias;             /* fp32 indexed like proj's columns, or NULL: added to q, k and v before anything else */
    float q_temp_coef; int32_t q_temp_every;   /* every > 0: the normed query at position p is multiplied by
                                      1 + coef * ln(floor((p + 1) / every) + 1) */
} p3_qkv_post_args;
int p3_qkv_post(const p3_qkv_post_args* args, cudaStream_t st);

/* Sliding-window attention with sink and distance penalty over the page pools (csrc/attention_window.cu). tiles = int32 x 4 per
 * CTA row: {first batch row, number of query rows (<= 32; decode: 1), sequence slot, position of the first row}. window 0 = no
 * limit. sink fp32 [n_heads] or NULL; penalty fp32 [n_heads][n_penalty] (value at distance i - j, clamped to the table) or NULL;
 * gate fp32 [T, n_heads] or NULL multiplies the head outputs. out (act) [T, ld_out], head h at column h * vdim. */
typedef struct {
    const void* q; int64_t ld_q;
    const void* k_pool; const void* v_pool; const int32_t* block_table; int32_t bt_stride;
    const float* sink; const float* penalty; int32_t n_penalty; const float* gate;
    void* out; int64_t ld_out;
    int32_t n_heads, n_kv, dim, vdim; float scale; int32_t window;
    int32_t act_f32, cache_f32;
    const int32_t* tiles; int32_t n_tiles;
    int32_t n_splits; float* ws;   /* decode only: key slices per request (<= 1: none) and their workspace, fp32
                                      [n_tiles][n_heads][n_splits][vdim + 2] */
    int32_t v_ld;                  /* elements between the value rows of a page (0: vdim). With v_pool == k_pool and v_ld == dim
                                      the values are the leading vdim numbers of the key rows (one latent vector per token that
                                      serves as key and as value) */
    int32_t keep_first;            /* with a window: keys at positions < keep_first stay visible to every later query (at their
                                      true positions); 0: none */
    const float* sig_bias;         /* fp32 [n_heads] or NULL. Not NULL: no softmax; the weight of a visible key is
                                      sigmoid(score + sig_bias[h]) and the weights are not normalised over the keys (sink unused) */
    float out_scale;               /* factor on the head outputs (0 is read as 1) */
    const float* elem_gate; int64_t ld_elem_gate;   /* fp32 logits [T, ld_elem_gate] or NULL: output column c of a row (head h at
                                      column h * vdim) is multiplied by sigmoid(elem_gate[row][c]) */
} p3_attn_window_args;
/* query rows per tile that p3_attn_window_prefill takes for these sizes: 64 on its tensor-core path, else 32 */
int p3_attn_window_tile_rows(const p3_attn_window_args* args);
int p3_attn_window_prefill(const p3_attn_window_args* args, cudaStream_t st);
int p3_attn_window_decode(const p3_attn_window_args* args, cudaStream_t st);

/* out (act) [R, F] = g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit) with
 * g = gu[:, :F] + bias[:F], u = gu[:, F:2F] + bias[F:] (bias fp32 [2F] or NULL) */
int p3_glu_clamped(const float* gu, int64_t ld, void* out, int64_t ldo, int out_f32, int64_t R, int F, float limit, float alpha,
                   const float* bias, cudaStream_t st);
/* router: z = Wr x + br in fp32; the `top` largest (ties: lower index) -> ids [T, top]; wts = softmax over the chosen logits */
int p3_router_topk(const void* x, int64_t ldx, int x_f32, const float* Wr, const float* br, int T, int W, int E, int top, int32_t* ids,
                   float* wts, cudaStream_t st);
/* stable sort of the n = T * top (token, choice) pairs by expert: seg [E + 1], order [n] (sorted row -> pair), where [n] (pair ->
 * sorted row); feeds p3_gemm_any's segments and p3_moe_combine */
int p3_moe_sort(const int32_t* ids, int n, int E, int32_t* seg, int32_t* order, int32_t* where, cudaStream_t st);
/* out[r] = x[rows[r] / div] (activation rows brought into expert order for per-expert dense products) */
int p3_gather_rows(const void* x, int64_t ldx, int x_f32, const int32_t* rows, int div, void* out, int64_t R, int W, cudaStream_t st);
int p3_moe_combine(const float* y, int64_t ldy, const int32_t* where, const float* wts, int top, float* out, int64_t T, int W,
                   cudaStream_t st);
/* pen[h][i] = r1[h] * ln(1 + r2[h] * i), i < n */
int p3_distance_penalty_table(const float* r1, const float* r2, float* pen, int H, int n, cudaStream_t st);


/* ---- parts of decoders whose layers read ONE layer norm (weight and bias) and add all sublayer outputs at once, with a
 * latent-vector attention cache and sigmoid-scored, group-limited expert routing (Tapalix and designs built from these parts) */

/* v = x[t] + add1[t] + add2[t] (each may be NULL), t = rows ? rows[r] : r. Without `rows` and with an addend x[t] <- v.
 * x_act (may be NULL, pitch ld_xact): v in the activation type; h_out (may be NULL, pitch ld_h): (v - mean) / sqrt(var + eps)
 * * gain + bias in the activation type. Sums, mean and variance are fp32. */
int p3_residual_layernorm(float* x, const float* add1, int64_t ld1, const float* add2, int64_t ld2, const int32_t* rows,
                          const float* gain, const float* bias, void* x_act, int64_t ld_xact, void* h_out, int64_t ld_h,
                          int act_f32, int64_t R, int W, float eps, cudaStream_t st);

/* After the fused input projection of a latent-attention mixer (proj fp32 [T, ld_proj]):
 *   q at q_off: n_heads x (dim plain | rot_dim turning). Plain parts -> q_plain (act) [T, ld_qp], head h at column h * dim;
 *     turning parts are rotated and go to q_lat (act) [T, ld_ql] at column h * (kv_rank + rot_dim) + kv_rank (the leading kv_rank
 *     columns of every head are filled later by the product with the key up-projection).
 *   latent at c_off: kv_rank numbers, RMS-normed with c_gain -> cache row columns [0, kv_rank); the rot_dim numbers behind them
 *     are rotated (not normed) -> cache row columns [kv_rank, kv_rank + rot_dim). cache: [page][64][kv_rank + rot_dim].
 *   rotation: the first rot_n numbers of a turning part, element i paired with i + rot_n / 2, angle = position * freq[i]
 *     (freq fp32 [rot_n / 2]), cos and sin times rot_mag; the rest passes unchanged.
 *   gated unit (n_ff > 0): hid (act) [T, ld_hid] columns [hid_off, hid_off + n_ff) = silu(proj[gate_off + i]) * proj[up_off + i]. */
typedef struct {
    const float* proj; int64_t ld_proj; int32_t q_off, c_off, gate_off, up_off;
    int32_t n_heads, dim, rot_dim, kv_rank, rot_n, n_ff;
    const float* c_gain; float eps; const float* freq; float rot_mag;
    void* q_plain; int64_t ld_qp; void* q_lat; int64_t ld_ql; void* hid; int64_t ld_hid; int32_t hid_off;
    void* cache; const int32_t* block_table; int32_t bt_stride;
    const int32_t* tok_slot; const int32_t* tok_pos; int32_t T;
    int32_t act_f32, cache_f32;
    /* Queries that come from a second product (through a normed low-rank vector) make this two calls. First, on the input
     * projection: n_heads = 0, the latent part as above, and the query's low-rank vector (q_rank numbers at cq_off) RMS-normed with
     * cq_gain -> cq_out (act) [T, ld_cq]. Then, on the product of cq_out with the query up-projection: q_src (fp32 [T, ld_qsrc],
     * heads x (dim | rot_dim)) replaces proj + q_off and cache = NULL skips the latent part (proj may then be NULL). A layer that
     * reads another layer's cache makes the first call with cache = NULL too. */
    int32_t pair_mode;             /* rotation pairs: 0 = number i with i + rot_n / 2, 1 = neighbours 2i and 2i + 1 (freq[i] each) */
    const float* q_src; int64_t ld_qsrc;
    int32_t cq_off, q_rank; const float* cq_gain; void* cq_out; int64_t ld_cq;
} p3_latent_post_args;
int p3_latent_post(const p3_latent_post_args* args, cudaStream_t st);

/* out (act) [R, F] = silu(g[r][c]) * u[r][c]; g and u fp32 with the common row pitch ld */
int p3_glu_silu(const float* g, const float* u, int64_t ld, void* out, int64_t ldo, int out_f32, int64_t R, int F, cudaStream_t st);

/* router with sigmoid scores: z = Wr x (fp32; or logits fp32 [T, ld_logits] when an earlier product already formed them with fp32
 * accumulation: x and Wr are then unused), s = sigmoid(z), choice = s + correction (correction fp32 [E] or NULL). The E
 * experts form n_groups equal groups of neighbours (n_groups <= 1: no groups); a group's score is the sum of its two largest
 * choice scores and only experts of the `keep` best groups can be chosen. ids [T, top] = the `top` largest choice scores among
 * those (ties: lower index); wts = s[ids] / (sum of them + 1e-20) * scale. */
int p3_router_sigmoid_groups(const void* x, int64_t ldx, int x_f32, const float* Wr, const float* correction, const float* logits,
                             int64_t ld_logits, int T, int W, int E, int top, int n_groups, int keep, float scale, int32_t* ids,
                             float* wts, cudaStream_t st);

/* logits <- cap * tanh(logits * scale / cap) (cap <= 0: logits * scale), n numbers in place */
int p3_logit_softcap(float* logits, int64_t n, float scale, float cap, cudaStream_t st);


/* ---- parts of decoders with a norm before AND after every sublayer, a token shift in front of the mixer, rotated windowed
 * attention (softmax with kept first tokens, or sigmoid weights over keys that double as values), a matrix-memory recurrence
 * and a mixture of experts with identity experts (Dugalix and designs built from these parts). Recurrent layers keep their
 * state per sequence slot; a step's sequences are described by `seqs`, int32 x 4 per sequence: {first batch row, number of
 * rows, sequence slot, position of the first row}; a sequence whose first row has position 0 starts from the zero state
 * whatever its slot holds. */

/* y' = y + y_bias (y_bias fp32 [W] or NULL); x += y' / sqrt(mean(y'^2) + eps) * gain_post (y NULL: x stays as it is). Then, with
 * gain_pre: h = x / sqrt(mean(x^2) + eps) * gain_pre -> h32 (fp32 [T, W], may be NULL) and h_act (activation type, may be NULL).
 * The gains are complete factors: a weight stored around zero enters as 1 + w, a residual multiplier is folded into gain_post. */
int p3_postnorm_prenorm(const float* y, int64_t ldy, const float* y_bias, const float* gain_post, float* x, const float* gain_pre,
                        float* h32, void* h_act, int act_f32, int64_t T, int W, float eps, cudaStream_t st);

/* out[t] = h[t] + (prev - h[t]) * shift, prev = h[t - 1] inside a sequence's rows, the slot's saved row for its first row
 * (zeros at position 0); afterwards state[slot] = h[last row of the sequence]. state fp32 [slots][W]; slot_seq int32 [slots] =
 * index of the slot's record in seqs for this step. */
int p3_token_shift(const float* h, const float* shift, float* state, const int32_t* seqs, const int32_t* slot_seq,
                   const int32_t* tok_slot, void* out, int out_f32, int64_t T, int W, cudaStream_t st);

/* After a fused q|k|v projection (proj fp32 [T, ld_proj]; bias fp32 indexed like proj's columns, or NULL): the leading rot_n
 * numbers of every query and key head turn by position * freq[i] (number i paired with i + rot_n / 2, freq fp32 [rot_n / 2]), the
 * rest passes; q -> q_out (act), k -> K pool, v -> V pool. v_off < 0: there is no value projection, the value of a token is its key
 * BEFORE the rotation (vdim == dim). */
typedef struct {
    const float* proj; int64_t ld_proj; int32_t q_off, k_off, v_off;
    const float* bias;
    int32_t n_heads, n_kv, dim, vdim, rot_n; const float* freq;
    void* q_out; int64_t ld_q;
    void* k_pool; void* v_pool; const int32_t* block_table; int32_t bt_stride;
    const int32_t* tok_slot; const int32_t* tok_pos; int32_t T;
    int32_t act_f32, cache_f32;
} p3_qkv_rope_post_args;
int p3_qkv_rope_post(const p3_qkv_rope_post_args* args, cudaStream_t st);

/* out (act) [R, F] = max(u, 0)^2 * (row_gate ? sigmoid(row_gate[r * ld_gate]) : 1), u fp32 with row pitch ld */
int p3_relu2(const float* u, int64_t ld, const float* row_gate, int64_t ld_gate, void* out, int64_t ldo, int out_f32, int64_t R, int F,
             cudaStream_t st);

/* Router over ready logits (fp32 [T, ld_logits], E outputs). mode bit 0: scores s = softmax over all E (else sigmoid); bit 1: a
 * group's score is its largest choice score (else the sum of its two largest); bit 2: wts = s[ids] as they are (else
 * s[ids] / (sum + 1e-20) * scale). choice = s + correction; groups and ties as in p3_router_sigmoid_groups. */
int p3_router_groups(const float* logits, int64_t ld_logits, const float* correction, int T, int E, int top, int n_groups, int keep,
                     float scale, int mode, int32_t* ids, float* wts, cudaStream_t st);

/* out[t] = sum_j wts[t][j] * (ids[t][j] < n_real ? y[where[t * top + j]] : h[t]) + (add ? add[t] : 0): experts with an index of
 * n_real or more are identity experts, whose output is the layer's input h (fp32 [T, W]); add fp32 [T, ld_add] or NULL */
int p3_moe_combine_identity(const float* y, int64_t ldy, const int32_t* where, const int32_t* ids, const float* wts, int top,
                            int n_real, const float* h, const float* add, int64_t ld_add, float* out, int64_t T, int W,
                            cudaStream_t st);

/* Matrix-memory recurrence (csrc/recurrent.cu). Per head: memory S [dim][vdim] (dim <= 512), normaliser n [dim], stabiliser m (0 at
 * the start).
 * From proj (fp32 [T, ld_proj]): q at q_off (times q_scale), k at k_off (heads x dim), v at v_off (heads x vdim), gate
 * pre-activations at i_off and f_off (one per head, biases i_bias / f_bias fp32 [heads]).
 *   a = cap tanh(pre_i / cap), b = logsigmoid(cap tanh(pre_f / cap)), m' = max(b + m, a),
 *   S' = e^(b + m - m') S + e^(a - m') k v^T, n' alike with k, y = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
 * token by token over the rows of every sequence of `seqs`. The numerators S'^T q go to out (fp32 [T, ld_out], head h at column
 * h * vdim), the denominators to den (fp32 [T, n_heads]); p3_headnorm_gate divides. The state of a slot is `state + slot *
 * p3_matrix_memory_state_floats(...)` floats, read at the start and written at the end of the step. rs_force (0: chosen by the
 * launch): 2 or 4 = row slices of S per warp with one column per lane, 8 = four slices with two columns; every choice gives the
 * same numbers. */
typedef struct {
    const float* proj; int64_t ld_proj; int32_t q_off, k_off, v_off, i_off, f_off;
    const float* i_bias; const float* f_bias;
    int32_t n_heads, dim, vdim; float q_scale, gate_cap;
    float* state; const int32_t* seqs; int32_t n_seqs;
    float* out; int64_t ld_out; float* den; int32_t rs_force;
} p3_matrix_memory_args;
int64_t p3_matrix_memory_state_floats(int n_heads, int dim, int vdim);
int p3_matrix_memory_scan(const p3_matrix_memory_args* args, cudaStream_t st);

/* out (act) [T, ldo] = v / sqrt(mean over the head's vdim numbers of v^2 + eps) * gain[c] * sigmoid(gate[t][c]) * scale with
 * v = y / den[t][head] (den fp32 [T, n_heads] or NULL: v = y), y fp32 [T, ldy] with n_heads x vdim columns, gate fp32 logits
 * [T, ld_gate] or NULL */
int p3_headnorm_gate(const float* y, int64_t ldy, const float* den, int n_heads, int vdim, const float* gain, const float* gate,
                     int64_t ld_gate, float scale, float eps, void* out, int64_t ldo, int out_f32, int64_t T, cudaStream_t st);


/* ---- parts of decoders with a hashed token-pair embedding, a gated linear-attention recurrence with a decay per key channel, and
 * attention whose distance bias is linear (Danalorn and designs built from these parts) */

/* x fp32 [T, W] = table[ids[t]] * scale + pair_table[r] (both bf16; pair_table NULL: no second term), r = (prev * mul_prev +
 * ids[t] * mul_cur) mod buckets with prev = the token before t in its sequence: the row above inside a step's run of rows, else the
 * slot's saved token prev_state[slot * state_stride]; r = buckets (the table's last row) for a sequence's first token (position
 * 0). Afterwards prev_state holds the last token of every sequence of the step. seqs / slot_seq / tok_slot as for p3_token_shift. */
int p3_embed_pair_rows_f32(const void* table, const void* pair_table, const int32_t* ids, const int32_t* seqs, const int32_t* slot_seq,
                           const int32_t* tok_slot, int32_t* prev_state, int64_t state_stride, float* x, int64_t T, int W, int vocab,
                           float scale, int64_t buckets, int64_t mul_prev, int64_t mul_cur, cudaStream_t st);

/* pen[h][i] = slope[h] * i, i < n: the table of a linear distance bias for p3_attn_window_* */
int p3_distance_linear_table(const float* slope, float* pen, int H, int n, cudaStream_t st);

/* Gated linear attention (csrc/recurrent.cu). Per head a state S [dim][vdim] (dim <= 512), zero at the start of a sequence:
 *   S' = diag(a) S + k v^T,  y = S'^T q * q_scale,  a[j] = exp(logsigmoid(z[j] + z_bias[j]) * inv_tau)   (sigmoid(z)^(1/tau))
 * token by token over the rows of every sequence of `seqs`. q at q_off, k at k_off (heads x dim) and v at v_off (heads x vdim) are
 * columns of proj (fp32 [T, ld_proj]); the decay logits z fp32 [n_rows, ld_z] (heads x dim, z_bias fp32 [heads * dim] or NULL) come
 * from a product of their own and are REPLACED by the decays (a first launch over all n_rows rows of the step; the sequences of
 * `seqs` lie inside them). With lr (fp32 [n_rows, ld_lr], `rank` <= 64 numbers per row: the low-rank vector of the decay projection,
 * e.g. columns of proj) and a2 (fp32 [heads * dim][rank]) that first launch forms the logits itself, z = a2 lr (+ z_bias, fp32 FMA
 * chain in ascending rank index), and z is only written. out fp32 [T, ld_out], head h at column h * vdim. The state of a slot is
 * `state + slot * p3_gla_state_floats(...)` floats, read at the start and written at the end of the step. rs_force as for the
 * matrix memory. */
typedef struct {
    const float* proj; int64_t ld_proj; int32_t q_off, k_off, v_off;
    float* z; int64_t ld_z; const float* z_bias; float inv_tau;
    int32_t n_heads, dim, vdim; float q_scale;
    float* state; const int32_t* seqs; int32_t n_seqs;
    float* out; int64_t ld_out; int32_t rs_force;
    int32_t n_rows;
    const float* lr; int64_t ld_lr; const float* a2; int32_t rank;
} p3_gla_args;
int64_t p3_gla_state_floats(int n_heads, int dim, int vdim);
int p3_gla_scan(const p3_gla_args* args, cudaStream_t st);

/* p3_headnorm_gate with two more choices: gain_shared != 0: gain is fp32 [vdim], the same for every head (else [n_heads * vdim]);
 * gate_silu != 0: the gate is g * sigmoid(g) instead of sigmoid(g) */
int p3_headnorm_gate_x(const float* y, int64_t ldy, const float* den, int n_heads, int vdim, const float* gain, int gain_shared,
                       const float* gate, int64_t ld_gate, int gate_silu, float scale, float eps, void* out, int64_t ldo, int out_f32,
                       int64_t T, cudaStream_t st);

#ifdef __cplusplus
}
#endif
#endif
