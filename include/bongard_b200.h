/* libbongard_b200 - C ABI of the B200 (sm_100a) kernels behind bongard's transformer
 * inference hot path.
 *
 * Conventions for every entry point
 *   - Pointers are DEVICE pointers borrowed from the caller (bf16 unless stated).  The caller
 *     keeps them alive until `stream` has passed the call.  The library allocates nothing.
 *   - Sizes and strides are in ELEMENTS.  `stream` is a cudaStream_t (NULL = default stream).
 *   - Return value: 0 on success, a negative BG_ERR_* code otherwise; bg_last_error_string()
 *     then describes the failure.  Nothing throws, exits or synchronises, except
 *     bg_read_status().
 *   - Kernels that wait on hardware barriers bound every wait; a wait that runs out is
 *     reported through bg_read_status(), never by a trap.
 *
 * "Replaces" names the reference code (path inside AgentBull/bongard, or `HF:` for
 * transformers/models/t5gemma2/modeling_t5gemma2.py, release 5.5.0) whose arithmetic the
 * entry point performs.
 */
#ifndef BONGARD_B200_H
#define BONGARD_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BG_OK 0
#define BG_ERR_SHAPE (-1)
#define BG_ERR_ALIGN (-2)
#define BG_ERR_ARCH (-3)
#define BG_ERR_LAUNCH (-4)
#define BG_ERR_WORKSPACE (-5)
#define BG_ERR_DRIVER (-6)
#define BG_ERR_TIMEOUT (-7)

int bg_version(void);
const char* bg_last_error_string(void);

/* 0 if the current device is sm_100 and the driver offers TMA descriptors.
 * Replaces the device gates of bongard/float8_training.py:31-34 and bongard/te_linear.py:110-111. */
int bg_device_check(void);

/* Synchronises `stream`, returns and clears the status word: 0, or the site code of the first
 * bounded wait that ran out (1xx BF16 GEMM, 2xx attention, 3xx FP8 GEMM). */
int bg_read_status(void* stream);

/* Self-test of the bounded device waits (no counterpart in the reference, which has no device
 * waits of its own).  Launches one CTA that waits, with a budget of `budget_us` microseconds
 * (1..100000), on a barrier that nothing completes; when the budget runs out the wait reports
 * site 901 exactly as the waits inside the GEMM and attention kernels report theirs, the kernel
 * sets *finished = 1 (device int32, may be NULL) and returns normally.  bg_read_status() then
 * returns 901 and the library keeps working.  Nothing traps or faults. */
int bg_selftest_bounded_wait(int64_t budget_us, int32_t* finished, void* stream);

/* Programmatic dependent launch for the latency path: with enable = 1 the kernels of the serving chain
 * (bg_gemm_bf16, bg_gemm_bf16_skinny, bg_varlen_attention, the norm / RoPE / embedding / head kernels) are
 * launched with programmatic stream serialization: a kernel may start while its predecessor in the stream is
 * still running, sets up its barriers and tensor memory, and waits (griddepcontrol.wait) before its first
 * access to global memory.  Default 0 (plain launches); process-wide.  No counterpart in the reference. */
void bg_set_programmatic_launch(int enable);

/* out[r, :] = rmsnorm(x[r, :]) * (1 + w), fp32 math, rounded once.
 * Replaces HF:61-69 T5Gemma2RMSNorm.forward / bongard/mps_inference.py:70-83 MPSRMSNorm. */
int bg_rmsnorm(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo, int64_t rows, int64_t h,
               float eps, void* stream);

/* resid += bf16(rmsnorm(y) * (1 + w_post)); normed = rmsnorm(resid) * (1 + w_next) (skipped when
 * w_next is NULL).  y, resid, normed are contiguous [rows, h].
 * Replaces the post-norm + residual + next pre-norm chain of HF:496-502 and HF:555-561. */
int bg_add_rmsnorm(const void* y, const void* w_post, void* resid, const void* w_next, void* normed,
                   int64_t rows, int64_t h, float eps, void* stream);

/* The same two calls over an fp32 residual stream (x / resid fp32, h a multiple of 256 up to 4096): the
 * residual is updated in fp32 and nothing is rounded on the way into it; the normed rows that feed the
 * GEMMs stay bf16.  This is the arithmetic of the reference run in float32 (HF:61-69 computes the norm in
 * fp32 for every dtype; HF:496-502 adds the residual in the model's dtype). */
int bg_rmsnorm_f32(const float* x, int64_t ldx, const void* w, void* out, int64_t ldo, int64_t rows, int64_t h,
                   float eps, void* stream);
int bg_add_rmsnorm_f32(const void* y, const void* w_post, float* resid, const void* w_next, void* normed,
                       int64_t rows, int64_t h, float eps, void* stream);
/* ... and with y in fp32 too: the unrounded projection from bg_gemm_bf16_f32out (h up to 3072). */
int bg_add_rmsnorm_f32y(const float* y, const void* w_post, float* resid, const void* w_next, void* normed,
                        int64_t rows, int64_t h, float eps, void* stream);

/* In-place per-head RMSNorm (1 + w gain) and rotate-half RoPE of q [tokens, q_heads, D] and
 * k [tokens, k_heads, D] (token strides ldq / ldk).  positions int32 [tokens]; inv_freq fp32 [D/2].
 * rotate = 0 normalises only; q or k may be NULL.
 * Replaces bongard/attention.py:172-180 project_qk (after the projections), the fused surface
 * bongard/flash_attention.py:76-125 metal_qk_norm_rope + bongard/qk_norm_rope.metal:4-33, and the
 * k_norm of bongard/model.py:135-139 project_state_kv (rotate = 0). */
int bg_qk_norm_rope(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads, const void* q_weight,
                    const void* k_weight, const int32_t* positions, const float* inv_freq, int64_t tokens,
                    int head_dim, float eps, int rotate, void* stream);

/* The same in-place norm + rotation with caller-supplied bf16 cos / sin tables [tokens, D]
 * (cat(freqs, freqs) layout, as the rotary module returns them).
 * Replaces the (q, k, q_norm, k_norm, position_embeddings) surface of
 * bongard/flash_attention.py:76-125 metal_qk_norm_rope and bongard/attention.py:172-180 project_qk. */
int bg_qk_norm_rope_table(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads,
                          const void* q_weight, const void* k_weight, const void* cos_table, const void* sin_table,
                          int64_t tokens, int head_dim, float eps, void* stream);

/* bg_qk_norm_rope with the angles read from a table made by bg_rope_table ([table_rows, head_dim / 2]
 * pairs (cos, sin) of position * inv_freq in fp32; positions are clamped to the table) instead of
 * four sincosf per lane and token: bit-identical results.  Same reference surface as bg_qk_norm_rope
 * (bongard/attention.py:172-180 project_qk with the rotary module's angles, HF:147-166). */
int bg_qk_norm_rope_cached(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads, const void* q_weight,
                           const void* k_weight, const int32_t* positions, const float* rope_table,
                           int64_t table_rows, int64_t tokens, int head_dim, float eps, void* stream);

/* out[r, :] = table[ids[r], :] * scale, or eoi_embedding where ids[r] == eoi_token.  ids int64.
 * Replaces HF:644-647 T5Gemma2TextScaledWordEmbedding.forward. */
int bg_embed(const int64_t* ids, const void* table, const void* eoi_embedding, void* out, int64_t rows, int64_t h,
             float scale, int64_t eoi_token, int64_t vocab, void* stream);
/* bg_embed writing the fp32 residual stream (out fp32, the product is not rounded).  Replaces HF:644-647. */
int bg_embed_f32(const int64_t* ids, const void* table, const void* eoi_embedding, float* out, int64_t rows, int64_t h,
                 float scale, int64_t eoi_token, int64_t vocab, void* stream);

/* out[m, n] = a[m, k] . w[n, k]^T on tcgen05 tensor cores, fp32 accumulate, bf16 out.
 * epilogue 0: plain.  epilogue 1 (GeGLU): w is the stacked [gate; up] weight of 2n rows and
 * out = gelu_tanh(a . gate^T) * (a . up^T).
 * Replaces F.linear in eval mode of bongard/te_linear.py:59-62 TELinear.forward (stacked weights,
 * 47-55), bongard/float8_training.py:17-21, and for epilogue 1 the gate_up -> GeGLU step of
 * bongard/te_linear.py:98-103 TEMLP.forward / HF:87-91 T5Gemma2MLP.forward. */
int bg_gemm_bf16(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo, int64_t m,
                 int64_t n, int64_t k, int epilogue, void* stream);

/* The plain GEMM with its fp32 accumulators written unrounded: out fp32, contiguous [m, n].  For the output and
 * down projections of a layer whose residual stream is fp32 (the post-norm then reads what the contraction
 * produced, not its bf16 rounding).  Replaces F.linear as bg_gemm_bf16 does. */
int bg_gemm_bf16_f32out(const void* a, int64_t lda, const void* w, int64_t ldw, float* out, int64_t m, int64_t n,
                        int64_t k, void* stream);

/* The q|k|v projection with QK-norm + RoPE fused into its epilogue: out[m, q_dim + 2 kv_dim] =
 * a[m, k] . w^T where w stacks the q, k and v projection weights; every query and key head gets the
 * fp32 RMSNorm over head_dim with gain (1 + q_gain / k_gain) and the rotate-half rotation by the
 * angles of its token's position before the single rounding to bf16 (the projection is rounded to
 * bf16 first, as the module chain does); value heads are stored as projected.  positions int32 [m];
 * rope_table fp32 [table_rows, head_dim / 2, 2] = (cos, sin), filled by bg_rope_table from the same
 * inv_freq bg_qk_norm_rope takes, covering every position in use.  head_dim 64, 128 or 256.
 * Replaces q_proj/k_proj/v_proj + q_norm/k_norm + apply_rotary_pos_emb of HF:248-262 and
 * bongard/attention.py:172-180 project_qk in one kernel (the reference fuses norm + RoPE only on
 * Metal, bongard/qk_norm_rope.metal:4-33, and keeps the projections separate). */
int bg_rope_table(float* table, int64_t rows, int head_dim, const float* inv_freq, void* stream);
int bg_gemm_bf16_qkv_rope(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo, int64_t m,
                          int64_t k, int q_dim, int kv_dim, int head_dim, const void* q_gain, const void* k_gain,
                          const int32_t* positions, const float* rope_table, int64_t table_rows, float eps,
                          void* stream);

/* bg_gemm_bf16 for 1..256 rows (k % 64 == 0, n % 128 == 0; GeGLU: n % 64 == 0), the single-request
 * serving case of bongard/model.py:448-458 (one question group decoded against a cached state), where
 * the contraction is bound by streaming the weights from HBM: every weight byte is fetched once, K is
 * split over the CTAs of a thread-block cluster sized so that one wave fills the GPU, and the partial
 * tiles are summed in rank order through distributed shared memory (deterministic; the fp32 summation
 * order differs from bg_gemm_bf16, so results may differ from it in the last bf16 bit).
 * bg_gemm_bf16_skinny_supported returns 1 for shapes it takes, else 0; other shapes are BG_ERR_SHAPE. */
int bg_gemm_bf16_skinny_supported(int64_t m, int64_t n, int64_t k, int epilogue);
int bg_gemm_bf16_skinny(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo, int64_t m,
                        int64_t n, int64_t k, int epilogue, void* stream);

/* Split-K form of bg_gemm_bf16 (plain epilogue) for problems whose 256 x 256 output tiles fill less than
 * half of the GPU: a few hundred rows against a narrow weight with a long contraction (the down projection
 * of a short request on the single-request path, bongard/inference.py:283-340).  Each (tile, K slice) is a
 * work item of the CTA-pair kernel; slices write fp32 partial tiles into the caller's workspace and a second
 * kernel sums them in slice order and rounds once to bf16.
 *   bg_gemm_bf16_splitk_choice: the number of slices worth using for a shape (1 = use bg_gemm_bf16).
 *   bg_gemm_bf16_splitk_workspace_bytes: split * m * n * 4. */
int bg_gemm_bf16_splitk_choice(int64_t m, int64_t n, int64_t k);
int64_t bg_gemm_bf16_splitk_workspace_bytes(int64_t m, int64_t n, int split);
int bg_gemm_bf16_splitk(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo, int64_t m,
                        int64_t n, int64_t k, int split, void* workspace, int64_t workspace_bytes, void* stream);

/* Helpers for the backward of the bf16 linears (the reference trains through them with autograd:
 * bongard/te_linear.py:59-77 TELinear.forward, 98-103 TEMLP.forward, bongard/fused_mlp.py:62-79).
 * With y = x W^T: dx = dy W and dW = dy^T x contract over dimensions that are not contiguous in dy, W
 * and x, while bg_gemm_bf16 wants both operands contiguous along the contraction, so the operands are
 * transposed first: dx = bg_gemm_bf16(dy, W^T), dW = bg_gemm_bf16(dy^T, x^T).
 *   bg_transpose_bf16: dst[c, r] = src[r, c] (row strides lds, ldd in elements).
 *   bg_geglu_backward: for gu = [g | u] [rows, 2 inter] and dh [rows, inter]:
 *       dgu = [dh * u * gelu_tanh'(g) | dh * gelu_tanh(g)]. */
int bg_transpose_bf16(const void* src, int64_t lds, void* dst, int64_t ldd, int64_t rows, int64_t cols, void* stream);
/* out[m, n] = sum_k at[k, m] * wt[k, n] (bf16 in and out, fp32 accumulate): both operands carry the contraction
 * as their ROW index, so the weight gradient dW = dy^T x is taken straight from dy [tokens, out features] and
 * x [tokens, in features] - the tensor core reads MN-major tiles, nothing is transposed.  m, n and the
 * leading dimensions must be multiples of 8 and the pointers 16-byte aligned.  split >= 2 cuts the contraction
 * into that many slices (bg_gemm_bf16_splitk_choice(m, n, k) says when that pays: a weight gradient has few output
 * tiles and a long contraction) and needs a workspace of bg_gemm_bf16_splitk_workspace_bytes(m, n, split);
 * split <= 1 ignores the workspace. */
int bg_gemm_bf16_tn(const void* at, int64_t ldat, const void* wt, int64_t ldwt, void* out, int64_t ldo, int64_t m,
                    int64_t n, int64_t k, int split, void* workspace, int64_t workspace_bytes, void* stream);
int bg_geglu_backward(const void* gu, const void* dh, void* dgu, int64_t rows, int64_t inter, void* stream);
/* h[rows, inter] = gelu_tanh(g) * u for gu = [g | u] [rows, 2 inter]: the activation as its own pass, for a
 * training forward that keeps gu for bg_geglu_backward instead of recomputing it (HF T5Gemma2MLP.forward,
 * modeling_t5gemma2.py:87-91, forms it from the bf16 projections the same way). */
int bg_geglu_forward(const void* gu, void* h, int64_t rows, int64_t inter, void* stream);

/* Backward of the norms the reference trains through with autograd (transformers T5Gemma2RMSNorm,
 * modeling_t5gemma2.py:55-69; QK-norm + RoPE: bongard/attention.py:172-180).  fp32 math, bf16 in and out,
 * gain gradients as fp32 vectors summed in a fixed order (no atomics).  The workspace holds one partial
 * gain-gradient row per block (per warp for the QK form); its size comes from the companion function.
 *   bg_rmsnorm_backward: y = x r (1 + w), r = rsqrt(mean(x^2) + eps):
 *       dx = r g - x r^3 mean(g x) with g = dy (1 + w);  dw[h] = sum_rows dy x r.
 *   bg_qk_norm_rope_backward: xq [tokens, q_heads, D] / xk [tokens, k_heads, D] are the inputs the forward
 *       normalised (it runs in place: keep a copy), dyq / dyk the gradients of its outputs; the rotation is
 *       undone first (da[j] = dy[j] cos[j] - sign(j) (dy sin)[partner(j)]), then the per-head norm backward.
 *       Angles as in the forward: positions + inv_freq, or bf16 cos / sin tables [tokens, D]; rotate = 0 for
 *       the state keys.  k_heads = 0 (xk NULL) handles q alone; dk_weight may then be NULL. */
int64_t bg_rmsnorm_backward_workspace_bytes(int64_t rows, int64_t h);
int bg_rmsnorm_backward(const void* x, int64_t ldx, const void* w, const void* dy, int64_t lddy, void* dx,
                        int64_t lddx, float* dw, void* workspace, int64_t workspace_bytes, int64_t rows, int64_t h,
                        float eps, void* stream);
int64_t bg_qk_norm_rope_backward_workspace_bytes(int64_t tokens, int head_dim);
int bg_qk_norm_rope_backward(const void* xq, int64_t ldxq, const void* dyq, int64_t lddyq, void* dxq, int64_t lddxq,
                             int q_heads, const void* xk, int64_t ldxk, const void* dyk, int64_t lddyk, void* dxk,
                             int64_t lddxk, int k_heads, const void* q_weight, const void* k_weight,
                             const int32_t* positions, const float* inv_freq, const void* cos_table,
                             const void* sin_table, float* dq_weight, float* dk_weight, void* workspace,
                             int64_t workspace_bytes, int64_t tokens, int head_dim, float eps, int rotate,
                             void* stream);

/* E4M3 quantisation with dynamic per-block scales: scale = 448 / max(amax, 1e-12), values clamped
 * to +-448 and rounded to nearest; the INVERSE scales are stored as fp32.
 *   rows : 1 x 128 blocks of x [m, k] -> q (uint8 [m, k], row stride ldq bytes), inv_scale_t [k/128, m].
 *   tiles: 128 x 128 blocks of w [n, k] -> q, inv_scale [ceil(n/128), k/128].
 * Replaces the per-call dynamic scaling of the reference's FP8 linears
 * (bongard/float8_training.py:35-44; torchao Float8Linear casts) at 128-element granularity. */
int bg_quantize_e4m3_rows(const void* x, int64_t ldx, void* q, int64_t ldq, float* inv_scale_t, int64_t m, int64_t k,
                          void* stream);
int bg_quantize_e4m3_tiles(const void* w, int64_t ldw, void* q, int64_t ldq, float* inv_scale, int64_t n, int64_t k,
                           void* stream);

/* out[m, n] = sum over 128-deep K blocks of a_inv_t[kb, m] * w_inv[n/128, kb] * (aq . wq^T), E4M3
 * operands on tcgen05 (kind::f8f6f4), fp32 accumulate, bf16 out.  Epilogues as bg_gemm_bf16.
 * Replaces the scaled GEMM behind bongard/float8_training.py:12-24 TrainingLinear.forward
 * (torch._scaled_mm) and the `fp8` recipe of bongard/te_linear.py:32-39 / bongard/fused_mlp.py:21-79. */
int bg_gemm_fp8_block128(const void* aq, int64_t lda, const float* a_inv_t, const void* wq, int64_t ldw,
                         const float* w_inv, void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue,
                         void* stream);

/* bf16 activation in, FP8 contraction: x is quantised (1 x 128 blocks) into `workspace`, then
 * multiplied with pre-quantised weights.  bg_linear_fp8_workspace_bytes(m, k) gives the scratch
 * size; the workspace must be 256-byte aligned and is owned by the caller.
 * Replaces bongard/float8_training.py:17-22 / bongard/te_linear.py:59-77 forward in FP8 mode. */
int64_t bg_linear_fp8_workspace_bytes(int64_t m, int64_t k);
int bg_linear_fp8(const void* x, int64_t ldx, const void* wq, int64_t ldw, const float* w_inv, void* out,
                  int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* workspace,
                  int64_t workspace_bytes, void* stream);

/* MXFP8: E4M3 values with one power-of-two (UE8M0) scale per 32 consecutive K elements, the block
 * format the tensor cores scale themselves (tcgen05.mma kind::mxf8f6f4.block_scale).
 *   bg_quantize_mxfp8: x [rows, k] bf16 -> q uint8 [rows, k] (row stride ldq bytes) and scales:
 *       e = ceil(log2(amax_32 / 448)) clamped to [-127, 127], q = e4m3(x * 2^-e), scale byte = e + 127,
 *       stored in 512-byte atoms, one per 128 rows x 128 K elements, atom (r / 128, k / 128) at
 *       (r / 128 * (k_total / 128) + k / 128) * 512, byte (r % 32) * 16 + (r % 128) / 32 * 4 + (k / 32) % 4
 *       (the layout tcgen05.cp moves into tensor memory unchanged); bg_mxfp8_scale_bytes gives the size,
 *       which the caller zero-fills once (rows beyond `rows` in the last atom are never written).
 *   bg_gemm_mxfp8: out[m, n] = sum_k (2^ea Aq)(2^ew Wq)^T, fp32 accumulate in tensor memory, bf16 out,
 *       epilogues as bg_gemm_bf16; k and n multiples of 128.
 * Replaces the `mxfp8` recipe of bongard/te_linear.py:32-39 and bongard/fused_mlp.py:21-34 (Transformer
 * Engine MXFP8BlockScaling) for the forward pass. */
int64_t bg_mxfp8_scale_bytes(int64_t rows, int64_t k);
int bg_quantize_mxfp8(const void* x, int64_t ldx, void* q, int64_t ldq, void* scales, int64_t rows, int64_t k,
                      void* stream);
int bg_gemm_mxfp8(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw, const void* w_scales,
                  void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* stream);
/* bg_rmsnorm / bg_add_rmsnorm writing the normalised rows as MXFP8 (contiguous uint8 [rows, h] + scale atoms of
 * a [rows, h] matrix, zero-filled by the caller) for the GEMM that consumes them; values equal
 * bg_quantize_mxfp8 of the bf16 result.  h a multiple of 128. */
int bg_rmsnorm_mxfp8(const void* x, int64_t ldx, const void* w, void* out_q, void* out_scales, int64_t rows, int64_t h,
                     float eps, void* stream);
int bg_add_rmsnorm_mxfp8(const void* y, const void* w_post, void* resid, const void* w_next, void* normed_q,
                         void* normed_scales, int64_t rows, int64_t h, float eps, void* stream);
/* bg_gemm_mxfp8 with the GeGLU epilogue, writing its result as MXFP8 (out_q uint8 [m, n], row stride ldq
 * bytes, out_scales in the atom layout of a [m, n] matrix, zero-filled by the caller) instead of bf16:
 * the values equal bg_quantize_mxfp8 of the bf16 result, without the two extra passes over it. */
int bg_gemm_mxfp8_geglu_q(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw,
                          const void* w_scales, void* out_q, int64_t ldq, void* out_scales, int64_t m, int64_t n,
                          int64_t k, void* stream);

/* bg_linear_fp8 for callers that cannot supply scratch memory.  (No counterpart in the reference.)
 * The quantised activations go to a fixed buffer inside the library instead of a caller-owned
 * workspace, so the call allocates nothing; in exchange the activation is limited to
 * bg_linear_fp8_static_max_bytes() of scratch (9 MiB: e.g. 3 574 rows of 2 560, at 2 560 bytes of E4M3 plus 80 bytes of block scales a row),
 * larger ones are refused with BG_ERR_WORKSPACE.  Every GPU that loads the library holds the buffer
 * until exit.  The first call on each device looks up the buffer's device address: make it before
 * any stream capture.  All calls on a device share the buffer, so calls that may overlap on the GPU
 * must be ordered by the caller.  Same arguments and results as bg_linear_fp8 otherwise. */
int64_t bg_linear_fp8_static_max_bytes(void);
int bg_linear_fp8_static(const void* x, int64_t ldx, const void* wq, int64_t ldw, const float* w_inv, void* out,
                         int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* stream);

/* Packed variable-length attention, one softmax over [prefix keys | own keys].
 *   q [tq, q_heads, D] (token stride ldq, head stride hsq); k, v [tk, kv_heads, D] (strides ldkv,
 *   hskv); ck, cv [ts, kv_heads, D] (strides ldc, hsc) or NULL - any token/head strides that are
 *   multiples of 8 elements, so both [T, H, D] and [H, T, D] storage work without a copy;
 *   out [tq, q_heads * D] contiguous;
 *   lse fp32 [q_heads, tq] (natural log) or NULL.
 *   tiles int32 [n_tiles, 8] = {q_start, q_count, own_lo, own_hi, lo_max, hi_min, prefix_start,
 *   prefix_len}: q_count <= bg_attention_tile_rows(head_dim) / (q_heads / kv_heads) consecutive
 *   query tokens; [own_lo, own_hi)
 *   covers every row's own-key range, [lo_max, hi_min) is the part visible to all rows; the
 *   prefix keys are visible to every row.  row_lo / row_hi int32 [tq]: own-key range per token.
 * Replaces bongard/flash_varlen.py:129-139 attention, 13-22 _forward (op bongard::flash_packed_forward),
 * 61-77 _prefix (op bongard::flash_prefix_forward, without materialising the gathered keys), the
 * windowed layers bongard/packing.py:154-175 packed_attention serves, and the two-partition
 * serving path bongard/attention.py:122-169. */
int bg_attention_tile_rows(int head_dim);

/* The persistent attention kernel's dealing rule: the work item (tile record * kv_heads + KV head) that
 * CTA `cta` of `grid` CTAs takes in its `round`-th turn (a CTA stops at the first index that is not
 * below tile records x kv_heads); -1 for arguments out of range.  Host code only (no device work);
 * no counterpart in the reference, whose kernels are scheduled by their libraries. */
int bg_attention_item_index(int grid, int cta, int round);
int bg_varlen_attention(const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v, int64_t ldkv,
                        int64_t hskv, const void* ck, const void* cv, int64_t ldc, int64_t hsc, void* out,
                        float* lse, const int32_t* tiles,
                        int32_t n_tiles, const int32_t* row_lo, const int32_t* row_hi, int64_t tq, int64_t tk,
                        int64_t ts, int q_heads, int kv_heads, int head_dim, float scale, void* stream);

/* The same attention for head_dim 256 on CTA pairs: a tile record covers bg_attention_pair_tile_rows() = 256
 * query rows (0 for head sizes without a pair kernel), two CTAs of a cluster take 128 rows each and share the
 * key stream - each loads half of every K tile and half of every V tile's columns.  Arguments, results and
 * errors as bg_varlen_attention.  Replaces the same reference code. */
int bg_attention_pair_tile_rows(int head_dim);
int bg_varlen_attention_pair(const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v, int64_t ldkv,
                        int64_t hskv, const void* ck, const void* cv, int64_t ldc, int64_t hsc, void* out,
                        float* lse, const int32_t* tiles,
                        int32_t n_tiles, const int32_t* row_lo, const int32_t* row_hi, int64_t tq, int64_t tk,
                        int64_t ts, int q_heads, int kv_heads, int head_dim, float scale, void* stream);

/* Backward of bg_varlen_attention: dq [tq, q_heads, D], dk, dv [tk, kv_heads, D] and, with a state
 * prefix, dck, dcv [ts, kv_heads, D] (all contiguous bf16, every row written once, no atomics).
 *   out [tq, q_heads * D] and lse fp32 [q_heads, tq] are the forward's results; dout [tq, q_heads, D]
 *   with token stride ldd and head stride hsd; delta fp32 [q_heads, tq] is scratch (rowsum(dout * out)).
 *   q_tiles / row_lo / row_hi as in the forward; kv_tiles int32 [n_kv_tiles, 8] = {k_start, k_count,
 *   q_lo, q_hi, is_state, 0, 0, 0}: up to 128 consecutive keys (of k/v, or of ck/cv when is_state) and
 *   the query tokens [q_lo, q_hi) that may see them; state tiles are seen by all of those tokens, own
 *   tiles by a token t iff row_lo[t] <= key < row_hi[t].  Every key of k/v needs exactly one tile.
 * Three passes of one kernel (dQ per query tile; dK and dV per key tile) recompute the probabilities
 * from lse on the tensor cores.
 * Replaces bongard/flash_varlen.py:30-39 _backward (op bongard::flash_packed_backward) and 85-105
 * _prefix_backward (op bongard::flash_prefix_backward, without the gathered keys and the index_add_
 * scatter of their gradients). */
int bg_varlen_attention_backward(const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v, int64_t ldkv,
                                 int64_t hskv, const void* ck, const void* cv, int64_t ldc, int64_t hsc,
                                 const void* out, const void* dout, int64_t ldd, int64_t hsd, const float* lse,
                                 float* delta, void* dq, void* dk, void* dv, void* dck, void* dcv,
                                 const int32_t* q_tiles, int32_t n_q_tiles, const int32_t* kv_tiles,
                                 int32_t n_kv_tiles, const int32_t* row_lo, const int32_t* row_hi, int64_t tq,
                                 int64_t tk, int64_t ts, int q_heads, int kv_heads, int head_dim, float scale,
                                 void* stream);

/* logits[c] = w . h + (C h) . (G g) / sqrt(rank) with h = hidden[cand_rows[c]], g = hidden[dec_rows[c]].
 * Replaces bongard/model.py:85-95 JudgmentHead.forward as called by 520-529 score_readouts. */
int bg_judgment_head(const void* hidden, int64_t ldh, const int32_t* cand_rows, const int32_t* dec_rows,
                     const void* w, const void* cmat, const void* gmat, float* logits, int64_t candidates,
                     int64_t h, int rank, void* stream);

/* Per-question float64 temperature softmax: question i owns logits [offsets[i], offsets[i+1]).
 * Replaces bongard/inference.py:54-73 probabilities. */
int bg_candidate_softmax(const float* logits, const int32_t* offsets, double* probs, int64_t questions,
                         double temperature, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BONGARD_B200_H */
