/*
 * superl8_b200 -- C ABI of the B200 (sm_100a) INT8 attention engine.
 *
 * The library replaces, for one hot path only, the compiled operators that the
 * reference binds into its `superl8._C` module (reference csrc/fni8_api.cpp:213-291):
 * the per-row symmetric int8 quantiser, the int8-QK FlashAttention-2 forward and
 * the split-KV int8-K / fp16-V decode.  Every entry point takes plain device
 * pointers, sizes and a CUDA stream (passed as void*); none of them allocates
 * device memory unless its comment says so: callers own inputs, outputs and the
 * workspace.  All launches are asynchronous on the given stream.  Return value:
 * SL8_OK or a negative SL8_ERR_* code; sl8_status_string() names it.
 *
 * Tensor layout everywhere: [B, H, S, D] contiguous, head dim innermost, exactly
 * the reference layout (reference csrc/include/attn_int8_fwd.cuh:47-58).
 */
#ifndef SUPERL8_B200_H_
#define SUPERL8_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SL8_ABI_VERSION 1

/* ---- status codes ------------------------------------------------------- */
#define SL8_OK 0
#define SL8_ERR_BAD_HEAD_DIM (-1)   /* reference: "head dim must be 32/64/72/80/128/256" */
#define SL8_ERR_BAD_DTYPE (-2)      /* reference: "v must be float16 or bfloat16" */
#define SL8_ERR_MISALIGNED (-3)     /* pointer not 16-byte aligned (TMA / vector loads) */
#define SL8_ERR_BAD_NUM_SPLITS (-4) /* reference: "num_splits must be 1..256" */
#define SL8_ERR_WORKSPACE (-5)      /* workspace null or too small */
#define SL8_ERR_BAD_SHAPE (-6)      /* negative size, Hq % Hkv != 0, ... */
#define SL8_ERR_NULL (-7)           /* required pointer is null */
#define SL8_ERR_CUDA (-8)           /* a CUDA runtime / driver call failed */
#define SL8_ERR_DEVICE_TIMEOUT (-9) /* a bounded device-side wait expired */
#define SL8_ERR_UNSUPPORTED (-10)   /* valid request this backend cannot serve */
#define SL8_ERR_TOO_LARGE (-11)     /* request exceeds a fixed built-in capacity */

/* element types of floating-point tensors */
#define SL8_F16 0
#define SL8_BF16 1
#define SL8_F32 2

/* prefill backends (sl8_fwd_params.backend) */
#define SL8_BACKEND_AUTO 0
#define SL8_BACKEND_TCGEN05 1 /* TMA + tcgen05 (D = 64, 128, 256): 128 x 64 tiles, two blocks per SM */
#define SL8_BACKEND_MMA 2     /* warp-level mma.sync path (every supported D) */
#define SL8_BACKEND_TCGEN05_2Q 3 /* TMA + tcgen05, one block per SM with two 128-row query tiles and 128-key tiles
                                    (D = 128, dense layout, no window; other calls fall back to BACKEND_TCGEN05).
                                    Measured equal to BACKEND_TCGEN05 for 16-bit Q/K and 10 % slower for int8 Q/K on
                                    B16 Hq64 S8192, so BACKEND_AUTO does not pick it. */

int sl8_abi_version(void);
const char* sl8_status_string(int status);

/* ---- quantiser ---------------------------------------------------------- */

/*
 * Per-row symmetric int8 quantisation of x[M, K] (row-major, contiguous).
 * scale[r] = amax(|x[r,:]|) * float(1/127), 1.0 for an all-zero row;
 * q[r,c] = clamp(rint(x[r,c] / scale[r]), -127, 127)  (never -128).
 * Replaces `quantize_i8_rowwise` (reference csrc/kernel/quant_rowwise.cu:84-121,
 * kernel csrc/include/quant_rowwise.cuh:42-92; binding csrc/fni8_api.cpp:286-291).
 * M == 0 or K == 0 is a no-op (reference quant_rowwise.cu:96).
 */
int sl8_quantize_i8_rowwise(const void* x, int x_dtype, int64_t M, int64_t K,
                            int8_t* q, float* scale, void* stream);

/*
 * Q prologue: quantise q[rows, D] like sl8_quantize_i8_rowwise and store the
 * FOLDED scale  scale * fold  (fold = float(softmax_scale * log2 e)), which is
 * what the attention kernels consume (reference superl8/quant/core.py:193-195).
 * If outlier_flag != NULL the kernel also evaluates the reference's accuracy
 * gate in the same pass (reference superl8/quant/core.py:113-145): a row is
 * outlier-dominated when  max|q| / (median|q| + 1e-10) > ratio_threshold
 * (median = lower middle element, as torch.median); *outlier_flag is OR-ed
 * with 1 when any row is.  The caller zeroes the flag beforehand.
 * plain_scale (nullable) receives the unfolded scale.
 */
int sl8_quant_q_prologue(const void* q, int dtype, int64_t rows, int64_t D, float fold,
                         float ratio_threshold, int8_t* q_i8, float* q_scale_folded,
                         float* plain_scale, int32_t* outlier_flag, void* stream);

/*
 * The accuracy gate alone (reference superl8/quant/core.py:113-145, which superl8/ops.py:118-130 runs
 * before it quantises): *outlier_flag |= 1 when some row of q [rows, D] has
 * max|q| / (median|q| + 1e-10) > ratio_threshold.  Reads q once, writes nothing else.
 */
int sl8_q_outlier_gate(const void* q, int dtype, int64_t rows, int64_t D, float ratio_threshold,
                       int32_t* outlier_flag, void* stream);

/*
 * K prologue, step 1: per-(batch, kv-head) fp32 mean over the keys,
 * k[BH, N, D] -> mean[BH, D]  (reference superl8/quant/core.py:29-44, 81-85).
 * seqlens (nullable, int32[B], with heads_per_batch = Hkv) restricts sequence b
 * to its first seqlens[b] keys.  The sum runs in a fixed order (bitwise
 * repeatable).  workspace: sl8_k_mean_workspace() bytes.
 */
size_t sl8_k_mean_workspace(int64_t BH, int64_t N, int64_t D);
int sl8_k_mean(const void* k, int dtype, int64_t BH, int64_t N, int64_t D,
               const int32_t* seqlens, int32_t heads_per_batch, float* mean,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * K prologue, step 2: smooth and quantise in one pass:
 * k_s = T(float(k) - mean[bh, :]) rounded to k's own dtype, then the row
 * quantiser (reference superl8/quant/core.py:86-95 then :47-62).  k_smoothed
 * (nullable) receives k_s.
 */
int sl8_smooth_quant_k(const void* k, int dtype, int64_t BH, int64_t N, int64_t D,
                       const float* mean, int8_t* k_i8, float* k_scale, void* k_smoothed,
                       void* stream);

/*
 * The rotate=True prologue (reference superl8/quant/core.py:186-194 with
 * superl8/quant/rotation.py:28-51): every row of x [rows, D] is, in one pass and in registers,
 *   [mean != NULL]  smoothed:  x - mean[row / rows_per_head, :], rounded to x's dtype;
 *   rotated:        y = x @ (H_D / sqrt(D)), H_D the Sylvester-Hadamard matrix, computed in fp32 as a
 *                   Walsh-Hadamard butterfly and rounded to x's dtype (the reference's matmul adds in
 *                   another order: results agree to fp32 rounding before that cast);
 *   [rotated != NULL]  stored as x's dtype;
 *   [q != NULL]        quantised per row: codes to q, scale * fold to scale (fold = softmax_scale *
 *                      log2(e) for Q, 1 for K).
 * Q: mean = NULL.  K: mean = the slab means of sl8_k_mean, rows_per_head = N.  The rotation alone
 * (`rotate_last`): q = NULL.  fp16 / bf16, D a power of two in [32, 1024], 16-byte aligned rows.
 */
int sl8_hadamard_quant_rows(const void* x, int dtype, int64_t rows, int64_t D, const float* mean,
                            int64_t rows_per_head, float fold, int8_t* q, float* scale, void* rotated,
                            void* stream);

/*
 * K prologue in ONE launch: steps 1 and 2 together (reference superl8/quant/core.py:29-44, 70-95, then
 * :47-62).  A thread-block cluster owns each (batch, kv-head) slab: it forms the fp32 mean (the same
 * chunked, fixed-order sum as sl8_k_mean: the results are bitwise equal), shares it through distributed
 * shared memory, and quantises the slab on a second walk that finds the rows in L2, so K crosses HBM once.
 * mean [BH, D] receives the mean; k_smoothed is nullable.  sl8_k_prologue_fused_ok() says whether the
 * shape is served (fp16 / bf16, D in {64, 128, 256}, BH <= 65535, N <= about 90 000 at D = 128); otherwise
 * SL8_ERR_UNSUPPORTED: use the two steps.
 */
int sl8_k_prologue_fused_ok(int dtype, int64_t BH, int64_t N, int64_t D);
int sl8_k_prologue(const void* k, int dtype, int64_t BH, int64_t N, int64_t D,
                   const int32_t* seqlens, int32_t heads_per_batch, float* mean,
                   int8_t* k_i8, float* k_scale, void* k_smoothed, void* stream);

/* ---- prefill: int8-QK FlashAttention-2 forward -------------------------- */

typedef struct sl8_fwd_params {
  const int8_t* q;        /* [B, Hq, M, D] int8 */
  const float* q_scale;   /* [B, Hq, M] folded: scale * softmax_scale * log2(e) */
  const int8_t* k;        /* [B, Hkv, N, D] int8 (smoothed) */
  const float* k_scale;   /* [B, Hkv, N] */
  const void* v;          /* [B, Hkv, N, D] fp16 or bf16 */
  void* out;              /* [B, Hq, M, D], dtype of v */
  float* lse;             /* [B, Hq, M] natural-log LSE, or NULL */
  const int32_t* seqlens_q; /* int32[B] or NULL: valid query rows per sequence  */
  const int32_t* seqlens_k; /* int32[B] or NULL: valid keys per sequence        */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t v_dtype;        /* SL8_F16 or SL8_BF16 */
  int32_t causal;         /* bottom-right aligned: query i sees keys <= i + N - M */
  int32_t window_left;    /* < 0: none; else keys in (pos - window_left, pos] */
  int32_t backend;        /* SL8_BACKEND_* */
  /* Device-side dispatch (nullable; tcgen05 backend only; no counterpart in the reference, which reads
   * its gate back to the host, superl8/quant/core.py:145): when gate_flag is non-NULL the kernel
   * runs only if (*gate_flag != 0) == (gate_want != 0) and otherwise exits at once, leaving `out`
   * untouched.  Launching this op with gate_want = 0 and sl8_attn_fp16_fwd with gate_want = 1 on
   * the same `out`, behind the pass that raises the flag (sl8_quant_q_prologue), applies the
   * accuracy gate without a host read-back, so the whole call can be captured in a CUDA graph. */
  const int32_t* gate_flag;
  int32_t gate_want;
} sl8_fwd_params;

/*
 * out = softmax2(int32(q k^T) * q_scale[m] * k_scale[n]) v, rows with no valid
 * key give 0 (LSE -inf).  Replaces `attn_int8_fwd` / `attn_int8_fwd_train`
 * (reference csrc/kernel/attn_int8_fwd.cu:101-200, kernels
 * csrc/include/attn_int8_fwd.cuh:47-209 and :228-373; bindings
 * csrc/fni8_api.cpp:225-233).  D in {32, 64, 72, 80, 128, 256}.
 * workspace: sl8_attn_int8_fwd_workspace() bytes; its first int32 is a device
 * status word the kernel sets non-zero when a bounded wait expires (read it
 * with sl8_read_device_status after synchronising).
 * With seqlens_*, sequence b is computed as if the reference had been called on
 * its [:, :, :len] slices; padded output rows are written as zeros.  One difference
 * from a slice: K and V rows between seqlens_k[b] and N are still LOADED with the tile
 * that holds the last valid key (their P is exactly 0), so they must hold finite
 * numbers -- 0 * NaN in the P.V contraction would poison the row.  Zero-initialised or
 * previously used cache memory is fine; memory that may hold NaN / Inf bit patterns
 * (a fresh allocation that was never written) is not.  The same holds for the keys
 * past context_lens in the decode entries.
 */
size_t sl8_attn_int8_fwd_workspace(const sl8_fwd_params* p);
int sl8_attn_int8_fwd(const sl8_fwd_params* p, void* workspace, size_t workspace_bytes,
                      void* stream);

/*
 * Raw int32 logits of one (batch, head): s[M, N] = q[M, D] . k[N, D]^T computed
 * by the same tcgen05 kind::i8 tile path as the forward kernel.  Exists so the
 * integer contraction can be pinned bit-exactly; the reference has the same
 * quantity only inside its kernel (csrc/include/attn_int8_fwd.cuh:129-138).
 */
int sl8_qk_logits_i32(const int8_t* q, const int8_t* k, int32_t M, int32_t N, int32_t D,
                      int32_t* s, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Full-precision sibling used when the accuracy gate demotes a call
 * (reference superl8/ops.py:120-130 -> csrc/kernel/attn_fp16_fwd.cu:105-207):
 * q, k, v one dtype (fp16 or bf16), logits = (q . k) * softmax_scale.
 */
typedef struct sl8_fp16_fwd_params {
  const void* q; const void* k; const void* v; void* out; float* lse;
  const int32_t* seqlens_q; const int32_t* seqlens_k;
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype; int32_t causal; int32_t window_left;
  float softmax_scale;
  int32_t backend;        /* SL8_BACKEND_* (tcgen05 for D = 64/128/256, else mma.sync) */
  /* optional additive bias [B|1, H|1, M, N] in natural-log units, element type = dtype, indexed in
   * place through element strides (0 on broadcast axes); served by both kernels -- on the
   * tensor-memory kernel (D = 64/128/256) every thread adds its own query row's values to the
   * finished logits, eight contiguous 16-byte aligned values per load, any other layout element
   * by element (reference csrc/kernel/attn_fp16_fwd.cu:146-168, csrc/include/attn_fp16_fwd.cuh:176-178) */
  const void* mask;
  int64_t mask_stride_b, mask_stride_h, mask_stride_m, mask_stride_n;
  const int32_t* gate_flag;   /* device-side dispatch, as in sl8_fwd_params (nullable; tcgen05 backend, no mask) */
  int32_t gate_want;
} sl8_fp16_fwd_params;
size_t sl8_attn_fp16_fwd_workspace(const sl8_fp16_fwd_params* p);
int sl8_attn_fp16_fwd(const sl8_fp16_fwd_params* p, void* workspace, size_t workspace_bytes,
                      void* stream);

/*
 * The whole `attn_int8_fwd` step from 16-bit q, k, v in one host call: accuracy gate, Q / K
 * quantisation prologue and attention (the sequence of superl8/ops.py:70-175) queued back to back,
 * with the gate decided on the device (gate_flag / gate_want above), so nothing is read back to
 * the host and the call can be captured in a CUDA graph.  One dtype for q, k, v, out; D in
 * {64, 128, 256}, N > 0 (SL8_ERR_UNSUPPORTED otherwise: use the separate entry points).
 * ratio_threshold: the gate's max|q| / median|q| bound (reference: 12); <= 0 switches the gate
 * off (always the int8 kernel).  After the call the int32 at workspace + 256 (or *gate_flag) is the
 * gate's flag (non-zero: the full-precision kernel produced `out`) and the status word is at
 * workspace + 0 (or device_status).
 * No counterpart in the reference's C layer (its Python entry makes these calls one by one).
 */
typedef struct sl8_fused_fwd_params {
  const void* q; const void* k; const void* v; void* out;
  const int32_t* seqlens_q; const int32_t* seqlens_k;   /* nullable, int32[B] */
  int32_t* gate_flag;     /* nullable: a caller-owned device int32 that receives the gate's flag (zeroed by this
                             call) instead of workspace + 256 */
  void* device_status;    /* nullable: a caller-owned status word (256 bytes, zeroed by the caller, as the other
                             ops' workspace) used instead of workspace + 0, which this call zeroes itself */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype; int32_t causal; int32_t window_left;
  float ratio_threshold;
  double softmax_scale;
} sl8_fused_fwd_params;
size_t sl8_attn_int8_fwd_fused_workspace(const sl8_fused_fwd_params* p);
int sl8_attn_int8_fwd_fused(const sl8_fused_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same step for tensors in HOST memory (q, k, v, out are host pointers; pinned memory makes
 * the copies asynchronous and lets the two directions overlap): the call cuts the batch into
 * chunks of whole (batch, kv-head) units -- consecutive KV heads of one batch element with their
 * query heads, contiguous in every tensor -- and pipelines host->device copies, the fused step
 * above (gate decided per chunk on the device, as if the op were called on every chunk) and
 * device->host copies over a copy-in stream, the caller's stream and a copy-out stream, `slots`
 * staging slots deep.  The host thread never blocks; on return the caller's stream is ordered
 * after the last copy-out.  The reference has no such entry: its callers copy tensors to the
 * device themselves before superl8/ops.py:70-175 runs.
 * workspace: DEVICE memory, sl8_attn_int8_fwd_host_workspace() bytes (status word at + 0, then
 * the staging slots); the call allocates nothing on the device.  The first call on a device
 * creates the two copy streams and the events it keeps (make it before any stream capture).
 * kv_heads_per_chunk: 0 = choose (about 16 chunks per call, every chunk still filling the GPU);
 * slots: 0 = 3.  gate_flags (nullable): host int32 [sl8_attn_int8_fwd_host_chunks()], receives every
 * chunk's gate flag.  Same shape limits as sl8_attn_int8_fwd_fused; no seqlens.
 */
typedef struct sl8_host_fwd_params {
  const void* q; const void* k; const void* v; void* out;   /* HOST pointers, [B, H, S, D] contiguous */
  int32_t* gate_flags;                                       /* nullable HOST int32 [chunks] */
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype; int32_t causal; int32_t window_left;
  float ratio_threshold;
  double softmax_scale;
  int32_t kv_heads_per_chunk; int32_t slots;
} sl8_host_fwd_params;
size_t sl8_attn_int8_fwd_host_workspace(const sl8_host_fwd_params* p);
int sl8_attn_int8_fwd_host_chunks(const sl8_host_fwd_params* p);
int sl8_attn_int8_fwd_host(const sl8_host_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ---- full W8A8 prefill (int8 P.V) ------------------------------------------------------ */

/*
 * Replaces `attn_w8a8_fwd` (reference csrc/kernel/attn_w8a8_fwd.cu:72-160, kernel
 * csrc/include/attn_w8a8_fwd.cuh:30-235, binding csrc/fni8_api.cpp:249-255; the
 * `int8_pv=True` branch of superl8/ops.py:152-166).  q, k as for sl8_attn_int8_fwd; v int8
 * [B, Hkv, N, D] with v_scale fp32 [B, Hkv, D] (sl8_quantize_v_perchannel); out fp16.
 * P is re-quantised to int8 per query row and 64-key tile (per_warp_quant == 0) or per row and
 * 32-key half of the tile (per_warp_quant != 0, the reference's default).  causal_diag = N - M
 * aligns the causal diagonal to the sequence end (the Python layer passes it).  D in
 * {32, 64, 128, 256}.  No workspace.
 */
typedef struct sl8_w8a8_params {
  const int8_t* q; const float* q_scale;
  const int8_t* k; const float* k_scale;
  const int8_t* v; const float* v_scale;
  void* out;
  int32_t B, Hq, Hkv, M, N, D;
  int32_t causal; int32_t causal_diag; int32_t per_warp_quant;
} sl8_w8a8_params;
int sl8_attn_w8a8_fwd(const sl8_w8a8_params* p, void* stream);

/*
 * The same operator on the tensor-memory kernel of sl8_attn_int8_fwd (TMA tiles, Q.K^T as
 * tcgen05 kind::i8): P is snapped to the reference's int8 grid (same p_scale, same codes) and
 * code * p_scale enters a kind::f16 P.V against V's int8 codes held exactly as fp16, so the
 * result differs from the integer P.V only by the fp16 rounding of code * p_scale (2^-11
 * relative).  Serves D in {64, 128, 256}, N > 0 and causal_diag == N - M; anything else returns
 * SL8_ERR_UNSUPPORTED and belongs to sl8_attn_w8a8_fwd.  The workspace
 * (sl8_attn_w8a8_fwd_tc_workspace bytes, 16-byte aligned) holds the status word of the bounded
 * device-side waits in its first int32 (zeroed by the call) and V's codes as fp16.
 */
size_t sl8_attn_w8a8_fwd_tc_workspace(const sl8_w8a8_params* p);
int sl8_attn_w8a8_fwd_tc(const sl8_w8a8_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ---- packed variable-length prefill ------------------------------------------------- */

/*
 * Replaces `attn_int8_varlen` (reference csrc/kernel/attn_varlen_fwd.cu:45-110, kernel
 * csrc/include/attn_varlen_fwd.cuh:25-190, binding csrc/fni8_api.cpp; Python wrapper
 * superl8/ops.py:318-364).  Token-major packed tensors, the flash_attn_varlen convention:
 * q / out [total_q, Hq, D], k / v [total_k, Hkv, D], q_scale [total_q, Hq] (folded),
 * k_scale [total_k, Hkv]; cu_seqlens_q / cu_seqlens_k: int32 [B + 1] cumulative token offsets on
 * the device.  Every sequence attends within itself; the causal diagonal is aligned to the
 * sequence end.  D in {32, 64, 128} (the reference's set); V fp16 (reference) or bf16.
 * max_seqlen_q sizes the grid (no host read of cu_seqlens).  workspace: 256 bytes (status word).
 */
typedef struct sl8_varlen_params {
  const int8_t* q; const float* q_scale;
  const int8_t* k; const float* k_scale;
  const void* v; void* out;
  const int32_t* cu_seqlens_q; const int32_t* cu_seqlens_k;
  int32_t B, Hq, Hkv, D;
  int64_t total_q, total_k;
  int32_t max_seqlen_q;
  int32_t v_dtype; int32_t causal;
  int32_t backend;        /* SL8_BACKEND_* (tcgen05 for D = 64/128, else mma.sync) */
} sl8_varlen_params;
int sl8_attn_int8_varlen(const sl8_varlen_params* p, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Per-sequence K mean and smoothing + quantisation for the packed layout (reference
 * superl8/ops.py:268-315 `_varlen_smooth_k`, then `quantize_int8_rowwise`):
 * mean[b, h, :] = fp32 mean of k[cu[b]:cu[b+1], h, :]; k_i8 / k_scale = row quantisation of
 * round_to_dtype(k - mean of the token's own sequence).  k_smoothed (nullable) receives the
 * smoothed keys.  mean: fp32 [B, heads, D].
 */
int sl8_k_mean_packed(const void* k, int dtype, int64_t total_tokens, int32_t heads, int64_t D,
                      const int32_t* cu_seqlens, int32_t n_seq, float* mean, void* stream);
int sl8_smooth_quant_k_packed(const void* k, int dtype, int64_t total_tokens, int32_t heads, int64_t D,
                              const int32_t* cu_seqlens, int32_t n_seq, const float* mean,
                              int8_t* k_i8, float* k_scale, void* k_smoothed, void* stream);

/* ---- backward -------------------------------------------------------------- */

/*
 * Replaces `attn_bwd` (reference csrc/kernel/attn_bwd.cu:62-109, kernels
 * csrc/include/attn_bwd.cuh:156-331 and :337-535, binding csrc/fni8_api.cpp:256-259; the
 * mathematics it implements are superl8/autograd.py:29-45).  q, o, dout, dq: [B, Hq, M, D];
 * k, v, dk, dv: [B, Hkv, N, D]; lse: fp32 [B, Hq, M], natural log, as the forward returns it.
 * One dtype for all 16-bit tensors (reference: fp16 only; bf16 also served).  D in {32, 64, 128}
 * (the reference's set).  dk / dv are summed over the query heads of a KV head.  M == 0 or
 * N == 0 zero-fills the gradients (attn_bwd.cu:88).  Two passes, no atomics: bitwise
 * reproducible.  workspace: sl8_attn_bwd_workspace() bytes (status word + fp32 [B, Hq, M]);
 * the tcgen05 passes zero the status word themselves and raise it to
 * SL8_ERR_DEVICE_TIMEOUT if a bounded device-side wait expires (sl8_read_device_status).
 */
typedef struct sl8_bwd_params {
  const void* q; const void* k; const void* v; const void* o; const void* dout;
  const float* lse;
  void* dq; void* dk; void* dv;
  int32_t B, Hq, Hkv, M, N, D;
  int32_t dtype; int32_t causal;
  float softmax_scale;
  int32_t backend;        /* SL8_BACKEND_* (AUTO: tcgen05 for D = 64/128, else mma.sync) */
} sl8_bwd_params;
size_t sl8_attn_bwd_workspace(const sl8_bwd_params* p);
int sl8_attn_bwd(const sl8_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ---- decode: split-KV, one query row per sequence ----------------------- */

typedef struct sl8_decode_params {
  const int8_t* q;        /* [B, Hq, 1, D] int8 */
  const float* q_scale;   /* [B, Hq] folded */
  const int8_t* k;        /* [B, Hkv, N, D] int8 cache */
  const float* k_scale;   /* [B, Hkv, N] per-token scales */
  const void* v;          /* [B, Hkv, N, D] fp16 cache */
  void* out;              /* [B, Hq, 1, D] fp16 */
  const int32_t* context_lens; /* int32[B] or NULL (every sequence uses N keys) */
  int32_t B, Hq, Hkv, N, D;
  int32_t num_splits;     /* 1..256, or -1 = choose (sl8_choose_n_splits) */
} sl8_decode_params;

/*
 * Split count used when num_splits == -1.  The reference's heuristic
 * (csrc/kernel/attn_decode.cu:33-53) sizes one-warp blocks for 80 SMs; this one
 * sizes 128-thread blocks that each serve a whole GQA group for 148 SMs.
 */
int sl8_choose_n_splits(int64_t N, int64_t B_times_Hkv);

/*
 * Replaces `attn_int8_decode` (reference csrc/kernel/attn_decode.cu:163-240;
 * kernels csrc/include/attn_decode.cuh:47-132 and :430-466; binding
 * csrc/fni8_api.cpp:260-263).  Split s of a sequence owns keys
 * [s*per, min(len, (s+1)*per)), per = ceil(N / num_splits); partials
 * (O, m, l) go to the workspace and a second kernel merges them by
 * log-sum-exp.  N == 0 writes zeros.  num_splits 0 or > 256 is rejected.
 * workspace: sl8_attn_int8_decode_workspace() bytes (status word + partials).
 */
size_t sl8_attn_int8_decode_workspace(const sl8_decode_params* p);
int sl8_attn_int8_decode(const sl8_decode_params* p, void* workspace, size_t workspace_bytes,
                         void* stream);

/*
 * Decode against an int8 V cache with one fp32 scale per (batch, KV head, channel): replaces
 * `attn_int8_decode_kv8` (reference csrc/include/attn_decode.cuh:141-224 `decode_split_i8v_kernel`,
 * Python wrapper superl8/ops.py:671-727 `attn_decode_cached`).  p->v is int8 [B, Hkv, N, D];
 * v_scale fp32 [B, Hkv, D]; everything else as sl8_attn_int8_decode (same workspace size).
 * O accumulates p * float(v) and the channel scale multiplies the split partial.
 */
int sl8_attn_int8_decode_kv8(const sl8_decode_params* p, const float* v_scale, void* workspace,
                             size_t workspace_bytes, void* stream);

/*
 * Per-channel symmetric int8 of V for that cache (reference superl8/quant/core.py:98-110
 * `quantize_v_perchannel`): v_scale[bh, d] = max_n |v[bh, n, d]| / 127 (0 -> 1),
 * v_i8 = clamp(rint(v / v_scale), -127, 127).  v: fp16 / bf16 [BH, N, D].
 * workspace: sl8_k_mean_workspace(BH, N, D) bytes.
 */
int sl8_quantize_v_perchannel(const void* v, int dtype, int64_t BH, int64_t N, int64_t D, int8_t* v_i8,
                              float* v_scale, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Decode for callers that cannot allocate device memory.  No counterpart in the
 * reference (its op allocates its partials with at::empty on every call,
 * csrc/kernel/attn_decode.cu:214-217).
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a plugin handed a
 * fixed memory budget by its host application, a real-time serving loop that must not
 * take the allocator's locks or risk an out-of-memory in steady state, or a host that
 * keeps every byte of the device under its own arena and gives a library none.  Such a
 * caller passes inputs and the output exactly as for sl8_attn_int8_decode; the split
 * partials (O, m, l) go to a fixed array of SL8_DECODE_STATIC_SCRATCH_BYTES inside the
 * library image instead of a caller workspace.  Every GPU that loads the library holds
 * that array until the process exits.
 *
 * Limits and rules:
 *  - need = 256 + num_splits * B * Hq * (D + 2) * 4 bytes must fit the array.  With
 *    num_splits == -1 the split count is lowered until it fits; an explicit num_splits
 *    that does not fit, or a batch too large even for one split, returns
 *    SL8_ERR_TOO_LARGE and launches nothing.
 *  - This function calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - The first call on each device looks up the array's device address (once per
 *    device, with that device current, under a host lock).
 *  - All calls on a device share the one array, and it keeps the previous call's
 *    contents (every value a call reads it has written itself first, so nothing needs
 *    clearing between calls).  Two calls that overlap on the GPU -- different streams,
 *    or the same stream from two threads without ordering -- race on it: serialise them.
 *  - device_status (nullable): a caller-owned, 4-byte aligned device int32, zeroed by the
 *    caller; it is set to SL8_ERR_DEVICE_TIMEOUT if a bounded device-side wait expires
 *    (only that one word is touched; read it with sl8_read_device_status).  With NULL the
 *    word lives at the start of the built-in array: every call zeroes it on the stream
 *    before its kernels, and sl8_decode_static_status(stream) synchronises the stream
 *    and returns (and clears) it -- SL8_OK or SL8_ERR_DEVICE_TIMEOUT for the calls made
 *    on the current device since the last read.
 */
#define SL8_DECODE_STATIC_SCRATCH_BYTES (32u << 20)
int sl8_attn_int8_decode_static(const sl8_decode_params* p, int32_t* device_status, void* stream);
int sl8_decode_static_status(void* stream);

/*
 * Tensor-pipe peak probe: one block per SM issues `iters` x 4 back-to-back tcgen05.mma
 * (M128 N256, 32-byte K step; kind::i8 if kind_i8 != 0, else kind::f16 on fp16) on constant
 * shared-memory operands.  *ops_per_launch (host, nullable) receives the operation count
 * (2 x MACs) of the launch; time the launch with events to get the sustained peak that
 * "fraction of INT8 peak" is quoted against.  No counterpart in the reference.
 */
int sl8_tensor_peak_probe(int kind_i8, int iters, double* ops_per_launch, void* workspace,
                          size_t workspace_bytes, void* stream);
/* The same probe with N = n_cols (64, 128 or 256) columns per instruction: what the pipe sustains
 * for the instruction shapes a kernel actually issues (smaller N = shorter instructions). */
int sl8_tensor_peak_probe_n(int kind_i8, int n_cols, int iters, double* ops_per_launch, void* workspace,
                            size_t workspace_bytes, void* stream);

/*
 * Self-test of the bounded device-side wait every kernel of this library uses: one block waits
 * on a barrier nothing ever arrives at, with a limit of limit_ns (1 .. 100 000 000) nanoseconds;
 * when the limit runs out the kernel raises the status word (the first int32 of `workspace`, at
 * least 256 bytes, zeroed by the caller) to SL8_ERR_DEVICE_TIMEOUT and returns normally, so the
 * context stays usable.  The second int32 of the workspace receives 2 (the wait gave up) or 1
 * (it was satisfied, which cannot happen).  Shows a host how an expired wait looks
 * (sl8_read_device_status) without making any real kernel fail.  No counterpart in the
 * reference, whose kernels have no inter-thread waits.
 */
int sl8_wait_timeout_selftest(void* workspace, size_t workspace_bytes, uint64_t limit_ns, void* stream);

/* Synchronises the stream and returns the device status word of a workspace
 * (SL8_OK or SL8_ERR_DEVICE_TIMEOUT); clears it. */
int sl8_read_device_status(void* workspace, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SUPERL8_B200_H_ */
