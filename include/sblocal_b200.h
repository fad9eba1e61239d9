/*
 * sblocal_b200 -- C ABI of the B200 (sm_100a) SBLocal attention forward.
 *
 * The reference (HazyResearch/fly) is pure Python and has no FFI of its own;
 * each entry point below names the reference function(s) whose work it
 * replaces (paths relative to the reference tree).  All tensors are BORROWED
 * device pointers: the caller (PyTorch in the Python shell) owns inputs,
 * outputs and the workspace.  Every function returns 0 on success or a
 * negative SblStatus; sbl_last_error() then describes the failure for the
 * calling thread.  No function takes or returns a C++ or torch type.
 *
 * Notation: tau = softmax_temp, r = rows of the projection W (the feature
 * count is m = 2r, the "cosh" Performer map), w = local_context, the window
 * of query i is keys i - w/2 ... i - w/2 + w - 1 (integer division).
 */
#ifndef SBLOCAL_B200_H_
#define SBLOCAL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SBL_ABI_VERSION 1

typedef enum SblStatus {
  SBL_OK = 0,
  SBL_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad shape/stride/alignment            */
  SBL_ERR_UNSUPPORTED = -2,      /* valid request this build has no kernel for          */
  SBL_ERR_WORKSPACE = -3,        /* workspace null, misaligned or too small             */
  SBL_ERR_CUDA = -4,             /* a CUDA runtime/driver call failed                   */
  SBL_ERR_DEVICE_STATUS = -5     /* a kernel recorded an error (e.g. a bounded wait ran out) */
} SblStatus;

typedef enum SblDType { SBL_DTYPE_F32 = 0, SBL_DTYPE_BF16 = 1 } SblDType;

/* Run the generic fp32-math kernels even where the bf16 tensor-core kernels apply (needed by
 * sbl_attention_weights, which reads the fp32 phi(Q)/phi(K) those kernels leave in the workspace). */
#define SBL_FLAG_GENERIC_PATH 1

/*
 * One problem description shared by all entry points.
 *
 * q (B,T,H,E), k (B,S,H,E), v (B,S,H,D), out (B,T,H,D): the layouts of
 * SBLocalAttention.forward's arguments (src/models/attention/
 * sblocal_attention.py:48-50).  The last axis is contiguous; the other three
 * carry ELEMENT strides, so the permuted copies the reference makes
 * (sblocal_attention.py:73-75) are never needed.
 *
 * Sequence sharding: T and S count the rows present in THIS call's buffers.
 * q_pos0 / k_pos0 are the global sequence positions of row 0 of q/out and of
 * k/v; key_lengths (or S_total when key_lengths is null) bound the valid
 * global key positions.  sum_lo..sum_hi (buffer rows) select the keys this
 * rank contributes to the global summary; halo rows lie outside that range.
 * A single-GPU call uses q_pos0 = k_pos0 = 0, S_total = S, sum_lo = 0,
 * sum_hi = S.
 */
typedef struct SblParams {
  int32_t dtype;              /* SblDType of q, k, v, out                                  */
  int32_t B, H, T, S, E, D;   /* batch, heads, query rows, key rows, qk dim, value dim      */
  int32_t r;                  /* projection rows; features m = 2r                          */
  int32_t w;                  /* local_context                                             */
  float softmax_temp;         /* tau > 0                                                   */
  float softmax_eps;          /* eps added to every feature as eps/sqrt(m)                 */
  const void* q;  int64_t q_stride_b, q_stride_t, q_stride_h;
  const void* k;  int64_t k_stride_b, k_stride_s, k_stride_h;
  const void* v;  int64_t v_stride_b, v_stride_s, v_stride_h;
  void* out;      int64_t o_stride_b, o_stride_t, o_stride_h;
  const float* W;             /* (r,E) fp32 row-major: projection_matrix, passed unchanged */
  const int64_t* key_lengths; /* (B,) device int64, or null = no padding                   */
  int64_t q_pos0, k_pos0;     /* global positions of buffer row 0                          */
  int64_t S_total;            /* global number of keys                                     */
  int32_t sum_lo, sum_hi;     /* key buffer rows that enter this rank's summary            */
  int32_t flags;              /* SBL_FLAG_* bits                                           */
  int32_t reserved[3];        /* must be 0                                                 */
} SblParams;

/* ABI version (SBL_ABI_VERSION of the built library). */
int sbl_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* sbl_last_error(void);

/* 1 if the library was built with the tcgen05/TMA bf16 kernels. */
int sbl_has_tensor_path(void);

/* Bytes of device workspace (256-byte aligned base) any entry point below
 * needs for this problem.  The workspace carries phi(K) from sbl_key_summary
 * to sbl_band_forward, so a staged call sequence must reuse one buffer. */
int sbl_workspace_bytes(const SblParams* p, size_t* bytes);

/*
 * Whole forward on one stream; replaces SBLocalAttention.forward
 * (sblocal_attention.py:43-137) for need_weights=False, causal=False,
 * attn_mask=None, dropout inactive: equals sbl_key_logscale +
 * sbl_key_summary + sbl_band_forward with the summary kept in the workspace.
 */
int sbl_forward(const SblParams* p, void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Stage 1: beta[b,h] = max over the key rows sum_lo..sum_hi and all m
 * features of (+-sqrt(tau) W k - tau|k|^2/2 - ln(m)/2): the key log-scale of
 * softmax_kernel(is_query=False) (src/models/attention/feature_maps_sb.py:77-78).
 * beta: (B,H) fp32 device.  Sequence-sharded callers all-reduce it with MAX.
 * For bf16 inputs with E = D = 128, r = 256 and eps = 0 (the second shape of
 * the tensor-core kernels) the value is an upper bound of that maximum taken
 * from the key norms (wmax|k| - tau|k|^2/2 - ln(m)/2, wmax the largest row
 * norm of sqrt(tau) W): with eps = 0 every stabiliser >= the maximum gives
 * the same output, and stages 2 and 3 only need the SAME beta.
 */
int sbl_key_logscale(const SblParams* p, void* workspace, size_t workspace_bytes, float* beta,
                     void* cuda_stream);

/*
 * Stage 2: phi(K) = exp(kd - beta) + eps/sqrt(m), zero at padded keys
 * (feature_maps_sb.py:79-81, sblocal_attention.py:83-85), kept in the
 * workspace for every key buffer row; kv[b,h] = phi(K)^T V (m,D) and
 * ksum[b,h] = sum_s phi(k_s) (m) over rows sum_lo..sum_hi: linear_attention
 * and linear_attention_normalization (src/models/attention/
 * scatterbrain_utils.py:18-20,48-49).  kv (B,H,m,D), ksum (B,H,m): fp32
 * device.  Sequence-sharded callers all-reduce both with SUM.
 */
int sbl_key_summary(const SblParams* p, void* workspace, size_t workspace_bytes, const float* beta,
                    float* kv, float* ksum, void* cuda_stream);

/*
 * Stage 3: per query block: phi(Q) (feature_maps_sb.py:70-75), banded
 * tau QK^T and phi(Q)phi(K)^T (the two local_dot_product calls,
 * sblocal_attention.py:90-105), the joint normaliser (:109-115), the combined
 * weights (:119), the banded weighted average plus the low-rank term
 * (local_weighted_average, :121-122), written to out in (B,T,H,D) layout.
 */
int sbl_band_forward(const SblParams* p, void* workspace, size_t workspace_bytes, const float* beta,
                     const float* kv, const float* ksum, void* cuda_stream);

/*
 * Dense attention matrices of the need_weights / return_attn_unnormalized branch
 * (sblocal_attention.py:124-136), for tests and inspection: O(T*S) memory.  Call after sbl_forward (or
 * the three stages) on the same workspace with SBL_FLAG_GENERIC_PATH set in both calls.
 *   attn            (B,H,T,S) fp32: banded weights scattered into the dense matrix + phi(Q)phi(K)^T * prime_scale
 *   attn_unnorm     attn * exp(log_normalization)                     (null to skip)
 *   attn_lr_unnorm  phi(Q)phi(K)^T * exp(prime_log_scale)             (null to skip)
 */
int sbl_attention_weights(const SblParams* p, void* workspace, size_t workspace_bytes, float* attn,
                          float* attn_unnorm, float* attn_lr_unnorm, void* cuda_stream);

/*
 * Synchronises the stream and reports whether any kernel of the preceding
 * calls on this workspace gave up on a bounded wait (every device-side wait
 * has an iteration limit, after which the kernel records the wait site,
 * finishes and frees its tensor memory), or whether the bf16 tensor-core
 * kernels met logits so large that an exponential left the fp32 range (those
 * kernels never rescale; the generic kernels, SBL_FLAG_GENERIC_PATH, do), or
 * met query rows whose in-window low-rank estimate is more than 16 times their
 * exact in-window softmax mass, where bf16 products lose accuracy (row error
 * about that ratio times 2^-8; logits 3-4 times the unit scale do this):
 * SBL_ERR_DEVICE_STATUS in all three cases; the outputs of those calls are
 * invalid in the first two and degraded in the third.  No counterpart in the reference (its device faults surface as
 * CUDA errors, and its logsumexp form has no such range limit).
 */
int sbl_check_status(const SblParams* p, void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * For hosts that must not synchronise: *offset receives the byte offset, inside
 * the workspace of this problem, of three int32 status words the tensor-core
 * kernels write (word 0: site of a bounded wait that ran out, word 1: 1 if an
 * exponential left the fp32 range because the logits are far above unit
 * scale, word 2: 1 if a row's low-rank estimate swamped its exact part, see
 * sbl_check_status; all 0 = fine).  A caller may copy them out asynchronously behind a
 * forward and look at them later; sbl_check_status reads the same words with
 * a synchronisation.  Returns SBL_ERR_UNSUPPORTED for problems that run the
 * generic kernels (they keep no status words).  No counterpart in the
 * reference.
 */
int sbl_status_words(const SblParams* p, size_t* offset);

/*
 * Self-test of that mechanism: launches one warp that waits on a barrier
 * nothing arrives on.  The wait runs out after its iteration limit (about a
 * second at most), the kernel records the wait site and ends normally, and
 * the call returns SBL_ERR_DEVICE_STATUS with the site (99) in
 * sbl_last_error(); the device context stays usable.  SBL_OK would mean the
 * limit did not work.  workspace: >= 256 bytes of device memory, 16-byte
 * aligned.  No counterpart in the reference.
 */
int sbl_selftest_wait_timeout(void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Feature maps alone, for parity checks against
 * SBPerformerFeatures.forward_queries / forward_keys
 * (feature_maps_sb.py:148-156 -> softmax_kernel :51-82).
 *   sbl_query_features: q_prime (B,H,T,m) fp32, q_log_scale (B,H,T) fp32.
 *   sbl_key_features:   k_prime (B,H,S,m) fp32 (padding zeroed as
 *                       sblocal_attention.py:83-85), k_log_scale (B,H) fp32.
 */
int sbl_query_features(const SblParams* p, void* workspace, size_t workspace_bytes, float* q_prime,
                       float* q_log_scale, void* cuda_stream);
int sbl_key_features(const SblParams* p, void* workspace, size_t workspace_bytes, float* k_prime,
                     float* k_log_scale, void* cuda_stream);

/*
 * No counterpart in the reference: an addition for hosts that are not allowed
 * to allocate device memory (a process whose GPU memory is owned by one
 * start-up arena, or a loop in which cudaMalloc is banned because it stalls
 * the device) and so cannot supply a workspace.  Same value as
 * sbl_key_logscale run with SBL_FLAG_GENERIC_PATH (the exact maximum, fp32
 * projection); for bf16 inputs with E = 64, r = 128 the plain sbl_key_logscale
 * takes the tensor-core kernels, which round the projection to bf16, and the
 * two then differ by up to a few 1e-2 (both are valid stabilisers); with
 * E = 128, r = 256 the plain call returns an upper bound from the key norms.  The
 * scratch (sqrt(tau)*W, r*E floats) is a fixed 128 KiB array inside the
 * library image, present on every GPU that loads the library.  Limits:
 * r*E <= SBL_STATIC_PROJ_FLOATS, else SBL_ERR_UNSUPPORTED.  All calls on a
 * device share that array; calls that overlap on the GPU race on it, so keep
 * them on one stream.  The first call on each device resolves the array's
 * address through the CUDA runtime, and the first launch per input dtype may
 * load kernel code: make one call per dtype at start-up, before any stream
 * capture.  Allocates nothing.  Errors: sbl_static_last_error().
 */
#define SBL_STATIC_PROJ_FLOATS 32768
int sbl_key_logscale_static(const SblParams* p, float* beta, void* cuda_stream);
const char* sbl_static_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* SBLOCAL_B200_H_ */
