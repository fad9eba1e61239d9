// C-ABI layer of sblocal_b200: argument validation, workspace planning and
// dispatch between the generic SIMT kernels and the bf16 tensor-core kernels.
// Declared in include/sblocal_b200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "sbl_common.cuh"

namespace sbl {
namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

int cuda_fail(cudaError_t e, const char* what) {
  return fail(SBL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Shape, pointer and sharding checks common to every entry point.
int validate(const SblParams* p) {
  if (!p) return fail(SBL_ERR_INVALID_ARGUMENT, "params is null");
  if (p->dtype != SBL_DTYPE_F32 && p->dtype != SBL_DTYPE_BF16)
    return fail(SBL_ERR_INVALID_ARGUMENT, "dtype %d is not SBL_DTYPE_F32 or SBL_DTYPE_BF16", p->dtype);
  if (p->B <= 0 || p->H <= 0 || p->T <= 0 || p->S <= 0 || p->E <= 0 || p->D <= 0)
    return fail(SBL_ERR_INVALID_ARGUMENT, "B,H,T,S,E,D must be positive (got %d,%d,%d,%d,%d,%d)", p->B, p->H,
                p->T, p->S, p->E, p->D);
  if (p->r <= 0) return fail(SBL_ERR_INVALID_ARGUMENT, "projection rows r must be positive (got %d)", p->r);
  if (p->w <= 0) return fail(SBL_ERR_INVALID_ARGUMENT, "local_context w must be positive (got %d)", p->w);
  if (!(p->softmax_temp > 0.f)) return fail(SBL_ERR_INVALID_ARGUMENT, "softmax_temp must be > 0");
  if (!(p->softmax_eps >= 0.f)) return fail(SBL_ERR_INVALID_ARGUMENT, "softmax_eps must be >= 0");
  if (!p->q || !p->k || !p->v || !p->out || !p->W)
    return fail(SBL_ERR_INVALID_ARGUMENT, "q, k, v, out and W must be non-null device pointers");
  if (p->D > 128) return fail(SBL_ERR_UNSUPPORTED, "value dim D=%d > 128 has no kernel", p->D);
  if ((int64_t)p->B * p->H > 65535)
    return fail(SBL_ERR_UNSUPPORTED, "B*H=%lld exceeds the grid limit 65535", (long long)p->B * p->H);
  if (p->flags & ~SBL_FLAG_GENERIC_PATH) return fail(SBL_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", p->flags);
  for (int i = 0; i < 3; ++i)
    if (p->reserved[i] != 0) return fail(SBL_ERR_INVALID_ARGUMENT, "reserved fields must be 0");
  if (p->S_total <= 0 || p->q_pos0 < 0 || p->k_pos0 < 0)
    return fail(SBL_ERR_INVALID_ARGUMENT, "S_total must be positive and q_pos0/k_pos0 non-negative");
  if (p->k_pos0 + p->S > p->S_total)
    return fail(SBL_ERR_INVALID_ARGUMENT, "key buffer rows [%lld,%lld) exceed S_total=%lld", (long long)p->k_pos0,
                (long long)(p->k_pos0 + p->S), (long long)p->S_total);
  if (p->sum_lo < 0 || p->sum_hi > p->S || p->sum_lo > p->sum_hi)
    return fail(SBL_ERR_INVALID_ARGUMENT, "summary rows [%d,%d) are not inside the key buffer [0,%d)", p->sum_lo,
                p->sum_hi, p->S);
  // every key a local query can see must be present in the key buffer (halo)
  int64_t need_lo = p->q_pos0 - p->w / 2;
  if (need_lo < 0) need_lo = 0;
  int64_t need_hi = p->q_pos0 + p->T - 1 - p->w / 2 + p->w;  // exclusive
  if (need_hi > p->S_total) need_hi = p->S_total;
  if (need_lo < need_hi && (p->k_pos0 > need_lo || p->k_pos0 + p->S < need_hi))
    return fail(SBL_ERR_INVALID_ARGUMENT,
                "key buffer rows [%lld,%lld) do not cover the window halo [%lld,%lld) of the local queries",
                (long long)p->k_pos0, (long long)(p->k_pos0 + p->S), (long long)need_lo, (long long)need_hi);
  return SBL_OK;
}

int check_workspace(const Workspace& ws, void* workspace, size_t bytes) {
  if (!workspace) return fail(SBL_ERR_WORKSPACE, "workspace is null (need %zu bytes)", ws.total);
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
    return fail(SBL_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (bytes < ws.total) return fail(SBL_ERR_WORKSPACE, "workspace has %zu bytes, need %zu", bytes, ws.total);
  return SBL_OK;
}

int prepare(const SblParams* p, void* workspace, size_t bytes, Workspace* ws) {
  int rc = validate(p);
  if (rc != SBL_OK) return rc;
  plan_workspace(*p, ws);
  return check_workspace(*ws, workspace, bytes);
}

}  // namespace

void plan_workspace(const SblParams& p, Workspace* ws) {
  const size_t BH = (size_t)p.B * p.H, m = 2 * (size_t)p.r;
  ws->tensor = tc_supported(p) && !(p.flags & SBL_FLAG_GENERIC_PATH);
  // split the summary over key rows: at most 64 splits, at least 256 rows each
  const int rows = p.sum_hi - p.sum_lo;
  int split_rows = 256;
  while (div_up(rows > 0 ? rows : 1, split_rows) > 64) split_rows *= 2;
  ws->split_rows = split_rows;
  ws->nsplit = (int)div_up(rows > 0 ? rows : 1, split_rows);
  if (ws->tensor) {
    // tensor path: CTAs stream 128-key tiles; about two CTAs per SM-count over all (b,h)
    const int ntiles = (int)div_up(p.S, 128);
    // (head dim 128 runs four CTAs, one per projection quarter, on every split)
    const size_t units = BH * (p.E == 128 ? 4 : 1);
    int ns = (int)((296 + units / 2) / units);
    if (ns < 1) ns = 1;
    if (ns > ntiles) ns = ntiles;
    ws->nsplit = ns;
    ws->split_rows = 0;
  }
  size_t off = 0;
  ws->wt = off;      off = align_up(off + (size_t)p.r * p.E * sizeof(float));
  ws->phik = off;    off = align_up(off + BH * p.S * m * (ws->tensor ? 2 : 4));
  ws->phiq = off;    off = align_up(off + (ws->tensor ? (size_t)p.r * p.E * 2 : BH * p.T * m * 4));
  ws->qls = off;     off = align_up(off + (ws->tensor ? BH * m * p.D * 2 : BH * p.T * 4));
  ws->beta = off;    off = align_up(off + BH * 4);
  ws->kv = off;      off = align_up(off + BH * m * p.D * 4);
  ws->ksum = off;    off = align_up(off + BH * m * 4);
  ws->partial = off; off = align_up(off + BH * ws->nsplit * m * (ws->tensor ? p.D + 16 : p.D + 1) * 4);
  ws->lognorm = off; off = align_up(off + (ws->tensor ? BH * m * 4 : BH * p.T * 4));
  ws->status = off;  off = align_up(off + 64);
  ws->total = off;
}

}  // namespace sbl

using namespace sbl;

extern "C" {

int sbl_version(void) { return SBL_ABI_VERSION; }

const char* sbl_last_error(void) { return g_err; }

int sbl_has_tensor_path(void) {
  SblParams p{};
  p.dtype = SBL_DTYPE_BF16;
  p.B = p.H = 1; p.T = p.S = 256; p.E = p.D = 64; p.r = 128; p.w = 256;
  p.softmax_temp = 0.125f; p.S_total = 256; p.sum_hi = 256;
  p.q_stride_t = p.k_stride_s = p.v_stride_s = p.o_stride_t = 64;
  p.q = p.k = p.v = p.out = reinterpret_cast<void*>(256);
  p.W = reinterpret_cast<const float*>(256);
  return tc_supported(p) ? 1 : 0;
}

int sbl_workspace_bytes(const SblParams* p, size_t* bytes) {
  if (!bytes) return fail(SBL_ERR_INVALID_ARGUMENT, "bytes is null");
  int rc = validate(p);
  if (rc != SBL_OK) return rc;
  Workspace ws;
  plan_workspace(*p, &ws);
  *bytes = ws.total;
  return SBL_OK;
}

int sbl_key_logscale(const SblParams* p, void* workspace, size_t workspace_bytes, float* beta, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!beta) return fail(SBL_ERR_INVALID_ARGUMENT, "beta is null");
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if (ws.tensor) {
    if ((e = tc_prepare_projection(*p, ws, base, st, true)) != cudaSuccess) return cuda_fail(e, "prepare projection");
    if ((e = tc_key_logscale(*p, ws, base, beta, st)) != cudaSuccess) return cuda_fail(e, "key logscale");
  } else {
    if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
    if ((e = f32_key_logscale(*p, ws, base, beta, st)) != cudaSuccess) return cuda_fail(e, "key logscale");
  }
  return SBL_OK;
}

int sbl_key_summary(const SblParams* p, void* workspace, size_t workspace_bytes, const float* beta, float* kv,
                    float* ksum, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!beta || !kv || !ksum) return fail(SBL_ERR_INVALID_ARGUMENT, "beta, kv and ksum must be non-null");
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if (ws.tensor) {
    if ((e = tc_prepare_projection(*p, ws, base, st, false)) != cudaSuccess) return cuda_fail(e, "prepare projection");
    if ((e = tc_key_summary(*p, ws, base, beta, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "key summary");
    return SBL_OK;
  }
  float* phik = reinterpret_cast<float*>(base + ws.phik);
  if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
  if ((e = f32_key_features(*p, ws, base, beta, phik, st)) != cudaSuccess) return cuda_fail(e, "key features");
  if ((e = f32_key_summary(*p, ws, base, phik, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "key summary");
  return SBL_OK;
}

int sbl_band_forward(const SblParams* p, void* workspace, size_t workspace_bytes, const float* beta,
                     const float* kv, const float* ksum, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!beta || !kv || !ksum) return fail(SBL_ERR_INVALID_ARGUMENT, "beta, kv and ksum must be non-null");
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if (ws.tensor) {
    if ((e = tc_prepare_projection(*p, ws, base, st, false)) != cudaSuccess) return cuda_fail(e, "prepare projection");
    if ((e = tc_band(*p, ws, base, beta, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "band forward");
    return SBL_OK;
  }
  if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
  if ((e = f32_query_features(*p, ws, base, reinterpret_cast<float*>(base + ws.phiq),
                              reinterpret_cast<float*>(base + ws.qls), st)) != cudaSuccess)
    return cuda_fail(e, "query features");
  if ((e = f32_band(*p, ws, base, beta, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "band forward");
  return SBL_OK;
}

int sbl_forward(const SblParams* p, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  float* beta = reinterpret_cast<float*>(base + ws.beta);
  float* kv = reinterpret_cast<float*>(base + ws.kv);
  float* ksum = reinterpret_cast<float*>(base + ws.ksum);
  cudaError_t e;
  if (ws.tensor) {
    // five launches: projection (+ log-scale reset), log-scale bound, keys, combine (+ bf16 KV), band
    if ((e = tc_prepare_projection(*p, ws, base, st, true, beta)) != cudaSuccess)
      return cuda_fail(e, "prepare projection");
    if ((e = tc_key_logscale_bound(*p, ws, base, beta, st, true)) != cudaSuccess)
      return cuda_fail(e, "key logscale bound");
    if ((e = tc_key_summary(*p, ws, base, beta, kv, ksum, st, true)) != cudaSuccess) return cuda_fail(e, "key summary");
    if ((e = tc_band(*p, ws, base, beta, kv, ksum, st, true)) != cudaSuccess) return cuda_fail(e, "band forward");
    return SBL_OK;
  }
  float* phik = reinterpret_cast<float*>(base + ws.phik);
  if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
  if ((e = f32_key_logscale(*p, ws, base, beta, st)) != cudaSuccess) return cuda_fail(e, "key logscale");
  if ((e = f32_key_features(*p, ws, base, beta, phik, st)) != cudaSuccess) return cuda_fail(e, "key features");
  if ((e = f32_key_summary(*p, ws, base, phik, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "key summary");
  if ((e = f32_query_features(*p, ws, base, reinterpret_cast<float*>(base + ws.phiq),
                              reinterpret_cast<float*>(base + ws.qls), st)) != cudaSuccess)
    return cuda_fail(e, "query features");
  if ((e = f32_band(*p, ws, base, beta, kv, ksum, st)) != cudaSuccess) return cuda_fail(e, "band forward");
  return SBL_OK;
}

int sbl_attention_weights(const SblParams* p, void* workspace, size_t workspace_bytes, float* attn,
                          float* attn_unnorm, float* attn_lr_unnorm, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!attn) return fail(SBL_ERR_INVALID_ARGUMENT, "attn is null");
  if (ws.tensor)
    return fail(SBL_ERR_INVALID_ARGUMENT, "sbl_attention_weights needs SBL_FLAG_GENERIC_PATH in this and the forward call");
  if (p->q_pos0 != 0 || p->k_pos0 != 0 || p->S_total != p->S)
    return fail(SBL_ERR_UNSUPPORTED, "dense attention weights are not built for sequence shards");
  char* base = static_cast<char*>(workspace);
  cudaError_t e = f32_attention_weights(*p, ws, base, reinterpret_cast<const float*>(base + ws.beta), attn, attn_unnorm,
                                        attn_lr_unnorm, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "attention weights");
  return SBL_OK;
}

int sbl_check_status(const SblParams* p, void* workspace, size_t workspace_bytes, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  if (!ws.tensor) {
    cudaError_t e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? SBL_OK : cuda_fail(e, "stream synchronize");
  }
  int host[3] = {0, 0, 0};
  cudaError_t e = tc_read_status(ws, static_cast<char*>(workspace), host, st);
  if (e != cudaSuccess) return cuda_fail(e, "read device status");
  if (host[0] != 0)
    return fail(SBL_ERR_DEVICE_STATUS, "a bounded wait ran out inside a kernel (wait site %d); results are invalid",
                host[0]);
  if (host[1] != 0)
    return fail(SBL_ERR_DEVICE_STATUS,
                "numeric range: an exponential of the bf16 tensor-core kernels left the fp32 range (logits far above "
                "unit scale); results are invalid -- rerun with SBL_FLAG_GENERIC_PATH");
  if (host[2] != 0)
    return fail(SBL_ERR_DEVICE_STATUS,
                "precision: for some query rows the in-window low-rank estimate is more than 16 times the exact "
                "in-window softmax mass (logits 3-4 times the unit scale), where the bf16 tensor-core kernels lose "
                "accuracy (row error ~ that ratio x 2^-8); rerun with SBL_FLAG_GENERIC_PATH");
  return SBL_OK;
}

int sbl_status_words(const SblParams* p, size_t* offset) {
  if (!offset) return fail(SBL_ERR_INVALID_ARGUMENT, "offset is null");
  int rc = validate(p);
  if (rc != SBL_OK) return rc;
  Workspace ws;
  plan_workspace(*p, &ws);
  if (!ws.tensor) return fail(SBL_ERR_UNSUPPORTED, "the generic kernels keep no status words");
  *offset = ws.status;
  return SBL_OK;
}

int sbl_selftest_wait_timeout(void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (!workspace || workspace_bytes < 256) return fail(SBL_ERR_INVALID_ARGUMENT, "self-test needs a 256-byte workspace");
  if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0)
    return fail(SBL_ERR_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
  int host = 0;
  cudaError_t e = tc_wait_selftest(static_cast<int*>(workspace), &host, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "wait self-test");
  if (host != 0)
    return fail(SBL_ERR_DEVICE_STATUS, "a bounded wait ran out inside a kernel (wait site %d); results are invalid",
                host);
  return SBL_OK;
}

// The two feature-map entry points always run the fp32 generic kernels: they
// exist to compare phi(Q), phi(K) and their log-scales with the reference's
// softmax_kernel element by element.
int sbl_query_features(const SblParams* p, void* workspace, size_t workspace_bytes, float* q_prime,
                       float* q_log_scale, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!q_prime || !q_log_scale) return fail(SBL_ERR_INVALID_ARGUMENT, "q_prime and q_log_scale must be non-null");
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
  if ((e = f32_query_features(*p, ws, base, q_prime, q_log_scale, st)) != cudaSuccess)
    return cuda_fail(e, "query features");
  return SBL_OK;
}

int sbl_key_features(const SblParams* p, void* workspace, size_t workspace_bytes, float* k_prime,
                     float* k_log_scale, void* cuda_stream) {
  Workspace ws;
  int rc = prepare(p, workspace, workspace_bytes, &ws);
  if (rc != SBL_OK) return rc;
  if (!k_prime || !k_log_scale) return fail(SBL_ERR_INVALID_ARGUMENT, "k_prime and k_log_scale must be non-null");
  char* base = static_cast<char*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e;
  if ((e = f32_prepare_projection(*p, ws, base, st)) != cudaSuccess) return cuda_fail(e, "prepare projection");
  if ((e = f32_key_logscale(*p, ws, base, k_log_scale, st)) != cudaSuccess) return cuda_fail(e, "key logscale");
  if ((e = f32_key_features(*p, ws, base, k_log_scale, k_prime, st)) != cudaSuccess)
    return cuda_fail(e, "key features");
  return SBL_OK;
}

}  // extern "C"
