// Shared declarations of the sblocal_b200 library: the internal view of a
// problem, the workspace layout, and the launch functions each kernel file
// exports to the C-ABI layer (sbl_api.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sblocal_b200.h"

namespace sbl {

// Workspace sections (byte offsets from the 256-byte aligned base).  The
// generic path keeps phi(Q) and phi(K) in fp32; the tensor path keeps phi(K)
// in bf16 and never materialises phi(Q).
struct Workspace {
  size_t wt;        // scaled projection sqrt(tau)*W: fp32 (r,E) [generic] / bf16 (r,E) [tensor]
  size_t phik;      // (B,H,S,m)
  size_t phiq;      // generic: phi(Q) (B,H,T,m) fp32; tensor: scaled projection in bf16 (r,E)
  size_t qls;       // generic: query log-scales (B,H,T) fp32; tensor: KV in bf16 (B,H,m,D)
  size_t beta;      // (B,H) fp32
  size_t kv;        // (B,H,m,D) fp32
  size_t ksum;      // (B,H,m) fp32
  size_t partial;   // split-S partial summaries
  size_t lognorm;   // generic: log_normalization per query row (B,H,T) fp32; tensor: sum phi(K) in the kernels' feature order (B,H,m)
  size_t status;    // int32[4] device status words, then small scalars
  size_t total;
  int nsplit;       // number of S splits of the summary GEMM
  int split_rows;   // key rows per split
  bool tensor;      // true: tcgen05/TMA bf16 kernels are used
};

// Fills the layout for a problem.
void plan_workspace(const SblParams& p, Workspace* ws);

inline __host__ __device__ int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- generic SIMT path (any E, D, r, w; fp32 or bf16 storage, fp32 math) ----
cudaError_t f32_prepare_projection(const SblParams& p, const Workspace& ws, char* base, cudaStream_t st);
cudaError_t f32_key_logscale(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st);
cudaError_t f32_key_features(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                             float* phik_out, cudaStream_t st);
cudaError_t f32_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* phik,
                            float* kv, float* ksum, cudaStream_t st);
cudaError_t f32_combine_partials(const SblParams& p, const Workspace& ws, char* base, float* kv, float* ksum,
                                 cudaStream_t st);
cudaError_t f32_query_features(const SblParams& p, const Workspace& ws, char* base, float* phiq_out,
                               float* qls_out, cudaStream_t st);
cudaError_t f32_band(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                     const float* kv, const float* ksum, cudaStream_t st);

cudaError_t f32_attention_weights(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                                  float* attn, float* attn_un, float* attn_lr, cudaStream_t st);

// ---- tensor-core path (bf16 storage, tcgen05 + TMA), sbl_tc.cu ----
bool tc_supported(const SblParams& p);
// reset_status: clear the device status words (first stage of a call sequence)
// beta_fill: when given, the B*H key log-scales there are reset to -inf by the same launch
cudaError_t tc_prepare_projection(const SblParams& p, const Workspace& ws, char* base, cudaStream_t st,
                                  bool reset_status, float* beta_fill = nullptr);
cudaError_t tc_key_logscale(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st);
// one-pass upper bound on the key log-scale (valid stabiliser when eps = 0); used by the fused forward
cudaError_t tc_key_logscale_bound(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st,
                                  bool beta_is_reset = false);
// also_bf16: also leave KV in bf16 in the workspace, where a tc_band call with kv16_ready picks it up
cudaError_t tc_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                           float* kv, float* ksum, cudaStream_t st, bool also_bf16 = false);
cudaError_t tc_band(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                    const float* kv, const float* ksum, cudaStream_t st, bool kv16_ready = false);
// runs a kernel whose only wait can never be satisfied; *host_status receives the recorded wait site (99)
cudaError_t tc_wait_selftest(int* device_status, int* host_status, cudaStream_t st);
// copies the three device status words (host_status[0]: wait site that ran out, host_status[1]: 1 if an
// exponential left the fp32 range, host_status[2]: 1 if a row's low-rank estimate swamped its exact part) and
// synchronises the stream
cudaError_t tc_read_status(const Workspace& ws, char* base, int* host_status, cudaStream_t st);

}  // namespace sbl
