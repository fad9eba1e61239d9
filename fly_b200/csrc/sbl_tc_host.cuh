// Host-side helpers shared by the tensor-core kernel files: the tensor-map
// cache, per-device facts, the tensor path's view of the workspace, and the
// entry points of the head-dim-128 kernels (sbl_tc128.cu) that sbl_tc.cu's
// public functions forward to.
#pragma once

#include <mutex>

#include "sbl_common.cuh"
#include "sbl_tc_ptx.cuh"

namespace sbl {
namespace tch {

bool aligned16(const void* p);

// Encoded tensor maps are cached by what they describe (base, dims, strides, box).
bool cached_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                 const uint32_t* box);
// (B, rows, H, E) bf16 tensor with element strides sb, ss, sh; box = 64 columns x box_rows rows.
bool map_bthe(CUtensorMap* m, const void* base, int B, int rows, int H, int E, int64_t sb, int64_t ss, int64_t sh,
              uint32_t box_rows);

// Per-device facts that do not change: SM count, and that a kernel's shared-memory limit has been raised.
struct DeviceInfo {
  int sms = 0;
  bool attr_keys[2] = {false, false};
  bool attr_band = false;
  bool attr_keys128 = false;
  bool attr_band128 = false;
};
cudaError_t device_info(DeviceInfo** out);

struct TcLayout {
  float* wmax;
  __nv_bfloat16* wt16;
  float* wt32;
  __nv_bfloat16* phik;
  __nv_bfloat16* kv16;
  float* partial;
  int* status;
};
TcLayout tc_layout(const Workspace& ws, char* base);

}  // namespace tch

// ---- head dim 128 (E = D = 128, r = 256), sbl_tc128.cu ----
bool tc128_shape(const SblParams& p);
cudaError_t tc128_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* beta, float* kv,
                              float* ksum, cudaStream_t st, bool also_bf16);
cudaError_t tc128_band(const SblParams& p, const Workspace& ws, char* base, const float* beta, const float* kv,
                       const float* ksum, cudaStream_t st, bool kv16_ready);

}  // namespace sbl
