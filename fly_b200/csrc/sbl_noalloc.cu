// sbl_key_logscale_static: the key log-scale stage for callers that must not
// allocate device memory.
//
// Who needs this: hosts that hand the GPU's memory to one arena at start-up
// and never call cudaMalloc again (inference servers with a fixed memory plan,
// plugins loaded into a process whose allocator already owns every byte),
// and latency-critical loops in which cudaMalloc/cudaFree are banned because
// they synchronise the whole device.  Such a caller cannot provide the
// workspace the regular entry points ask for, so this variant keeps its
// scratch -- the projection scaled by sqrt(tau), r*E floats -- in a fixed
// array that is part of the library image itself.
//
// Consequences the caller has to know about:
//   * the array has a fixed capacity: r*E <= SBL_STATIC_PROJ_FLOATS (32768
//     floats, 128 KiB); larger problems are rejected with
//     SBL_ERR_UNSUPPORTED.  Every GPU that loads the library carries those
//     128 KiB until the process exits.
//   * the array is shared by all calls on a device and keeps what the last
//     call left in it.  Each call rewrites the r*E floats it reads before
//     reading them, so nothing has to be cleared, but two calls that overlap
//     on the GPU (different streams) race on it: serialise them.
//   * the first call on each device looks up the array's device address.
//     That lookup is a CUDA runtime call, so make this first call during
//     start-up, ahead of any stream capture.  The first launch of a kernel
//     in a process may also load its code: make one start-up call per input
//     dtype you will use (fp32 and bf16 keys run different instantiations).
//     The address is remembered per device for the life of the process; a
//     cudaDeviceReset invalidates it, so do not reset a device and go on
//     using this entry point.
//   * the value is the exact key log-scale computed with the fp32 projection
//     by the generic kernels: equal to sbl_key_logscale with
//     SBL_FLAG_GENERIC_PATH.  For bf16 inputs of the tensor-core shape
//     (E = 64, r = 128) the plain sbl_key_logscale rounds the projection to
//     bf16 first, so the two differ there by up to a few 1e-2 (either is a
//     valid stabiliser).
//   * neither this function nor anything it calls allocates or frees memory.
#include <cstdio>
#include <mutex>

#include "sbl_common.cuh"

namespace {

constexpr int kStaticProjFloats = 32768;
constexpr int kMaxDevices = 64;

// Scratch lives in the module's global segment.  In host code this name is
// only a handle for the runtime; the device address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_projection[kStaticProjFloats];

std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {};
thread_local char g_msg[256] = "";

// Device address of the array on the current device, resolved once per device.
cudaError_t scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_projection);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

int reject(int code, const char* msg) {
  snprintf(g_msg, sizeof(g_msg), "%s", msg);
  return code;
}

}  // namespace

extern "C" {

const char* sbl_static_last_error(void) { return g_msg; }

int sbl_key_logscale_static(const SblParams* p, float* beta, void* cuda_stream) {
  if (!p || !beta) return reject(SBL_ERR_INVALID_ARGUMENT, "params and beta must be non-null");
  if (p->dtype != SBL_DTYPE_F32 && p->dtype != SBL_DTYPE_BF16)
    return reject(SBL_ERR_INVALID_ARGUMENT, "dtype must be SBL_DTYPE_F32 or SBL_DTYPE_BF16");
  if (p->B <= 0 || p->H <= 0 || p->S <= 0 || p->E <= 0 || p->r <= 0)
    return reject(SBL_ERR_INVALID_ARGUMENT, "B, H, S, E and r must be positive");
  if ((int64_t)p->B * p->H > 65535) return reject(SBL_ERR_UNSUPPORTED, "B*H exceeds the grid limit 65535");
  if (!(p->softmax_temp > 0.f)) return reject(SBL_ERR_INVALID_ARGUMENT, "softmax_temp must be > 0");
  if (!p->k || !p->W) return reject(SBL_ERR_INVALID_ARGUMENT, "k and W must be non-null device pointers");
  if (p->sum_lo < 0 || p->sum_hi > p->S || p->sum_lo > p->sum_hi)
    return reject(SBL_ERR_INVALID_ARGUMENT, "summary rows must lie inside the key buffer");
  if (p->k_stride_b < 0 || p->k_stride_s < p->E || p->k_stride_h < 0)
    return reject(SBL_ERR_INVALID_ARGUMENT, "key strides must be non-negative element strides, rows at least E apart");
  for (int i = 0; i < 3; ++i)
    if (p->reserved[i] != 0) return reject(SBL_ERR_INVALID_ARGUMENT, "reserved fields must be 0");
  if (p->flags & ~SBL_FLAG_GENERIC_PATH) return reject(SBL_ERR_INVALID_ARGUMENT, "unknown flag bits");
  if ((int64_t)p->r * p->E > kStaticProjFloats) {
    snprintf(g_msg, sizeof(g_msg),
             "r*E = %lld floats exceeds the built-in scratch of %d floats; use sbl_key_logscale with a workspace",
             (long long)p->r * p->E, kStaticProjFloats);
    return SBL_ERR_UNSUPPORTED;
  }
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    snprintf(g_msg, sizeof(g_msg), "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    return SBL_ERR_CUDA;
  }
  sbl::Workspace ws{};  // every section at offset 0: only the projection is used
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  char* base = reinterpret_cast<char*>(scratch);
  if ((e = sbl::f32_prepare_projection(*p, ws, base, st)) != cudaSuccess ||
      (e = sbl::f32_key_logscale(*p, ws, base, beta, st)) != cudaSuccess) {
    snprintf(g_msg, sizeof(g_msg), "kernel launch: %s", cudaGetErrorString(e));
    return SBL_ERR_CUDA;
  }
  return SBL_OK;
}

}  // extern "C"
