// Microbenchmark: cost per tcgen05.mma (M = 128, K = 16, bf16, fp32 accumulate) by N, by where A comes from (shared
// memory "SS" / tensor memory "TS"), by the number of warps issuing at the same time, and with or without sixteen
// busy warps (exponentials and FMAs) beside the issuers.  One CTA per SM; every issuer sends 512 MMAs back to back
// and reads the clock when the last has been issued and when its commit has arrived.  Operands are zeros.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I fly_b200/csrc -I include \
//        -o mma_cost fly_b200/microbench/mma_cost.cu && ./mma_cost
#include <cstdio>
#include <cstdlib>
#include "sbl_tc_ptx.cuh"
using namespace sbl; using namespace sbl::ptx;
__device__ __forceinline__ float ex2f_(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__global__ void __launch_bounds__(640) bench(long long* out, uint32_t idesc, int form, int R, int noise, int nissuers, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  __shared__ volatile int stop;
  const int tid = threadIdx.x, warp = tid / 32;
  for (int i = tid; i < 49152 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (tid == 0) { for (int i = 0; i < 4; ++i) mbar_init(bar + i, 1); fence_mbar_init(); stop = 0; }
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint64_t dA = smem_desc_sw128(smem_u32(smem), 16, 1024);
  const uint64_t dB = smem_desc_sw128(smem_u32(smem + 16384), 16, 1024);
  if (warp < nissuers) {
    if (elect_one()) {
      const uint32_t td = warp * 128;       // each issuer its own accumulator (N <= 128 when nissuers > 1)
      const long long t0 = clock64();
      for (int i = 0; i < R; i += 8) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (form == 0) mma_ss(td, dA + 2 * (k & 3), dB + 2 * (k & 3), idesc, true);
          else mma_ts(td, 384 + 8 * k, dB + 2 * (k & 3), idesc, true);
        }
      }
      const long long t1 = clock64();
      mma_commit(bar + warp);
      mbar_wait(bar + warp, 0, status, 1);
      const long long t2 = clock64();
      if (warp == 0) { out[2 * blockIdx.x] = t1 - t0; out[2 * blockIdx.x + 1] = t2 - t0; }
    }
    __syncwarp();
    if (warp == 0) { __threadfence_block(); if (tid == 0) stop = 1; }
  } else if (warp >= 4 && noise) {
    float x = tid * 1e-3f, acc = 0.f;
    while (!stop) {
#pragma unroll
      for (int k = 0; k < 32; ++k) { acc = fmaf(acc, 0.999f, ex2f_(x)); x += 1e-4f; }
    }
    if (acc == 12345.f) out[0] = 0;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(0, 512);
}

int main() {
  long long* out; cudaMalloc(&out, 148 * 16);
  int* status; cudaMalloc(&status, 16); cudaMemset(status, 0, 16);
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 49152 + 1024 + 32768);
  long long h[2];
  const int R = 512;
  for (int noise = 0; noise < 2; ++noise)
    for (int nis = 1; nis <= 3; nis += 1)
      for (int form = 0; form < 2; ++form)
        for (int N : {64, 128, 256}) {
          if (nis > 1 && N > 128) continue;
          const uint32_t id = idesc_bf16(128, N, false, false);
          for (int rep = 0; rep < 2; ++rep) bench<<<148, 640, 49152 + 1024 + 32768>>>(out, id, form, R, noise, nis, status);
          cudaError_t e = cudaDeviceSynchronize();
          cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
          int st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
          printf("noise %d issuers %d form %s N %3d: issue %.1f cyc/mma, complete %.1f cyc/mma (per issuer)  %s st %d\n", noise, nis, form ? "TS" : "SS", N,
                 (double)h[0] / R, (double)h[1] / R, cudaGetErrorString(e), st);
        }
  return 0;
}
