// Microbenchmark: per-SM delivery rate of 32 KB pieces into a shared-memory ring, by tensor-map boxes
// ({64,128} bf16 = 128-byte rows out of 1024-byte-pitch rows) or by contiguous bulk copies.  One thread issues the
// loads, a second one releases every slot as soon as it has landed; the figure is cycles per piece seen by the
// releasing thread, averaged over the CTAs.  It is the ceiling for the operand rings of the band kernels.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I fly_b200/csrc -I include \
//        -o tma_ring fly_b200/microbench/tma_ring.cu fly_b200/csrc/sbl_tmap.cu && ./tma_ring [rows of the source]
#include <cstdio>
#include <cstdlib>
#include "sbl_tc_ptx.cuh"
using namespace sbl; using namespace sbl::ptx;

__device__ __forceinline__ void bulk_load(void* smem, const void* g, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(smem_u32(smem)), "l"(g), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(64) bench(const __grid_constant__ CUtensorMap tm, const uint8_t* flat, long long* out,
                                            int ns, int npieces, int mode, int S, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[8], empty[8];
  const int tid = threadIdx.x;
  if (tid == 0) { for (int i = 0; i < 8; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); } fence_mbar_init(); }
  __syncthreads();
  const int ntile = S / 128;
  if (tid == 0) {
    for (int n = 0; n < npieces; ++n) {
      const int s = n % ns, u = n / ns;
      if (u >= 1) mbar_wait(empty + s, (u - 1) & 1, status, 1);
      const long long g = (long long)blockIdx.x * npieces + n;     // global piece number
      uint8_t* dst = smem + s * 32768;
      mbar_expect_tx(full + s, 32768);
      if (mode == 0) {
        const int tile = (int)((g / 4) % ntile), j = (int)(g % 4);
        tma_load_3d(dst, &tm, full + s, 128 * j, tile * 128, 0);
        tma_load_3d(dst + 16384, &tm, full + s, 128 * j + 64, tile * 128, 0);
      } else {
        const uint8_t* src = flat + (g * 32768) % ((long long)S * 1024);
        if (mode == 1) { bulk_load(dst, src, 16384, full + s); bulk_load(dst + 16384, src + 16384, 16384, full + s); }
        else bulk_load(dst, src, 32768, full + s);
      }
    }
  } else if (tid == 32) {
    long long t0 = clock64();
    for (int n = 0; n < npieces; ++n) {
      const int s = n % ns, u = n / ns;
      mbar_wait(full + s, u & 1, status, 2);
      mbar_arrive(empty + s);
    }
    long long t1 = clock64();
    out[blockIdx.x] = (t1 - t0) / npieces;
  }
}

int main(int argc, char** argv) {
  const int S = argc > 1 ? atoi(argv[1]) : 65536;       // rows of the (S, 512) bf16 tensor: S * 1 KB
  uint8_t* buf; cudaMalloc(&buf, (size_t)S * 1024); cudaMemset(buf, 0, (size_t)S * 1024);
  long long* out; cudaMalloc(&out, 148 * 8);
  int* status; cudaMalloc(&status, 16); cudaMemset(status, 0, 16);
  CUtensorMap tm;
  const uint64_t dims[3] = {512, (uint64_t)S, 1}; const uint64_t str[2] = {1024, (uint64_t)S * 1024}; const uint32_t box[3] = {64, 128, 1};
  if (!encode_tmap_bf16(&tm, buf, 3, dims, str, box)) { printf("tmap failed\n"); return 1; }
  cudaFuncSetAttribute(bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * 32768 + 1024);
  long long h[148];
  for (int grid : {1, 148}) for (int mode = 0; mode < 3; ++mode) for (int ns : {2, 4, 6}) {
    for (int rep = 0; rep < 2; ++rep) bench<<<grid, 64, ns * 32768 + 1024>>>(tm, buf, out, ns, 400, mode, S, status);
    cudaError_t e = cudaGetLastError(); cudaDeviceSynchronize();
    cudaMemcpy(h, out, grid * 8, cudaMemcpyDeviceToHost);
    double m = 0; for (int i = 0; i < grid; ++i) m += h[i]; m /= grid;
    int st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    printf("grid %3d mode %d (%s) slots %d: %.0f cycles per 32 KB piece = %.1f B/clk  [%s status %d]\n", grid, mode,
           mode == 0 ? "tensor boxes" : mode == 1 ? "bulk 2x16K" : "bulk 32K", ns, m, 32768.0 / m, cudaGetErrorString(e), st);
  }
  return 0;
}
