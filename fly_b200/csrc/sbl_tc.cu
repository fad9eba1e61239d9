// bf16 tensor-core path of the SBLocal forward for sm_100a: TMA tile loads,
// tcgen05.mma with accumulators (and the phi(Q) / weight operands) in tensor
// memory, warp-specialised pipelines with mbarriers whose waits are bounded.
// Shapes: E = D = 64, r = 128 (m = 256), eps = 0, any T, S, w, key lengths.
// Everything else takes the generic kernels of sbl_f32.cu.
//
// Kernels
//   prep      sqrt(tau)*W -> bf16 (and fp32), clears the status words
//   keys<MAX> per (split, b*h): streams 128-key tiles; U = K Wt^T on tensor
//             cores; MAX: running max of (|u| - tau|k|^2/2) -> beta (atomic);
//             else phi(K) -> bf16 to the workspace and, MN-major, to shared
//             memory for KV += phi(K)^T [V | 1] (accumulators in tensor memory),
//             then one partial summary per CTA
//   combine   (sbl_f32.cu) sums the split partials -> KV, sum phi(K)
//   band      per (128-query tile, b*h): U = Q Wt^T -> phi(Q) packed bf16 into
//             tensor memory (the A operand of every phi(Q) product); then per
//             64-key tile S = Q K^T, P = phi(Q) phi(K)^T (double-buffered in
//             tensor memory), the softmax warps form
//             D = exp(tau S - c) - P e^{pls-c} (masked to the window and key
//             length) as packed bf16 in tensor memory, O += D V; finally
//             LR = phi(Q) KV and out = (O + e^{pls-c} LR) /
//             (L + max(Z - dps, 1e-24) e^{pls-c}), written as 128-byte rows.
//   The row stabiliser c is the Cauchy-Schwarz bound tau |q| max|k| over the
//   keys the CTA visits, so no accumulator is ever rescaled.
#include "sbl_common.cuh"
#include "sbl_tc_ptx.cuh"

namespace sbl {
namespace {

using namespace ptx;

constexpr int kE = 64;    // head dim (qk and v)
constexpr int kR = 128;   // projection rows
constexpr int kM = 256;   // features
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// sum of squares of one 64-element bf16 row held in a 128-byte swizzled line
__device__ __forceinline__ float row_sumsq_sw128(const uint8_t* tile, int row) {
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(tile + row * 128 + ((c ^ (row & 7)) << 4));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = bf16_lo(w[j]), b = bf16_hi(w[j]);
      s = fmaf(a, a, s);
      s = fmaf(b, b, s);
    }
  }
  return s;
}

// ---------------------------------------------------------------------------
__global__ void tc_prep_kernel(const float* W, float c, float* wt32, __nv_bfloat16* wt16, int n, int* status,
                               int reset_status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float v = c * W[i];
    wt32[i] = v;
    wt16[i] = __float2bfloat16_rn(v);
  }
  if (reset_status && i < 4) status[i] = 0;
}

__global__ void tc_kv_to_bf16_kernel(const float* kv, __nv_bfloat16* kv16, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) kv16[i] = __float2bfloat16_rn(kv[i]);
}

// ---------------------------------------------------------------------------
// keys kernel
struct KeysArgs {
  CUtensorMap tm_k, tm_v, tm_w;
  const int64_t* lengths;
  const float* beta_in;   // !MAX
  float* beta_out;        // MAX
  __nv_bfloat16* phik;    // (BH, S, 256)
  float* partial;         // (BH, nsplit, 256, 65)
  int* status;
  int S, H, sum_lo, sum_hi, nsplit;
  int64_t k_pos0, S_total;
  float tau, half_log_m;
};

namespace keys {
constexpr int TILE = 128;
constexpr uint32_t OFF_W = 0;                    // 16 KB  [128 r][64 e]
constexpr uint32_t OFF_ONES = 16384;             // 4 KB   [128 keys][16] (32-byte swizzle)
constexpr uint32_t OFF_STAGE = 24576;            // 2 x { K 16 KB, V 16 KB }
constexpr uint32_t STAGE_BYTES = 32768;
constexpr uint32_t OFF_A = OFF_STAGE + 2 * STAGE_BYTES;  // 64 KB: 4 blocks [128 keys][64 f]
constexpr uint32_t OFF_BAR = OFF_A + 65536;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 + 1024;    // + alignment slack
// tensor memory columns
constexpr uint32_t T_UK = 0;      // 2 x 128
constexpr uint32_t T_KV = 256;    // 2 x 64
constexpr uint32_t T_KS = 384;    // 2 x 16
}  // namespace keys

template <bool MAX_ONLY>
__global__ void __launch_bounds__(192) tc_keys_kernel(const __grid_constant__ KeysArgs a) {
  using namespace keys;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* bar_w = bars + 0;
  uint64_t* bar_done = bars + 1;
  uint64_t* full = bars + 2;      // [2]
  uint64_t* empty = bars + 4;     // [2]
  uint64_t* uk_full = bars + 6;   // [2]
  uint64_t* uk_free = bars + 8;   // [2]
  uint64_t* a_full = bars + 10;
  uint64_t* a_free = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  float* red = reinterpret_cast<float*>(bars + 13);  // [4]

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int ntiles = (a.S + TILE - 1) / TILE;
  const int split = blockIdx.x;
  const int t_lo = (int)((int64_t)ntiles * split / a.nsplit);
  const int t_hi = (int)((int64_t)ntiles * (split + 1) / a.nsplit);
  const int nt = t_hi - t_lo;

  if (tid == 0) {
    mbar_init(bar_w, 1);
    mbar_init(bar_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, 1);
      mbar_init(uk_full + i, 1);
      mbar_init(uk_free + i, 128);
    }
    mbar_init(a_full, 128);
    mbar_init(a_free, 1);
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (!MAX_ONLY)
    for (int i = tid; i < 128 * 16; i += 192)
      reinterpret_cast<__nv_bfloat16*>(smem + OFF_ONES)[i] = __float2bfloat16(1.0f);
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *tmem_slot;

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      prefetch_tmap(&a.tm_k);
      prefetch_tmap(&a.tm_v);
      prefetch_tmap(&a.tm_w);
      mbar_expect_tx(bar_w, 16384);
      tma_load_2d(smem + OFF_W, &a.tm_w, bar_w, 0, 0);
      for (int i = 0; i < nt; ++i) {
        const int s = i & 1;
        if (i >= 2) mbar_wait(empty + s, ((i >> 1) - 1) & 1, a.status, 11);
        uint8_t* st = smem + OFF_STAGE + s * STAGE_BYTES;
        const int row0 = (t_lo + i) * TILE;
        mbar_expect_tx(full + s, MAX_ONLY ? 16384 : 32768);
        tma_load_4d(st, &a.tm_k, full + s, 0, row0, h, b);
        if (!MAX_ONLY) tma_load_4d(st + 16384, &a.tm_v, full + s, 0, row0, h, b);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t id_uk = idesc_bf16(128, 128, false, false);
      const uint32_t id_kv = idesc_bf16(128, 64, true, true);
      const uint32_t id_ks = idesc_bf16(128, 16, true, true);
      const uint32_t sW = smem_u32(smem + OFF_W), sA = smem_u32(smem + OFF_A), sOnes = smem_u32(smem + OFF_ONES);
      auto issue_kv = [&](int u) {
        mbar_wait(a_full, u & 1, a.status, 12);
        tc_fence_after_sync();
        const uint32_t sV = smem_u32(smem + OFF_STAGE + (u & 1) * STAGE_BYTES + 16384);
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t da = smem_desc_sw128(sA + mb * 32768 + k * 2048, 16384, 1024);
            mma_ss(tb + T_KV + mb * 64, da, smem_desc_sw128(sV + k * 2048, 16, 1024), id_kv, (u > 0) || (k > 0));
            mma_ss(tb + T_KS + mb * 16, da, smem_desc_sw32(sOnes + k * 512, 16, 256), id_ks, (u > 0) || (k > 0));
          }
        mma_commit(a_free);
        mma_commit(empty + (u & 1));
      };
      mbar_wait(bar_w, 0, a.status, 13);
      for (int i = 0; i < nt; ++i) {
        const int s = i & 1;
        mbar_wait(full + s, (i >> 1) & 1, a.status, 14);
        if (i >= 2) mbar_wait(uk_free + s, ((i >> 1) - 1) & 1, a.status, 15);
        tc_fence_after_sync();
        const uint32_t sK = smem_u32(smem + OFF_STAGE + s * STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss(tb + T_UK + s * 128, smem_desc_sw128(sK + k * 32, 16, 1024), smem_desc_sw128(sW + k * 32, 16, 1024),
                 id_uk, k > 0);
        mma_commit(uk_full + s);
        if (MAX_ONLY) {
          // the K stage is free once U is computed and the row norms were read (uk_free)
        } else if (i >= 1) {
          issue_kv(i - 1);
        }
      }
      if (!MAX_ONLY && nt > 0) issue_kv(nt - 1);
      mma_commit(bar_done);
    }
  } else {
    // ---------------- feature warps: thread <-> key row ----------------
    const uint32_t lane_base = tb + ((uint32_t)(warp * 32) << 16);
    const int64_t len_b = a.lengths ? min(a.lengths[b], a.S_total) : a.S_total;
    const float beta = MAX_ONLY ? 0.f : a.beta_in[bh];
    float run_max = -INFINITY;
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      const int row = (t_lo + i) * TILE + tid;
      mbar_wait(full + s, (i >> 1) & 1, a.status, 19);
      mbar_wait(uk_full + s, (i >> 1) & 1, a.status, 16);
      tc_fence_after_sync();
      const uint8_t* sK = smem + OFF_STAGE + s * STAGE_BYTES;
      const float g = 0.5f * a.tau * row_sumsq_sw128(sK, tid);
      if (MAX_ONLY) {
        float mx = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_base + T_UK + s * 128 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, fabsf(__uint_as_float(r[j])));
        }
        if (row >= a.sum_lo && row < a.sum_hi) run_max = fmaxf(run_max, (mx - g) - a.half_log_m);
        tc_fence_before_sync();
        mbar_arrive(uk_free + s);
        // MAX mode has no KV MMA to release the stage: the last reader does
        if (i + 2 < nt) {
          // all 128 rows must have read their K row before the stage is refilled
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (tid == 0) mbar_arrive(empty + s);
        }
      } else {
        if (i >= 1) mbar_wait(a_free, (i - 1) & 1, a.status, 17);
        const bool live = row < a.S && (a.k_pos0 + row) < len_b;
        const bool in_sum = live && row >= a.sum_lo && row < a.sum_hi;
        const float off = ((-g - a.half_log_m) - beta) * kLog2e;
        __nv_bfloat16* grow = a.phik + ((int64_t)bh * a.S + row) * kM;
        uint8_t* sA = smem + OFF_A;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_base + T_UK + s * 128 + c * 32, r);
          tmem_ld_wait();
          uint32_t p1[16], p2[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float u0 = __uint_as_float(r[2 * j]) * kLog2e, u1 = __uint_as_float(r[2 * j + 1]) * kLog2e;
            p1[j] = live ? pack_bf16(ex2(u0 + off), ex2(u1 + off)) : 0u;
            p2[j] = live ? pack_bf16(ex2(off - u0), ex2(off - u1)) : 0u;
          }
          if (row < a.S) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              reinterpret_cast<uint4*>(grow + 32 * c)[q] = make_uint4(p1[4 * q], p1[4 * q + 1], p1[4 * q + 2], p1[4 * q + 3]);
              reinterpret_cast<uint4*>(grow + kR + 32 * c)[q] =
                  make_uint4(p2[4 * q], p2[4 * q + 1], p2[4 * q + 2], p2[4 * q + 3]);
            }
          }
          // MN-major A operand: block = feature / 64, 16-byte chunk = (feature % 64) / 8, swizzled by key % 8
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int chunk = (c & 1) * 4 + q;
            const uint32_t o = (uint32_t)tid * 128u + (uint32_t)((chunk ^ (tid & 7)) << 4);
            const uint4 z = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(sA + (c >> 1) * 16384 + o) =
                in_sum ? make_uint4(p1[4 * q], p1[4 * q + 1], p1[4 * q + 2], p1[4 * q + 3]) : z;
            *reinterpret_cast<uint4*>(sA + (2 + (c >> 1)) * 16384 + o) =
                in_sum ? make_uint4(p2[4 * q], p2[4 * q + 1], p2[4 * q + 2], p2[4 * q + 3]) : z;
          }
        }
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(a_full);
        mbar_arrive(uk_free + s);
      }
    }
    if (MAX_ONLY) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) run_max = fmaxf(run_max, __shfl_xor_sync(0xffffffffu, run_max, o));
      if (lane == 0) red[warp] = run_max;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (tid == 0) {
        const float v = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        if (v > -INFINITY) atomic_max_float(a.beta_out + bh, v);
      }
    } else {
      mbar_wait(bar_done, 0, a.status, 18);
      tc_fence_after_sync();
      float* part = a.partial + ((int64_t)bh * a.nsplit + split) * kM * 65;
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        float* prow = part + (int64_t)(mb * 128 + tid) * 65;
        if (nt > 0) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_base + T_KV + mb * 64 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) prow[c * 32 + j] = __uint_as_float(r[j]);
          }
          uint32_t q[16];
          tmem_ld16(lane_base + T_KS + mb * 16, q);
          tmem_ld_wait();
          prow[64] = __uint_as_float(q[0]);
        } else {
          for (int j = 0; j < 65; ++j) prow[j] = 0.f;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------
// band kernel
struct BandArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_w, tm_phik, tm_kv;
  SblParams p;
  const float* beta;
  const float* ksum;
  int* status;
};

namespace band {
constexpr int BQ = 128, KT = 64, NS = 3;
constexpr uint32_t OFF_Q = 0;          // 16 KB [128 q][64 e]
constexpr uint32_t OFF_W = 16384;      // 16 KB [128 r][64 e]
constexpr uint32_t OFF_KV = 32768;     // 32 KB [256 f][64 d]
constexpr uint32_t OFF_STAGE = 65536;  // NS x { K 8 KB, V 8 KB, phi(K) 4 x 8 KB }
constexpr uint32_t STAGE_BYTES = 49152;
constexpr uint32_t OFF_KSUM = OFF_STAGE + NS * STAGE_BYTES;  // 1 KB fp32[256]
constexpr uint32_t OFF_BAR = OFF_KSUM + 1024;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256 + 1024;
// tensor memory columns
constexpr uint32_t T_PHIQ = 0;     // 128: phi(Q) packed bf16 (256 features)
constexpr uint32_t T_SP = 128;     // 2 x { S 64, P 64 }
constexpr uint32_t T_O = 384;      // 64
constexpr uint32_t T_D = 448;      // 2 x 32: D packed bf16 (64 keys)
constexpr uint32_t T_UQ = 128;     // 128, aliases S/P before the band loop
constexpr uint32_t T_LR = 128;     // 64, aliases S[0] after the band loop
}  // namespace band

__global__ void __launch_bounds__(192) tc_band_kernel(const __grid_constant__ BandArgs a) {
  using namespace band;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* bar_qw = bars + 0;
  uint64_t* bar_kv = bars + 1;
  uint64_t* bar_uq = bars + 2;
  uint64_t* bar_phiq = bars + 3;
  uint64_t* bar_lr = bars + 4;
  uint64_t* full = bars + 5;       // [NS]
  uint64_t* empty = bars + 8;      // [NS]
  uint64_t* sp_full = bars + 11;   // [2]
  uint64_t* sp_free = bars + 13;   // [2]
  uint64_t* d_full = bars + 15;    // [2]
  uint64_t* d_free = bars + 17;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  float* red = reinterpret_cast<float*>(bars + 20);  // [4]
  float* s_ksum = reinterpret_cast<float*>(smem + OFF_KSUM);

  const SblParams& p = a.p;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int i0 = blockIdx.x * BQ;
  const int hw = p.w / 2;
  int len_b = (int)(p.key_lengths ? min(p.key_lengths[b], p.S_total) : p.S_total);
  // key buffer rows any query of this tile can see, clipped to the buffer and to the key length
  const int nq = min(BQ, p.T - i0);
  int lo = (int)(p.q_pos0 + i0 - hw - p.k_pos0);
  int hi = (int)(p.q_pos0 + i0 + nq - 1 - hw + p.w - 1 - p.k_pos0);
  lo = max(lo, 0);
  hi = min(hi, min(p.S - 1, len_b - 1 - (int)p.k_pos0));
  const int j0 = (lo / KT) * KT;
  const int nt = hi >= lo ? (hi - j0) / KT + 1 : 0;

  if (tid == 0) {
    mbar_init(bar_qw, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_uq, 1);
    mbar_init(bar_phiq, 128);
    mbar_init(bar_lr, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(full + i, 1);
      mbar_init(empty + i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(sp_full + i, 1);
      mbar_init(sp_free + i, 128);
      mbar_init(d_full + i, 128);
      mbar_init(d_free + i, 1);
    }
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  for (int i = tid; i < kM; i += 192) s_ksum[i] = a.ksum[(int64_t)bh * kM + i];
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *tmem_slot;

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      prefetch_tmap(&a.tm_q);
      prefetch_tmap(&a.tm_k);
      prefetch_tmap(&a.tm_v);
      prefetch_tmap(&a.tm_w);
      prefetch_tmap(&a.tm_phik);
      prefetch_tmap(&a.tm_kv);
      mbar_expect_tx(bar_qw, 32768);
      tma_load_4d(smem + OFF_Q, &a.tm_q, bar_qw, 0, i0, h, b);
      tma_load_2d(smem + OFF_W, &a.tm_w, bar_qw, 0, 0);
      mbar_expect_tx(bar_kv, 32768);
      tma_load_3d(smem + OFF_KV, &a.tm_kv, bar_kv, 0, 0, bh);
      for (int t = 0; t < nt; ++t) {
        const int s = t % NS;
        if (t >= NS) mbar_wait(empty + s, ((t / NS) - 1) & 1, a.status, 21);
        uint8_t* st = smem + OFF_STAGE + s * STAGE_BYTES;
        const int row0 = j0 + t * KT;
        mbar_expect_tx(full + s, STAGE_BYTES);
        tma_load_4d(st, &a.tm_k, full + s, 0, row0, h, b);
        tma_load_4d(st + 8192, &a.tm_v, full + s, 0, row0, h, b);
#pragma unroll
        for (int j = 0; j < 4; ++j) tma_load_3d(st + 16384 + j * 8192, &a.tm_phik, full + s, j * 64, row0, bh);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t id_uq = idesc_bf16(128, 128, false, false);
      const uint32_t id_s = idesc_bf16(128, 64, false, false);
      const uint32_t id_o = idesc_bf16(128, 64, false, true);
      const uint32_t sQ = smem_u32(smem + OFF_Q), sW = smem_u32(smem + OFF_W), sKV = smem_u32(smem + OFF_KV);
      auto issue_o = [&](int u) {
        const int bu = u & 1, su = u % NS;
        mbar_wait(d_full + bu, (u >> 1) & 1, a.status, 22);
        tc_fence_after_sync();
        const uint32_t sV = smem_u32(smem + OFF_STAGE + su * STAGE_BYTES + 8192);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ts(tb + T_O, tb + T_D + bu * 32 + k * 8, smem_desc_sw128(sV + k * 2048, 16, 1024), id_o,
                 (u > 0) || (k > 0));
        mma_commit(empty + su);
        mma_commit(d_free + bu);
      };
      mbar_wait(bar_qw, 0, a.status, 23);
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_ss(tb + T_UQ, smem_desc_sw128(sQ + k * 32, 16, 1024), smem_desc_sw128(sW + k * 32, 16, 1024), id_uq,
               k > 0);
      mma_commit(bar_uq);
      mbar_wait(bar_phiq, 0, a.status, 24);
      tc_fence_after_sync();
      for (int t = 0; t < nt; ++t) {
        const int s = t % NS, bb = t & 1;
        mbar_wait(full + s, (t / NS) & 1, a.status, 25);
        if (t >= 2) mbar_wait(sp_free + bb, ((t >> 1) - 1) & 1, a.status, 26);
        tc_fence_after_sync();
        const uint32_t sK = smem_u32(smem + OFF_STAGE + s * STAGE_BYTES);
        const uint32_t sPK = sK + 16384;
        const uint32_t tS = tb + T_SP + bb * 128, tP = tS + 64;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss(tS, smem_desc_sw128(sQ + k * 32, 16, 1024), smem_desc_sw128(sK + k * 32, 16, 1024), id_s, k > 0);
#pragma unroll
        for (int k = 0; k < 16; ++k)
          mma_ts(tP, tb + T_PHIQ + k * 8, smem_desc_sw128(sPK + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), id_s,
                 k > 0);
        mma_commit(sp_full + bb);
        if (t >= 1) issue_o(t - 1);
      }
      if (nt > 0) issue_o(nt - 1);
      // low-rank numerator LR = phi(Q) KV into the (now idle) S[0] columns
      mbar_wait(bar_kv, 0, a.status, 27);
      tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < 16; ++k)
        mma_ts(tb + T_LR, tb + T_PHIQ + k * 8, smem_desc_sw128(sKV + k * 2048, 16, 1024), id_o, k > 0);
      mma_commit(bar_lr);
    }
  } else {
    // ---------------- softmax warps: thread <-> query row ----------------
    const uint32_t lane_base = tb + ((uint32_t)(warp * 32) << 16);
    const int gi = (int)p.q_pos0 + i0 + tid;  // global query position
    // max |k|^2 over the keys this tile visits (rows of the key buffer)
    float kmax2 = 0.f;
    {
      const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(p.k) + b * p.k_stride_b + h * p.k_stride_h;
      for (int rr = tid; rr < nt * KT; rr += 128) {
        const int row = j0 + rr;
        if (row < p.S) {
          const uint4* src = reinterpret_cast<const uint4*>(kb + (int64_t)row * p.k_stride_s);
          float s = 0.f;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = __ldg(src + c);
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x = bf16_lo(wv[j]), y = bf16_hi(wv[j]);
              s = fmaf(x, x, s);
              s = fmaf(y, y, s);
            }
          }
          kmax2 = fmaxf(kmax2, s);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) kmax2 = fmaxf(kmax2, __shfl_xor_sync(0xffffffffu, kmax2, o));
      if (lane == 0) red[warp] = kmax2;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      kmax2 = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    }
    // ---- phi(Q) ----
    mbar_wait(bar_qw, 0, a.status, 32);
    mbar_wait(bar_uq, 0, a.status, 28);
    tc_fence_after_sync();
    const float qn2 = row_sumsq_sw128(smem + OFF_Q, tid);
    const float g = 0.5f * p.softmax_temp * qn2;
    float M = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(lane_base + T_UQ + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) M = fmaxf(M, fabsf(__uint_as_float(r[j])));
    }
    float Z = 0.f;
    {
      const float mo = -M * kLog2e;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(lane_base + T_UQ + c * 32, r);
        tmem_ld_wait();
        uint32_t p1[16], p2[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float u0 = __uint_as_float(r[2 * j]) * kLog2e, u1 = __uint_as_float(r[2 * j + 1]) * kLog2e;
          p1[j] = pack_bf16(ex2(u0 + mo), ex2(u1 + mo));
          p2[j] = pack_bf16(ex2(mo - u0), ex2(mo - u1));
          // Z from the rounded features, so that Z - dps cancels what the MMA sees
          Z = fmaf(bf16_lo(p1[j]), s_ksum[32 * c + 2 * j], Z);
          Z = fmaf(bf16_hi(p1[j]), s_ksum[32 * c + 2 * j + 1], Z);
          Z = fmaf(bf16_lo(p2[j]), s_ksum[kR + 32 * c + 2 * j], Z);
          Z = fmaf(bf16_hi(p2[j]), s_ksum[kR + 32 * c + 2 * j + 1], Z);
        }
        // the U columns are dead after this pass; phi(Q) lives in its own columns
        tmem_st16(lane_base + T_PHIQ + 16 * c, p1);
        tmem_st16(lane_base + T_PHIQ + 64 + 16 * c, p2);
      }
      tmem_st_wait();
    }
    tc_fence_before_sync();
    mbar_arrive(bar_phiq);

    const float half_log_m = 0.5f * logf((float)kM);
    const float pls = (-g + M - half_log_m) + a.beta[bh];
    const float cstab = p.softmax_temp * sqrtf(qn2 * kmax2);       // >= tau q.k for every visited key
    const float psc = ex2((pls - cstab) * kLog2e);                 // e^{pls - c}
    const float sc = p.softmax_temp * kLog2e, co = -cstab * kLog2e;
    float L = 0.f, dps = 0.f;
    for (int t = 0; t < nt; ++t) {
      const int bb = t & 1;
      mbar_wait(sp_full + bb, (t >> 1) & 1, a.status, 29);
      if (t >= 2) mbar_wait(d_free + bb, ((t >> 1) - 1) & 1, a.status, 30);
      tc_fence_after_sync();
      const uint32_t tS = lane_base + T_SP + bb * 128, tP = tS + 64, tD = lane_base + T_D + bb * 32;
      const int gk0 = (int)p.k_pos0 + j0 + t * KT;   // global position of column 0
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tS + c * 32, rs);
        tmem_ld32(tP + c * 32, rp);
        tmem_ld_wait();
        uint32_t dpk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int gk = gk0 + c * 32 + 2 * j + e;
            const bool ok = (unsigned)(gk - gi + hw) < (unsigned)p.w && (unsigned)gk < (unsigned)len_b;
            const float ev = ok ? ex2(fmaf(__uint_as_float(rs[2 * j + e]), sc, co)) : 0.f;
            const float pv = ok ? __uint_as_float(rp[2 * j + e]) : 0.f;
            L += ev;
            dps += pv;
            dv[e] = fmaf(-pv, psc, ev);
          }
          dpk[j] = pack_bf16(dv[0], dv[1]);
        }
        tmem_st16(tD + c * 16, dpk);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(d_full + bb);
      mbar_arrive(sp_free + bb);
    }
    // ---- epilogue ----
    mbar_wait(bar_lr, 0, a.status, 31);
    tc_fence_after_sync();
    const float inv = 1.f / (L + fmaxf(Z - dps, 1e-24f) * psc);
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + b * p.o_stride_b + h * p.o_stride_h +
                          (int64_t)(i0 + tid) * p.o_stride_t;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      // tensor-memory loads are warp-wide: every lane runs them, only the store is predicated
      uint32_t ro[32], rl[32];
      if (nt > 0) tmem_ld32(lane_base + T_O + c * 32, ro);
      tmem_ld32(lane_base + T_LR + c * 32, rl);
      tmem_ld_wait();
      uint32_t o[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float o0 = nt > 0 ? __uint_as_float(ro[2 * j]) : 0.f, o1 = nt > 0 ? __uint_as_float(ro[2 * j + 1]) : 0.f;
        o[j] = pack_bf16(fmaf(psc, __uint_as_float(rl[2 * j]), o0) * inv,
                         fmaf(psc, __uint_as_float(rl[2 * j + 1]), o1) * inv);
      }
      if (tid < nq) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          reinterpret_cast<uint4*>(orow + 32 * c)[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------
// host side
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool map_bthe(CUtensorMap* m, const void* base, int B, int rows, int H, int64_t sb, int64_t ss, int64_t sh,
              uint32_t box_rows) {
  const uint64_t dims[4] = {(uint64_t)kE, (uint64_t)rows, (uint64_t)H, (uint64_t)B};
  // a size-1 axis may carry any stride in torch; give the encoder a legal one
  const uint64_t str[3] = {(uint64_t)ss * 2, (uint64_t)(H > 1 ? sh : kE) * 2, (uint64_t)(B > 1 ? sb : kE) * 2};
  const uint32_t box[4] = {64, box_rows, 1, 1};
  return encode_tmap_bf16(m, base, 4, dims, str, box);
}

struct TcLayout {
  __nv_bfloat16* wt16;
  float* wt32;
  __nv_bfloat16* phik;
  __nv_bfloat16* kv16;
  float* partial;
  int* status;
};

TcLayout tc_layout(const SblParams& p, const Workspace& ws, char* base) {
  TcLayout l;
  l.wt32 = reinterpret_cast<float*>(base + ws.wt);
  l.wt16 = reinterpret_cast<__nv_bfloat16*>(base + ws.phiq);  // the tensor path has no phi(Q) section
  l.phik = reinterpret_cast<__nv_bfloat16*>(base + ws.phik);
  l.kv16 = reinterpret_cast<__nv_bfloat16*>(base + ws.qls);   // nor query log-scales
  l.partial = reinterpret_cast<float*>(base + ws.partial);
  l.status = reinterpret_cast<int*>(base + ws.status);
  (void)p;
  return l;
}

template <bool MAX_ONLY>
cudaError_t launch_keys(const SblParams& p, const Workspace& ws, char* base, const float* beta_in, float* beta_out,
                        cudaStream_t st) {
  const TcLayout l = tc_layout(p, ws, base);
  KeysArgs a{};
  if (!map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, p.k_stride_b, p.k_stride_s, p.k_stride_h, 128) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, p.v_stride_b, p.v_stride_s, p.v_stride_h, 128))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_tmap_bf16(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  a.lengths = p.key_lengths;
  a.beta_in = beta_in;
  a.beta_out = beta_out;
  a.phik = l.phik;
  a.partial = l.partial;
  a.status = l.status;
  a.S = p.S;
  a.H = p.H;
  a.sum_lo = p.sum_lo;
  a.sum_hi = p.sum_hi;
  a.nsplit = ws.nsplit;
  a.k_pos0 = p.k_pos0;
  a.S_total = p.S_total;
  a.tau = p.softmax_temp;
  a.half_log_m = (float)(log((double)kM) / 2.0);
  cudaError_t e = cudaFuncSetAttribute(tc_keys_kernel<MAX_ONLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)keys::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)ws.nsplit, (unsigned)(p.B * p.H));
  tc_keys_kernel<MAX_ONLY><<<grid, 192, keys::SMEM_BYTES, st>>>(a);
  return cudaGetLastError();
}

__global__ void tc_fill_kernel(float* p, float v, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

}  // namespace

bool tc_supported(const SblParams& p) {
  if (p.dtype != SBL_DTYPE_BF16 || p.E != kE || p.D != kE || p.r != kR) return false;
  if (p.softmax_eps != 0.f) return false;
  const int64_t strides[] = {p.q_stride_b, p.q_stride_t, p.q_stride_h, p.k_stride_b, p.k_stride_s, p.k_stride_h,
                             p.v_stride_b, p.v_stride_s, p.v_stride_h, p.o_stride_b, p.o_stride_t, p.o_stride_h};
  for (int64_t s : strides)
    if (s % 8 != 0 || s < 0) return false;
  if (p.q_stride_t < kE || p.k_stride_s < kE || p.v_stride_s < kE || p.o_stride_t < kE) return false;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.out)) return false;
  if (p.S_total >= (1ll << 30) || p.q_pos0 + p.T >= (1ll << 30)) return false;
  return true;
}

cudaError_t tc_prepare_projection(const SblParams& p, const Workspace& ws, char* base, cudaStream_t st,
                                  bool reset_status) {
  const TcLayout l = tc_layout(p, ws, base);
  const int n = p.r * p.E;
  tc_prep_kernel<<<(unsigned)div_up(n, 256), 256, 0, st>>>(p.W, (float)sqrt((double)p.softmax_temp), l.wt32, l.wt16, n,
                                                           l.status, reset_status ? 1 : 0);
  return cudaGetLastError();
}

cudaError_t tc_key_logscale(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st) {
  const int bh = p.B * p.H;
  tc_fill_kernel<<<(unsigned)div_up(bh, 256), 256, 0, st>>>(beta, -INFINITY, bh);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_keys<true>(p, ws, base, nullptr, beta, st);
}

cudaError_t tc_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* beta, float* kv,
                           float* ksum, cudaStream_t st) {
  cudaError_t e = launch_keys<false>(p, ws, base, beta, nullptr, st);
  if (e != cudaSuccess) return e;
  return f32_combine_partials(p, ws, base, kv, ksum, st);
}

cudaError_t tc_band(const SblParams& p, const Workspace& ws, char* base, const float* beta, const float* kv,
                    const float* ksum, cudaStream_t st) {
  const TcLayout l = tc_layout(p, ws, base);
  const int64_t nkv = (int64_t)p.B * p.H * kM * kE;
  tc_kv_to_bf16_kernel<<<(unsigned)div_up(nkv, 256), 256, 0, st>>>(kv, l.kv16, nkv);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  BandArgs a{};
  if (!map_bthe(&a.tm_q, p.q, p.B, p.T, p.H, p.q_stride_b, p.q_stride_t, p.q_stride_h, 128) ||
      !map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, p.k_stride_b, p.k_stride_s, p.k_stride_h, 64) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, p.v_stride_b, p.v_stride_s, p.v_stride_h, 64))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 128};
    if (!encode_tmap_bf16(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  {
    const uint64_t dims[3] = {(uint64_t)kM, (uint64_t)p.S, (uint64_t)(p.B * p.H)};
    const uint64_t str[2] = {(uint64_t)kM * 2, (uint64_t)p.S * kM * 2};
    const uint32_t box[3] = {64, 64, 1};
    if (!encode_tmap_bf16(&a.tm_phik, l.phik, 3, dims, str, box)) return cudaErrorInvalidValue;
  }
  {
    const uint64_t dims[3] = {(uint64_t)kE, (uint64_t)kM, (uint64_t)(p.B * p.H)};
    const uint64_t str[2] = {(uint64_t)kE * 2, (uint64_t)kM * kE * 2};
    const uint32_t box[3] = {64, 256, 1};
    if (!encode_tmap_bf16(&a.tm_kv, l.kv16, 3, dims, str, box)) return cudaErrorInvalidValue;
  }
  a.p = p;
  a.beta = beta;
  a.ksum = ksum;
  a.status = l.status;
  e = cudaFuncSetAttribute(tc_band_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)band::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)div_up(p.T, band::BQ), (unsigned)(p.B * p.H));
  tc_band_kernel<<<grid, 192, band::SMEM_BYTES, st>>>(a);
  return cudaGetLastError();
}

cudaError_t tc_read_status(const Workspace& ws, char* base, int* host_status, cudaStream_t st) {
  cudaError_t e = cudaMemcpyAsync(host_status, base + ws.status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(st);
}

}  // namespace sbl
