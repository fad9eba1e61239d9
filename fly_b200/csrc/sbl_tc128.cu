// bf16 tensor-core path of the SBLocal forward for head dim 128 on sm_100a:
// E = D = 128, r = 256 projection rows (m = 512 features), eps = 0, any T, S,
// w, key lengths.  Same arithmetic and the same "feature units" as the
// head-dim-64 kernels of sbl_tc.cu (nothing is ever rescaled), but a different
// plan, because neither tensor memory nor shared memory holds what those
// kernels keep resident:
//
//   keys128   grid (4 x splits, b*h): one CTA per projection QUARTER (64
//             projections = 128 features) and run of 128-key tiles.  U = K Wq^T
//             (N = 64), the feature warps write phi(K) in bf16 to the workspace
//             and, MN-major, to shared memory, KV[128 f][128 d] += phi(K)^T V and
//             sum phi(K) (a second product with a block of ones) accumulate in
//             tensor memory; one partial summary per CTA (16 feature warps, 16
//             projections per thread).  The four quarter CTAs
//             of a split are neighbours in the grid, so the K and V tiles they
//             all read meet in L2.
//   combine128  sums the split partials -> KV (fp32 and bf16), sum phi(K)
//   band128   persistent, one CTA per SM, 128-query tiles dealt round-robin.
//             Tensor memory: O (128 columns) | two S/E/D buffers (2 x 128) | feature
//             half 0 of phi(Q) (128 columns = 256 bf16 features, formed in place
//             over its U).  Half 1 does not fit: its U is parked in the second
//             buffer at the start of a query tile and its features go to SHARED
//             memory as a K-major operand, so the products over half 1 are SS-form
//             MMAs.  Per key tile: S = Q K^T, E = exp(tau S - pls), E -= P_0 (A in
//             tensor memory), E -= P_1 (A in shared memory), pack to bf16,
//             O += D V; O += phi(Q)_h KV_h for both halves ahead of the key tiles.
//             Every B operand streams through a ring of 32 KB slots in exactly the
//             order its MMA-issuing warp consumes it: the phi(K) pieces through
//             one ring to the warp that issues the P products, K, V, Wt and KV
//             pieces through another to the warp that issues everything else; the
//             finished output tile is staged in a slot of the second ring.  Each
//             issuer issues in program order, so buffer reuse between its own MMAs
//             needs no barrier; barriers order the two issuers, the softmax warps
//             and the rings.
//
// Feature order inside this path: slot kp = 128*q + 32*c + 16*s + j holds
// feature exp((-1)^s u_p ...) of projection p = 64*q + 16*c + j (reference index
// p + 256*s): the 32 features a thread forms from 16 projections sit in the 16
// tensor-memory columns it read them from.  phi(K) in the workspace, the split
// partials and the bf16 KV use this order; kv / ksum exchanged with callers use
// the reference's.
#include "sbl_common.cuh"
#include "sbl_tc_dev.cuh"
#include "sbl_tc_host.cuh"

namespace sbl {
namespace {

using namespace ptx;
using namespace tcdev;
using namespace tch;

constexpr int kE = 128;    // head dim (qk and v)
constexpr int kR = 256;    // projection rows
constexpr int kM = 512;    // features
constexpr int kPitch = 144;   // row pitch (floats) of a split-partial summary: 128 KV columns, the feature sum, padding

// Reference feature index of internal slot kp.
__host__ __device__ constexpr int feat_of_slot(int kp) {
  return 64 * (kp >> 7) + 16 * ((kp >> 5) & 3) + (kp & 15) + 256 * ((kp >> 4) & 1);
}

// Waits on mbarriers by phase bit: every waiter keeps one bit per barrier and flips it after each wait, so
// no role has to count how often a barrier has completed.
struct Phases {
  uint32_t bits = 0;
  __device__ __forceinline__ void wait(uint64_t* bars, int bi, int* status, int code) {
    mbar_wait(bars + bi, (bits >> bi) & 1u, status, code);
    bits ^= 1u << bi;
  }
};

// ---------------------------------------------------------------------------
// kv (BH,512,128), ksum (BH,512) = sum over the splits of the per-CTA partial summaries.  The partials and
// kv16 (the band kernel's bf16 operand) are in the internal feature order, kv and ksum in the reference's.
__global__ void tc128_combine_kernel(const float* partial, int nsplit, int BH, float* kv, float* ksum,
                                     __nv_bfloat16* kv16, float* ksum_slots) {
  constexpr int G = kPitch / 4;   // float4 groups per partial row: 32 of KV, then the feature sum
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)BH * kM * G) return;
  const int g = (int)(i % G);
  const int64_t bf = i / G;       // bh * 512 + slot
  if (g > 32) return;
  const int64_t bh = bf / kM;
  const int kp = (int)(bf % kM);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < nsplit; ++k) {
    const float4 v = *reinterpret_cast<const float4*>(partial + ((bh * nsplit + k) * kM + kp) * kPitch + 4 * g);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const int64_t out_row = bh * kM + feat_of_slot(kp);
  if (g < 32) {
    *reinterpret_cast<float4*>(kv + out_row * kE + 4 * g) = acc;
    if (kv16) *reinterpret_cast<uint2*>(kv16 + bf * kE + 4 * g) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  } else {
    ksum[out_row] = acc.x;
    if (kv16) ksum_slots[bf] = acc.x;   // the band kernel reads the feature sums in the internal order
  }
}

// kv (BH,512,128) fp32 in the reference's feature order -> bf16 in the internal order
__global__ void tc128_kv_to_bf16_kernel(const float* kv, __nv_bfloat16* kv16, int64_t n, const float* ksum,
                                        float* ksum_slots) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (i < n / kE) ksum_slots[i] = ksum[(i / kM) * kM + feat_of_slot((int)(i % kM))];
  const int d = (int)(i % kE);
  const int64_t row = i / kE;
  const int64_t bh = row / kM;
  const int kp = (int)(row % kM);
  kv16[i] = __float2bfloat16_rn(kv[(bh * kM + feat_of_slot(kp)) * kE + d]);
}

// ---------------------------------------------------------------------------
// keys kernel
struct Keys128Args {
  CUtensorMap tm_k, tm_v, tm_w, tm_phik;
  const int64_t* lengths;
  const float* beta;
  __nv_bfloat16* phik;    // (BH, S, 512), internal feature order
  float* partial;         // (BH, nsplit, 512, 144)
  int* status;
  int S, H, sum_lo, sum_hi, nsplit;
  int64_t k_pos0, S_total;
  float tau, half_log_m;
};

namespace keys128 {
constexpr int TILE = 128;
constexpr int NFEAT = 512;                 // feature threads: warp w owns key rows 32*(w%4).., 16 projections w/4
constexpr int WPK = NFEAT / 32;            // producer warp of W and K; WPK+1: MMA warp; WPK+2: producer warp of V
constexpr int NTHREADS = NFEAT + 96;
constexpr uint32_t OFF_W = 0;                     // 16 KB: two blocks [64 r][64 e] (e 0-63, e 64-127) of this quarter of Wt
constexpr uint32_t OFF_K = 16384;                 // 2 x 32 KB: per key tile two blocks [128 keys][64 e]
constexpr uint32_t OFF_V = OFF_K + 65536;         // 2 x 32 KB: per key tile two blocks [128 keys][64 d] (MN-major, N = 128)
constexpr uint32_t OFF_A = OFF_V + 65536;         // 2 x 32 KB: two blocks [128 keys][64 f] = phi(K) tile, MN-major A operand
constexpr uint32_t OFF_ONES = OFF_A + 65536;      // 2 KB of bf16 ones: the B operand (N = 16) of the feature sum
constexpr uint32_t OFF_NORM = OFF_ONES + 2048;    // 4 KB: partial row norms, fp32 [2 tile parities][4 row quarters][128 keys]
constexpr uint32_t OFF_BAR = OFF_NORM + 4096;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 512 + 1024;    // + alignment slack
static_assert(SMEM_BYTES <= 232448, "dynamic shared memory of one CTA");
// tensor memory columns
constexpr uint32_t T_UK = 0;      // 2 x 64
constexpr uint32_t T_KV = 128;    // 128: KV of this quarter's 128 features
constexpr uint32_t T_KS = 256;    // 16 identical columns: sum phi(K)
}  // namespace keys128

__global__ void __launch_bounds__(keys128::NTHREADS) tc128_keys_kernel(const __grid_constant__ Keys128Args a) {
  using namespace keys128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* bar_w = bars + 0;
  uint64_t* bar_done = bars + 1;
  uint64_t* v_full = bars + 2;    // [2] V tile landed
  uint64_t* v_empty = bars + 4;   // [2] V tile consumed by the summary MMAs
  uint64_t* k_full = bars + 6;    // [2] K tile landed
  uint64_t* k_free = bars + 8;    // [2] K tile consumed: U computed and every row norm read
  uint64_t* uk_full = bars + 10;  // [2] U = K Wq^T computed
  uint64_t* uk_free = bars + 12;  // [2] U read by all feature threads
  uint64_t* a_full = bars + 14;   // [2] phi(K) tile written to shared memory
  uint64_t* a_free = bars + 16;   // [2] phi(K) tile consumed (MMAs done + bulk store has read it)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int ntiles = (a.S + TILE - 1) / TILE;
  const int split = blockIdx.x >> 2, qt = blockIdx.x & 3;   // qt: projection quarter
  const int t_lo = (int)((int64_t)ntiles * split / a.nsplit);
  const int t_hi = (int)((int64_t)ntiles * (split + 1) / a.nsplit);
  const int nt = t_hi - t_lo;
  const int64_t len_b = a.lengths ? min(a.lengths[b], a.S_total) : a.S_total;

  if (tid == 0) {
    mbar_init(bar_w, 1);
    mbar_init(bar_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(v_full + i, 1);
      mbar_init(v_empty + i, 1);
      mbar_init(k_full + i, 1);
      mbar_init(k_free + i, NFEAT / 32);   // one arrival per feature warp
      mbar_init(uk_full + i, 1);
      mbar_init(uk_free + i, NFEAT / 32);   // one arrival per feature warp
      mbar_init(a_full + i, NFEAT / 32);   // one arrival per feature warp
      mbar_init(a_free + i, 2);
    }
    fence_mbar_init();
  }
  if (warp == WPK) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  for (int i = tid; i < 1024; i += NTHREADS)
    reinterpret_cast<__nv_bfloat16*>(smem + OFF_ONES)[i] = __float2bfloat16(1.0f);
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  constexpr uint32_t tb = 0;   // the CTA owns all 512 tensor-memory columns of its SM
  if (tid == 0 && *tmem_slot != 0) atomicCAS(a.status, 0, 141);

  // a tile whose rows all enter the summary and hold real keys is stored to the workspace by bulk copies
  auto tile_is_plain = [&](int i) {
    const int row0 = (t_lo + i) * TILE;
    return row0 >= a.sum_lo && row0 + TILE <= a.sum_hi && a.k_pos0 + row0 + TILE <= len_b;
  };

  if (warp == WPK) {
    // ---------------- producer ----------------
    const bool leader = elect_one();
    if (leader) {
      prefetch_tmap(&a.tm_k);
      prefetch_tmap(&a.tm_v);
      prefetch_tmap(&a.tm_w);
      prefetch_tmap(&a.tm_phik);
      mbar_expect_tx(bar_w, 16384);
      tma_load_2d(smem + OFF_W, &a.tm_w, bar_w, 0, 64 * qt);
      tma_load_2d(smem + OFF_W + 8192, &a.tm_w, bar_w, 64, 64 * qt);
    }
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      const int row0 = (t_lo + i) * TILE;
      if (i >= 2) mbar_wait(k_free + s, ((i >> 1) - 1) & 1, a.status, 111);
      if (leader) {
        mbar_expect_tx(k_full + s, 32768);
        tma_load_4d(smem + OFF_K + s * 32768, &a.tm_k, k_full + s, 0, row0, h, b);
        tma_load_4d(smem + OFF_K + s * 32768 + 16384, &a.tm_k, k_full + s, 64, row0, h, b);
      }
    }
    __syncwarp();
  } else if (warp == WPK + 2) {
    // ---------------- producer of V: a warp of its own, so that the wait for a V slot (freed by the summary
    // MMAs, late in a tile) does not hold back the next K tile, which the projection needs early ----------------
    const bool leader = elect_one();
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      const int row0 = (t_lo + i) * TILE;
      if (i >= 2) mbar_wait(v_empty + s, ((i >> 1) - 1) & 1, a.status, 112);
      if (leader) {
        mbar_expect_tx(v_full + s, 32768);
        tma_load_4d(smem + OFF_V + s * 32768, &a.tm_v, v_full + s, 0, row0, h, b);
        tma_load_4d(smem + OFF_V + s * 32768 + 16384, &a.tm_v, v_full + s, 64, row0, h, b);
      }
    }
    __syncwarp();
  } else if (warp == WPK + 1) {
    // ---------------- MMA issuer ----------------
    const bool leader = elect_one();
    constexpr uint32_t id_uk = idesc_bf16(128, 64, false, false);
    constexpr uint32_t id_kv = idesc_bf16(128, 128, true, true);
    constexpr uint32_t id_ks = idesc_bf16(128, 16, true, true);
    const uint64_t dW = smem_desc_sw128(smem_u32(smem + OFF_W), 16, 1024);
    const uint64_t dK0 = smem_desc_sw128(smem_u32(smem + OFF_K), 16, 1024);
    // MN-major operands of two 64-element blocks 16 KB apart
    const uint64_t dA0 = smem_desc_sw128(smem_u32(smem + OFF_A), 16384, 1024);
    const uint64_t dV0 = smem_desc_sw128(smem_u32(smem + OFF_V), 16384, 1024);
    const uint64_t dOnes = smem_desc_sw128(smem_u32(smem + OFF_ONES), 16384, 1024);
    auto issue_kv = [&](int u) {
      const int s = u & 1;
      mbar_wait(a_full + s, (u >> 1) & 1, a.status, 113);
      mbar_wait(v_full + s, (u >> 1) & 1, a.status, 114);
      tc_fence_after_sync();
      if (leader) {
        // bulk copy of the phi(K) tile to the workspace (an empty group keeps the group count uniform)
        if (tile_is_plain(u)) {
          const int row0 = (t_lo + u) * TILE;
#pragma unroll
          for (int j = 0; j < 2; ++j)
            tma_store_3d(&a.tm_phik, smem + OFF_A + s * 32768 + j * 16384, 128 * qt + 64 * j, row0, bh);
        }
        tma_store_commit();
        const uint64_t dA = dA0 + (uint64_t)(s * (32768 >> 4));
        const uint64_t dV = dV0 + (uint64_t)(s * (32768 >> 4));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ss(tb + T_KV, dA + (uint64_t)(k * (2048 >> 4)), dV + (uint64_t)(k * (2048 >> 4)), id_kv, (u > 0) || (k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ss(tb + T_KS, dA + (uint64_t)(k * (2048 >> 4)), dOnes, id_ks, (u > 0) || (k > 0));
        mma_commit(a_free + s);
        mma_commit(v_empty + s);
        // the previous tile's bulk copy has read its buffer once at most one group is pending
        if (u >= 1) {
          tma_store_wait_read1();
          mbar_arrive(a_free + (s ^ 1));
        }
      }
      __syncwarp();
    };
    mbar_wait(bar_w, 0, a.status, 115);
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      mbar_wait(k_full + s, (i >> 1) & 1, a.status, 116);
      if (i >= 2) mbar_wait(uk_free + s, ((i >> 1) - 1) & 1, a.status, 117);
      tc_fence_after_sync();
      if (leader) {
        const uint32_t td = tb + T_UK + s * 64;
        const uint64_t dK = dK0 + (uint64_t)(s * (32768 >> 4));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ss(td, dK + (uint64_t)((k >> 2) * (16384 >> 4) + (k & 3) * 2),
                 dW + (uint64_t)((k >> 2) * (8192 >> 4) + (k & 3) * 2), id_uk, k > 0);
        mma_commit(uk_full + s);
      }
      __syncwarp();
      if (i >= 1) issue_kv(i - 1);
    }
    if (nt > 0) issue_kv(nt - 1);
    if (leader) {
      mma_commit(bar_done);
      tma_store_wait_all();
    }
    __syncwarp();
  } else {
    // ---------------- feature warps ----------------
    // Sixteen warps: with eight, a warp was busy 2.9 k cycles per tile (two warps per scheduler leave the latencies
    // of the row-norm loads, the tensor-memory load and the exponentials exposed).
    const int qd = warp & 3, cq = warp >> 2;         // lane quarter (key rows), group of 16 projections
    const int krow = qd * 32 + lane;                 // key row inside the tile
    const uint32_t lane_base = tb + ((uint32_t)(qd * 32) << 16);
    const float beta = a.beta[bh];
    float* s_norm = reinterpret_cast<float*>(smem + OFF_NORM);
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      const int row = (t_lo + i) * TILE + krow;
      mbar_wait(k_full + s, (i >> 1) & 1, a.status, 118);
      // |k|^2: each of the four threads of a row sums a quarter of it (64 bytes); they meet in shared memory behind
      // a named barrier of their four warps.  The buffer alternates with the tile, so one barrier per tile does.
      {
        const uint8_t* line = smem + OFF_K + s * 32768 + (cq >> 1) * 16384 + krow * 128;
        float part = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(line + (((4 * (cq & 1) + c) ^ (krow & 7)) << 4));
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x = bf16_lo(w4[j]), y = bf16_hi(w4[j]);
            part = fmaf(x, x, part);
            part = fmaf(y, y, part);
          }
        }
        s_norm[(s * 4 + cq) * 128 + krow] = part;
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + qd) : "memory");
      const float* nb = s_norm + s * 512 + krow;
      const float g = 0.5f * a.tau * ((nb[0] + nb[128]) + (nb[256] + nb[384]));
      mbar_wait(uk_full + s, (i >> 1) & 1, a.status, 119);   // U computed: the tensor core is done with the K tile too
      tc_fence_after_sync();
      warp_arrive(k_free + s, lane);
      const bool live = row < a.S && (a.k_pos0 + row) < len_b;
      const bool in_sum = live && row >= a.sum_lo && row < a.sum_hi;
      const bool plain = tile_is_plain(i);
      const float off = ((-g - a.half_log_m) - beta) * kLog2e;
      const int blk = cq >> 1, gi = cq & 1;            // 64-feature block, group of 16 projections inside it
      __nv_bfloat16* grow = a.phik + ((int64_t)bh * a.S + row) * kM + 128 * qt + 64 * blk;
      uint8_t* sA = smem + OFF_A + s * 32768 + blk * 16384;
      uint32_t r[16];
      tmem_ld16(lane_base + T_UK + s * 64 + 16 * cq, r);
      tmem_ld_wait();
      tc_fence_before_sync();
      warp_arrive(uk_free + s, lane);
      uint32_t p1[8], p2[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        constexpr float2 lp = {kLog2e, kLog2e}, lm = {-kLog2e, -kLog2e};
        const float2 u = make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        const float2 ap = fma2(u, lp, make_float2(off, off)), am = fma2(u, lm, make_float2(off, off));
        const float2 ep = make_float2(ex2(ap.x), ex2(ap.y));
        const float2 em = make_float2(ex2(am.x), ex2(am.y));
        p1[j] = live ? pack_bf16(ep.x, ep.y) : 0u;
        p2[j] = live ? pack_bf16(em.x, em.y) : 0u;
      }
      // A group of 16 projections fills half of a 64-feature block of the internal order: two 16-byte pieces of
      // the "+" features, then two of the "-" features.
      if (!plain && row < a.S) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const uint32_t* src = (x >> 1) ? p2 : p1;
          const int o = 4 * (x & 1);
          reinterpret_cast<uint4*>(grow)[4 * gi + x] = make_uint4(src[o], src[o + 1], src[o + 2], src[o + 3]);
        }
      }
      // the MMAs and the bulk store of the tile before the previous one must be done with the shared buffer
      if (i >= 2) mbar_wait(a_free + s, ((i >> 1) - 1) & 1, a.status, 120);
      // MN-major A operand: 16-byte piece q8 of the key's 128-byte line, swizzled by key % 8
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const uint32_t* src = (x >> 1) ? p2 : p1;
        const int o = 4 * (x & 1);
        const int q8 = 4 * gi + x;
        const uint32_t so = (uint32_t)krow * 128u + (uint32_t)((q8 ^ (krow & 7)) << 4);
        *reinterpret_cast<uint4*>(sA + so) =
            in_sum ? make_uint4(src[o], src[o + 1], src[o + 2], src[o + 3]) : make_uint4(0, 0, 0, 0);
      }
      fence_async_smem();
      warp_arrive(a_full + s, lane);
    }
    mbar_wait(bar_done, 0, a.status, 121);
    tc_fence_after_sync();
    // thread (feature row, quarter): writes 32 of the row's 128 KV columns; the last quarter also the feature sum
    float* prow = a.partial + (((int64_t)bh * a.nsplit + split) * kM + 128 * qt + krow) * kPitch;
#pragma unroll 1
    for (int gq = 0; gq < 2; ++gq) {
      uint32_t r[16];
      tmem_ld16(lane_base + T_KV + 32 * cq + 16 * gq, r);
      tmem_ld_wait();
      if (nt == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        reinterpret_cast<uint4*>(prow + 32 * cq + 16 * gq)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    }
    {
      uint32_t q[16];
      tmem_ld16(lane_base + T_KS, q);
      tmem_ld_wait();
      if (cq == 3) prow[128] = nt == 0 ? 0.f : __uint_as_float(q[0]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == WPK) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------
// band kernel
struct Band128Args {
  CUtensorMap tm_q, tm_k, tm_v, tm_w, tm_phik, tm_kv, tm_out;
  SblParams p;
  const float* beta;
  const float* ksum;     // (BH, 512) fp32, internal feature order
  const float* wmax;     // [1]: max_f |sqrt(tau) w_f| of the bf16 projection
  int* status;
  int ntq;               // query tiles per (b,h)
  int ntiles;            // ntq * B * H
};

namespace band128 {
constexpr int BQ = 128, KT = 128;
constexpr int NSOFT = 512;                 // softmax threads: two groups of 256, warp w owns rows 32*(w%4)..
constexpr int WGRP = 8;                    // warps per softmax group (exponential group, packing group)
constexpr int W_LOAD = 16;                 // producer warp of the main ring (Wt, K, KV, V) and of Q
constexpr int W_LOADP = 17;                // producer warp of the phi(K) ring
constexpr int W_MMA = 18;                  // MMA issuer warp: U, S, low-rank, O
constexpr int W_MMAP = 19;                 // MMA issuer warp: P
constexpr int NTHREADS = NSOFT + 128;
constexpr uint32_t OFF_Q = 0;              // 32 KB: two blocks [128 q][64 e]
constexpr uint32_t OFF_PHI1 = 32768;       // 64 KB: feature half 1 of phi(Q), bf16, four blocks [128 q][64 f] (A operand)
constexpr uint32_t OFF_RING = OFF_PHI1 + 65536;   // ring of 32 KB slots: every B operand, and the staged output tile
// Four slots (two per ring), the Q tile and half of phi(Q) leave 2.5 KB of the 227 KB: the feature sums are read
// from global memory (L1), the row sums of D are exchanged through the output staging slot, and the kernel relies
// on (and checks) a 1024-byte aligned shared-memory base.  (The rings are not deeper for a reason: what limits the
// operand stream is the rate at which one SM takes data in, 32 KB per 785 cycles whatever the depth.)
constexpr uint32_t NSLOT = 2, SLOT = 32768;       // slots of EACH of the two rings
constexpr uint32_t OFF_RINGP = OFF_RING + NSLOT * SLOT;  // second ring: phi(K) pieces only, consumed by the P issuer
constexpr uint32_t OFF_MISC = OFF_RINGP + NSLOT * SLOT;  // (L, Z) fp32[2][2][128]
constexpr uint32_t OFF_BAR = OFF_MISC + 2048;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 512;
static_assert(SMEM_BYTES <= 232448, "dynamic shared memory of one CTA");
// tensor memory columns (512)
constexpr uint32_t T_O = 0;        // 128
constexpr uint32_t T_BUF = 128;    // 2 x 128: S of a key tile, then E, then E - P (fp32), then D packed bf16 in place;
                                   //          at the start of a query tile one of them holds U half 1
constexpr uint32_t T_PHI = 384;    // 128: U half 0 (fp32), then 256 bf16 features in place
enum {
  B_QFULL = 0,                    // Q tile landed
  B_QFREE,                        // Q buffer reusable: last MMA reading it + one arrival per exponential warp
  B_FULL,                         // [NSLOT] ring slot landed
  B_EMPTY = B_FULL + NSLOT,       // [NSLOT] ring slot consumed (MMAs done, or the output store has read it)
  B_PKFULL = B_EMPTY + NSLOT,     // [NSLOT] the same for the phi(K) ring
  B_PKEMPTY = B_PKFULL + NSLOT,   // [NSLOT]
  B_PFREE = B_PKEMPTY + NSLOT,    // every P product of the query tile done: both halves of phi(Q) may be replaced
  B_UFULL,                        // [2] U half computed
  B_PHIFULL = B_UFULL + 2,        // [2] features of the half formed (one arrival per exponential warp)
  B_SFULL = B_PHIFULL + 2,        // [2] S computed into the buffer
  B_EDONE = B_SFULL + 2,          // [2] E written (one arrival per exponential warp)
  B_PDONE = B_EDONE + 2,          // [2] P subtracted
  B_DDONE = B_PDONE + 2,          // [2] D packed (one arrival per packing warp)
  B_OFREE = B_DDONE + 2,          // O read by the epilogue (one arrival per packing warp)
  B_DONE,                         // all MMAs of the query tile done
  B_LZFULL,                       // L and Z of the query tile published by the exponential group
  B_LZFREE,                       // ... and read by the packing group (one arrival per packing warp)
  B_OUTREADY,                     // the ring slot that stages this tile's output is free
  B_COUNT
};
static_assert(B_COUNT <= 32, "one phase bit per barrier");
}  // namespace band128

// Geometry of one 128-query tile: which key tiles it visits.
struct Tile128 {
  int bh, b, h, i0, nq, len_b, j0, nt;
};
// CTA c takes query tiles c, c + grid, c + 2 grid, ...: at any time the CTAs of the grid work on neighbouring
// query tiles, so the K, V and phi(K) tiles that five neighbouring query tiles share are fetched from HBM once
// and found in L2 by the other four (a CTA walking a contiguous run re-reads them long after L2 has lost them).
__device__ __noinline__ Tile128 tile128(const Band128Args& a, int it) {
  const SblParams& p = a.p;
  const int tile_id = blockIdx.x + it * gridDim.x;
  Tile128 t;
  t.bh = tile_id / a.ntq;
  t.b = t.bh / p.H;
  t.h = t.bh - t.b * p.H;
  t.i0 = (tile_id - t.bh * a.ntq) * band128::BQ;
  t.nq = min(band128::BQ, p.T - t.i0);
  t.len_b = (int)(p.key_lengths ? min(p.key_lengths[t.b], p.S_total) : p.S_total);
  const int hw = p.w / 2;
  // key buffer rows any query of this tile can see, clipped to the buffer and to the key length
  int lo = (int)(p.q_pos0 + t.i0 - hw - p.k_pos0);
  int hi = (int)(p.q_pos0 + t.i0 + t.nq - 1 - hw + p.w - 1 - p.k_pos0);
  lo = max(lo, 0);
  hi = min(hi, min(p.S - 1, t.len_b - 1 - (int)p.k_pos0));
  t.j0 = (lo / band128::KT) * band128::KT;
  t.nt = hi >= lo ? (hi - t.j0) / band128::KT + 1 : 0;
  return t;
}

// Ring position: slot of the next piece, and whether the ring has gone round once.
struct RingPos {
  uint32_t slot = 0;
  bool wrapped = false;
  __device__ __forceinline__ void advance() {
    if (++slot == band128::NSLOT) {
      slot = 0;
      wrapped = true;
    }
  }
  __device__ __forceinline__ void advance(int n) {
    for (int i = 0; i < n; ++i) advance();
  }
};

// Two rings of 32 KB slots, each with its own producer warp and its own MMA-issuing warp, so that the P products
// (which wait for E and take four pieces each) and the rest do not hold each other up.  Per query tile with nt key
// tiles the main ring carries 7 + 2 nt pieces in the order of its issuer's MMA groups:
//   Wt half 0 [first tile] | Wt half 1 | K(0) | KV half 0 (2) | K(1) | KV half 1 (2) |
//   t = 1..nt:  Wt half 0 of the next tile [t = nt] | V(t-1) | K(t+1) [t+1 < nt] |   the output staging slot
// and the phi(K) ring 4 nt pieces:  t = 0..nt-1:  phi(K)_0(t) (2), phi(K)_1(t) (2).
// Key tile t of a query tile uses buffer (G + t) & 1, G = key tiles of the earlier query tiles of this CTA.
__global__ void __launch_bounds__(band128::NTHREADS, 1) tc128_band_kernel(const __grid_constant__ Band128Args a) {
  using namespace band128;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled tiles need it; no slack is left to realign by hand
    if (threadIdx.x == 0) atomicCAS(a.status, 0, 142);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 62);
  float* s_lz = reinterpret_cast<float*>(smem + OFF_MISC);   // [L, Z][2 column halves][128 rows]

  const SblParams& p = a.p;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hw = p.w / 2;
  const int n_it = (a.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (warp == W_MMA) {
    for (int i = lane; i < B_COUNT; i += 32) {
      int count = 1;
      if ((i >= B_PHIFULL && i < B_PHIFULL + 2) || (i >= B_EDONE && i < B_EDONE + 2) ||
          (i >= B_DDONE && i < B_DDONE + 2) || i == B_OFREE || i == B_LZFULL || i == B_LZFREE)
        count = WGRP;
      if (i == B_QFREE) count = WGRP + 1;
      mbar_init(bars + i, count);
    }
    fence_mbar_init();
  }
  if (warp == W_LOAD) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  constexpr uint32_t tb = 0;   // the CTA owns all 512 tensor-memory columns of its SM
  if (tid == 0 && *tmem_slot != 0) atomicCAS(a.status, 0, 140);

  if (warp == W_LOAD) {
    // ---------------- producer: whole warp waits, one lane issues ----------------
    const bool leader = elect_one();
    if (leader) {
      prefetch_tmap(&a.tm_q);
      prefetch_tmap(&a.tm_k);
      prefetch_tmap(&a.tm_v);
      prefetch_tmap(&a.tm_w);
      prefetch_tmap(&a.tm_phik);
      prefetch_tmap(&a.tm_kv);
    }
    Phases ph;
    RingPos rp;
    // next ring slot, once its previous content has been consumed
    auto acquire = [&]() {
      const uint32_t s = rp.slot;
      if (rp.wrapped) ph.wait(bars, B_EMPTY + s, a.status, 150);
      rp.advance();
      return s;
    };
    auto load_q = [&](const Tile128& T) {
      if (leader) {
        mbar_expect_tx(bars + B_QFULL, 32768);
        tma_load_4d(smem + OFF_Q, &a.tm_q, bars + B_QFULL, 0, T.i0, T.h, T.b);
        tma_load_4d(smem + OFF_Q + 16384, &a.tm_q, bars + B_QFULL, 64, T.i0, T.h, T.b);
      }
    };
    auto load_w = [&](int half) {
      const uint32_t s = acquire();
      if (leader) {
        uint8_t* dst = smem + OFF_RING + s * SLOT;
        mbar_expect_tx(bars + B_FULL + s, 32768);
        tma_load_2d(dst, &a.tm_w, bars + B_FULL + s, 0, 128 * half);
        tma_load_2d(dst + 16384, &a.tm_w, bars + B_FULL + s, 64, 128 * half);
      }
    };
    auto load_rows = [&](const CUtensorMap* m, const Tile128& T, int t) {   // K or V tile t of the band
      const uint32_t s = acquire();
      if (leader) {
        uint8_t* dst = smem + OFF_RING + s * SLOT;
        mbar_expect_tx(bars + B_FULL + s, 32768);
        tma_load_4d(dst, m, bars + B_FULL + s, 0, T.j0 + t * KT, T.h, T.b);
        tma_load_4d(dst + 16384, m, bars + B_FULL + s, 64, T.j0 + t * KT, T.h, T.b);
      }
    };
    auto load_kv = [&](const Tile128& T, int half) {   // two pieces of 128 features each
      for (int fg = 0; fg < 2; ++fg) {
        const uint32_t s = acquire();
        if (leader) {
          uint8_t* dst = smem + OFF_RING + s * SLOT;
          mbar_expect_tx(bars + B_FULL + s, 32768);
          tma_load_3d(dst, &a.tm_kv, bars + B_FULL + s, 0, 256 * half + 128 * fg, T.bh);
          tma_load_3d(dst + 16384, &a.tm_kv, bars + B_FULL + s, 64, 256 * half + 128 * fg, T.bh);
        }
      }
    };
    Tile128 T = tile128(a, 0), Tn{};
    load_q(T);
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
      const bool have_next = it + 1 < n_it;
      if (have_next) Tn = tile128(a, it + 1);
      const int nt = T.nt;
      // Pull the diagonal key tile of the NEXT query tile (K, V, phi(K): 192 KB) into L2 now.  The CTAs of the grid
      // work on neighbouring query tiles, so between them they prefetch every key tile the grid's next round reads.
      if (have_next && leader) {
        const int row0 = (int)(p.q_pos0 + Tn.i0 - p.k_pos0) / KT * KT;
        if (row0 >= Tn.j0 && row0 < Tn.j0 + Tn.nt * KT) {
#pragma unroll 1
          for (int x = 0; x < kE; x += 64) {
            tma_prefetch_4d(&a.tm_k, x, row0, Tn.h, Tn.b);
            tma_prefetch_4d(&a.tm_v, x, row0, Tn.h, Tn.b);
          }
#pragma unroll 1
          for (int x = 0; x < kM; x += 64) tma_prefetch_3d(&a.tm_phik, x, row0, Tn.bh);
        }
      }
      if (it == 0) load_w(0);     // later tiles: loaded at the tail of the tile before, see below
      load_w(1);
      if (nt > 0) load_rows(&a.tm_k, T, 0);
      load_kv(T, 0);
      if (nt > 1) load_rows(&a.tm_k, T, 1);
      load_kv(T, 1);
      bool q_loaded = false;
#pragma unroll 1
      for (int t = 0; t <= nt; ++t) {
        if (have_next && !q_loaded && t >= nt - 1) {
          // every S of this tile and both U halves have been issued by now: the Q buffer is about to be free
          ph.wait(bars, B_QFREE, a.status, 151);
          load_q(Tn);
          q_loaded = true;
        }
        // The first U half of the NEXT tile is computed ahead of this tile's last O += D V: the exponential warps,
        // idle by then, turn it into features while this tile's packing and epilogue finish.
        if (t == nt && have_next) load_w(0);
        if (t >= 1) load_rows(&a.tm_v, T, t - 1);
        if (t >= 1 && t + 1 < nt) load_rows(&a.tm_k, T, t + 1);
      }
      // the slot that stages the output tile: hand it to the packing group
      acquire();
      if (leader) mbar_arrive(bars + B_OUTREADY);
      __syncwarp();
      T = Tn;
    }
  } else if (warp == W_LOADP) {
    // ---------------- producer of the phi(K) ring ----------------
    const bool leader = elect_one();
    if (leader) prefetch_tmap(&a.tm_phik);
    Phases ph;
    RingPos rp;
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
      const Tile128 T = tile128(a, it);
#pragma unroll 1
      for (int t = 0; t < T.nt; ++t)
#pragma unroll 1
        for (int hj = 0; hj < 4; ++hj) {             // half hj / 2, piece hj % 2 of 128 features
          const uint32_t s = rp.slot;
          if (rp.wrapped) ph.wait(bars, B_PKEMPTY + s, a.status, 152);
          rp.advance();
          if (leader) {
            uint8_t* dst = smem + OFF_RINGP + s * SLOT;
            mbar_expect_tx(bars + B_PKFULL + s, 32768);
            tma_load_3d(dst, &a.tm_phik, bars + B_PKFULL + s, 128 * hj, T.j0 + t * KT, T.bh);
            tma_load_3d(dst + 16384, &a.tm_phik, bars + B_PKFULL + s, 128 * hj + 64, T.j0 + t * KT, T.bh);
          }
          __syncwarp();
        }
    }
  } else if (warp == W_MMAP) {
    // ---------------- MMA issuer of the P products: buffer -= phi(Q) phi(K)^T, half 0 (A in tensor memory), then
    // half 1 (A in shared memory) ----------------
    const bool leader = elect_one();
    constexpr uint32_t id_neg = idesc_bf16(128, 128, false, false) | (1u << 13);   // bit 13 negates A
    const uint64_t dPhi1 = smem_desc_sw128(smem_u32(smem + OFF_PHI1), 16, 1024);
    const uint64_t dRingP = smem_desc_sw128(smem_u32(smem + OFF_RINGP), 16, 1024);
    auto koff = [](int k) { return (uint64_t)((k >> 2) * (16384 >> 4) + (k & 3) * 2); };
    Phases ph;
    RingPos rp;
    int G = 0;
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
      const int nt = tile128(a, it).nt;
      ph.wait(bars, B_PHIFULL, a.status, 167);
      ph.wait(bars, B_PHIFULL + 1, a.status, 168);
#pragma unroll 1
      for (int t = 0; t < nt; ++t) {
        const int buf = (G + t) & 1;
        ph.wait(bars, B_EDONE + buf, a.status, 165);
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          const uint32_t s = rp.slot;
          ph.wait(bars, B_PKFULL + s, a.status, 169);
          rp.advance();
          tc_fence_after_sync();
          if (leader) {
            const uint64_t dB = dRingP + (uint64_t)(s * (SLOT >> 4));
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (j < 2)
                mma_ts(tb + T_BUF + buf * 128, tb + T_PHI + 8 * (8 * j + k), dB + koff(k), id_neg, true);
              else
                mma_ss(tb + T_BUF + buf * 128, dPhi1 + koff(8 * (j - 2) + k), dB + koff(k), id_neg, true);
            }
            mma_commit(bars + B_PKEMPTY + s);
            if (j == 3) mma_commit(bars + B_PDONE + buf);
          }
          __syncwarp();
        }
      }
      if (leader) mma_commit(bars + B_PFREE);
      __syncwarp();
      G += nt;
    }
  } else if (warp == W_MMA) {
    // ---------------- main MMA issuer (U, S, low-rank, O): whole warp waits, one lane issues ----------------
    const bool leader = elect_one();
    constexpr uint32_t id_kk = idesc_bf16(128, 128, false, false);             // S, U: both operands K-major
    constexpr uint32_t id_mn = idesc_bf16(128, 128, false, true);              // low-rank, O: B = [K index][128 d]
    const uint64_t dQ = smem_desc_sw128(smem_u32(smem + OFF_Q), 16, 1024);
    const uint64_t dPhi1 = smem_desc_sw128(smem_u32(smem + OFF_PHI1), 16, 1024);
    const uint64_t dRingK = smem_desc_sw128(smem_u32(smem + OFF_RING), 16, 1024);       // K-major piece
    const uint64_t dRingMN = smem_desc_sw128(smem_u32(smem + OFF_RING), 16384, 1024);   // MN-major piece
    Phases ph;
    RingPos rp;
    auto take = [&]() {   // next piece has landed
      const uint32_t s = rp.slot;
      ph.wait(bars, B_FULL + s, a.status, 160);
      rp.advance();
      return s;
    };
    // K step k of a K-major operand made of 64-column blocks 16 KB apart
    auto koff = [](int k) { return (uint64_t)((k >> 2) * (16384 >> 4) + (k & 3) * 2); };
    auto issue_qk = [&](uint32_t td, uint64_t* full_bar) {   // td = Q x (piece)^T: S or a U half
      const uint32_t s = take();
      tc_fence_after_sync();
      if (leader) {
        const uint64_t dB = dRingK + (uint64_t)(s * (SLOT >> 4));
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ss(td, dQ + koff(k), dB + koff(k), id_kk, k > 0);
        mma_commit(bars + B_EMPTY + s);
        mma_commit(full_bar);
      }
      __syncwarp();
    };
    auto issue_lr = [&](int half) {   // O (+)= phi(Q)_half KV_half: half 0 from tensor memory, half 1 from shared memory
      ph.wait(bars, B_PHIFULL + half, a.status, 161);
      for (int fg = 0; fg < 2; ++fg) {
        const uint32_t s = take();
        tc_fence_after_sync();
        if (leader) {
          const uint64_t dB = dRingMN + (uint64_t)(s * (SLOT >> 4));
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (half == 0)
              mma_ts(tb + T_O, tb + T_PHI + 8 * (8 * fg + k), dB + (uint64_t)(k * (2048 >> 4)), id_mn, fg != 0 || k != 0);
            else
              mma_ss(tb + T_O, dPhi1 + koff(8 * fg + k), dB + (uint64_t)(k * (2048 >> 4)), id_mn, true);
          }
          mma_commit(bars + B_EMPTY + s);
        }
        __syncwarp();
      }
    };
    auto issue_o = [&](int buf) {   // O += D V: D packed bf16 sits in the first 16 of every 32 columns of the buffer
      ph.wait(bars, B_DDONE + buf, a.status, 162);
      const uint32_t s = take();
      tc_fence_after_sync();
      if (leader) {
        const uint64_t dB = dRingMN + (uint64_t)(s * (SLOT >> 4));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ts(tb + T_O, tb + T_BUF + buf * 128 + 32 * (k >> 1) + 8 * (k & 1), dB + (uint64_t)(k * (2048 >> 4)), id_mn,
                 true);
        mma_commit(bars + B_EMPTY + s);
      }
      __syncwarp();
    };
    int G = 0;
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
      const int nt = tile128(a, it).nt;
      const int b0 = G & 1, b1 = b0 ^ 1;       // buffers of this tile's key tiles 0 and 1
      if (it == 0) {
        ph.wait(bars, B_QFULL, a.status, 163);
        issue_qk(tb + T_PHI, bars + B_UFULL);                   // U half 0: features formed in place
      }                                                         // (later tiles: issued at the tail of the tile before)
      issue_qk(tb + T_BUF + b1 * 128, bars + B_UFULL + 1);      // U half 1: parked in the buffer of key tile 1
      if (nt > 0) issue_qk(tb + T_BUF + b0 * 128, bars + B_SFULL + b0);
      if (it >= 1) ph.wait(bars, B_OFREE, a.status, 164);       // the previous tile's epilogue has read O
      issue_lr(0);
      // feature half 1 has been written to shared memory: its U is out of the buffer
      if (nt > 1) {
        ph.wait(bars, B_PHIFULL + 1, a.status, 166);
        ph.bits ^= 1u << (B_PHIFULL + 1);                       // issue_lr(1) waits for the same phase again
        issue_qk(tb + T_BUF + b1 * 128, bars + B_SFULL + b1);
      }
      issue_lr(1);
      if (nt <= 2) {                                            // no later MMA of this tile reads Q
        if (leader) mma_commit(bars + B_QFREE);
        __syncwarp();
      }
#pragma unroll 1
      for (int t = 0; t <= nt; ++t) {
        const int buf = (G + t) & 1;
        if (t == nt && it + 1 < n_it) {
          // U half 0 of the next tile, ahead of this tile's last O += D V: its Q tile has landed (every S of this
          // tile has run), and this tile's P products are done with phi(Q)
          ph.wait(bars, B_QFULL, a.status, 163);
          ph.wait(bars, B_PFREE, a.status, 174);
          issue_qk(tb + T_PHI, bars + B_UFULL);
        }
        if (t >= 1) issue_o(buf ^ 1);
        if (t >= 1 && t + 1 < nt) {
          issue_qk(tb + T_BUF + (buf ^ 1) * 128, bars + B_SFULL + (buf ^ 1));
          if (t + 2 == nt) {                                    // that was the last S
            if (leader) mma_commit(bars + B_QFREE);
            __syncwarp();
          }
        }
      }
      if (leader) mma_commit(bars + B_DONE);
      __syncwarp();
      rp.advance();   // the output staging slot
      G += nt;
    }
  } else {
    // ---------------- softmax warps ----------------
    // Exponential group (warps 0-7): the features of both halves, E = exp(tau S - pls) of every key tile, the row
    //   sums L and Z.  Packing group (warps 8-15): D -> bf16 for every key tile, its row sum, the epilogue.
    // A thread of either group owns one query row and 64 columns (two chunks of 32) of every buffer.
    const int qd = warp & 3, cq = (warp >> 2) & 1;   // lane quarter (rows), column half
    const bool exp_group = warp < WGRP;
    const int row = qd * 32 + lane;
    const int gtid = tid & (32 * WGRP - 1);
    const uint32_t lane_base = tb + ((uint32_t)(qd * 32) << 16);
    const int c0 = 64 * cq;
    // Visibility of 32 columns starting at global key position gk0 for query position gi: bit k of vis = the
    // row sees column k (the columns a row sees form one interval); none: no row of this warp sees any of them.
    struct Geo {
      uint32_t vis;
      bool none;
    };
    auto geometry = [&](int gi, int gk0, int len_b) {
      const int lo = max(gi - hw - gk0, 0);
      const int hi = min(min(gi - hw + p.w - 1, len_b - 1) - gk0, 31);
      Geo G;
      G.vis = hi >= lo ? (0xFFFFFFFFu >> (31 - (hi - lo))) << lo : 0u;
      G.none = __all_sync(0xFFFFFFFFu, G.vis == 0u);
      return G;
    };
    Phases ph;
    int G = 0;
    if (exp_group) {
      const float wmax = __ldg(a.wmax);
      const float half_log_m = 0.5f * logf((float)kM);
      const float sc = p.softmax_temp * kLog2e;
      const float* ksum_bh = a.ksum;   // feature sums of the current (b,h), internal order
      float M = 0.f;
      // Features of one half: this thread's 64 projections (four groups of 16 fp32 columns) become, per group,
      // 16 "+" and 16 "-" features; returns its share of phi(Q) . sum phi(K).  Half 0 is written back in place
      // (2 x 8 packed columns per group: the A operand in tensor memory), half 1 is read from the buffer its U was
      // parked in and written to shared memory as a K-major bf16 operand (64 bytes of the row's 128-byte line of
      // block c / 2, 16-byte chunks XORed with row % 8).
      auto form_half = [&](int half, uint32_t tsrc) {
        ph.wait(bars, B_UFULL + half, a.status, 170);
        tc_fence_after_sync();
        const float mo = -M * kLog2e;
        const float2 mo2 = make_float2(mo, mo);
        const float2 lp = make_float2(kLog2e, kLog2e), lm = make_float2(-kLog2e, -kLog2e);
        float2 zz = make_float2(0.f, 0.f);
#pragma unroll 1
        for (int g2 = 0; g2 < 4; ++g2) {
          const int c = 4 * cq + g2;               // group of 16 projections inside the half
          const uint32_t taddr = lane_base + tsrc + 16 * c;
          const float* ks = ksum_bh + 256 * half + 32 * c;
          uint32_t r[16];
          tmem_ld16(taddr, r);
          tmem_ld_wait();
          uint32_t p1[8], p2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 uu = make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            const float2 ap = fma2(uu, lp, mo2), am = fma2(uu, lm, mo2);
            const float2 ep = make_float2(ex2(ap.x), ex2(ap.y));
            const float2 em = make_float2(ex2(am.x), ex2(am.y));
            p1[j] = pack_bf16(ep.x, ep.y);
            p2[j] = pack_bf16(em.x, em.y);
            zz = fma2(ep, __ldg(reinterpret_cast<const float2*>(ks + 2 * j)), zz);
            zz = fma2(em, __ldg(reinterpret_cast<const float2*>(ks + 16 + 2 * j)), zz);
          }
          if (half == 0) {
            tmem_st8(taddr, p1);
            tmem_st8(taddr + 8, p2);
          } else {
            uint8_t* line = smem + OFF_PHI1 + (c >> 1) * 16384 + row * 128;
            const int q0 = 4 * (c & 1);
            *reinterpret_cast<uint4*>(line + (((q0 + 0) ^ (row & 7)) << 4)) = make_uint4(p1[0], p1[1], p1[2], p1[3]);
            *reinterpret_cast<uint4*>(line + (((q0 + 1) ^ (row & 7)) << 4)) = make_uint4(p1[4], p1[5], p1[6], p1[7]);
            *reinterpret_cast<uint4*>(line + (((q0 + 2) ^ (row & 7)) << 4)) = make_uint4(p2[0], p2[1], p2[2], p2[3]);
            *reinterpret_cast<uint4*>(line + (((q0 + 3) ^ (row & 7)) << 4)) = make_uint4(p2[4], p2[5], p2[6], p2[7]);
          }
        }
        if (half == 0) tmem_st_wait(); else fence_async_smem();
        tc_fence_before_sync();
        warp_arrive(bars + B_PHIFULL + half, lane);
        return zz.x + zz.y;
      };
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const Tile128 T = tile128(a, it);
        const int nt = T.nt;
        ksum_bh = a.ksum + (int64_t)T.bh * kM;
        // row norm, stabiliser M = wmax |q| >= |u_f| for every projection (Cauchy-Schwarz), key log-scale
        ph.wait(bars, B_QFULL, a.status, 171);
        const float qn2 = row_sumsq_sw128(smem + OFF_Q, row) + row_sumsq_sw128(smem + OFF_Q + 16384, row);
        warp_arrive(bars + B_QFREE, lane);
        const float gq = 0.5f * p.softmax_temp * qn2;
        M = sqrtf(qn2) * wmax;
        const float beta = __ldg(a.beta + T.bh);
        float z = form_half(0, T_PHI);
        z += form_half(1, T_BUF + ((G + 1) & 1) * 128);
        const int gi = (int)p.q_pos0 + T.i0 + row;     // global query position
        const float pls = (-gq + M - half_log_m) + beta;               // query log-scale + key log-scale
        const float2 sc2 = make_float2(sc, sc);
        const float2 co2 = make_float2(-pls * kLog2e, -pls * kLog2e);  // exp(tau s - pls) = ex2(s * sc + co)
        float L = 0.f;             // row sum of the exponentials over this thread's columns
#pragma unroll 1
        for (int t = 0; t < nt; ++t) {
          // S(t) -> E = exp(tau S - pls) in place (fp32), zero outside the window; row sum
          const int s = (G + t) & 1;
          ph.wait(bars, B_SFULL + s, a.status, 172);
          tc_fence_after_sync();
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            const Geo Gm = geometry(gi, (int)p.k_pos0 + T.j0 + t * KT + c0 + 32 * ch, T.len_b);
            if (Gm.none) continue;   // a chunk nobody sees is left as it is: the packing group writes zeros for it
            const uint32_t tcol = lane_base + T_BUF + s * 128 + c0 + 32 * ch;
            uint32_t rs[32];
            tmem_ld32(tcol, rs);
            tmem_ld_wait();
            float2 l2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 x = fma2(make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1])), sc2, co2);
              float2 e = make_float2(0.f, 0.f);
              if (Gm.vis & (1u << (2 * j))) e.x = ex2(x.x);          // predicated: hidden columns cost no exponential
              if (Gm.vis & (2u << (2 * j))) e.y = ex2(x.y);
              l2 = add2(l2, e);
              rs[2 * j] = __float_as_uint(e.x);
              rs[2 * j + 1] = __float_as_uint(e.y);
            }
            tmem_st32(tcol, rs);
            L += l2.x + l2.y;
          }
          tmem_st_wait();
          tc_fence_before_sync();
          warp_arrive(bars + B_EDONE + s, lane);
        }
        G += nt;
        // the packing group has read the previous tile's L and Z
        if (it >= 1) ph.wait(bars, B_LZFREE, a.status, 173);
        s_lz[cq * 128 + row] = L;
        s_lz[256 + cq * 128 + row] = z;
        warp_arrive(bars + B_LZFULL, lane);
      }
    } else {
      RingPos rp;
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const Tile128 T = tile128(a, it);
        const int nt = T.nt;
        const int gi = (int)p.q_pos0 + T.i0 + row;
        float sd = 0.f;            // row sum of D over this thread's columns
#pragma unroll 1
        for (int t = 0; t < nt; ++t) {
          // E - P, fp32, left by the tensor core -> masked, packed bf16 over the first 16 of every 32 columns of
          // this thread
          const int s = (G + t) & 1;
          ph.wait(bars, B_PDONE + s, a.status, 180);
          tc_fence_after_sync();
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            const Geo Gm = geometry(gi, (int)p.k_pos0 + T.j0 + t * KT + c0 + 32 * ch, T.len_b);
            const uint32_t tcol = lane_base + T_BUF + s * 128 + c0 + 32 * ch;
            float2 d2 = make_float2(0.f, 0.f);
            uint32_t dpk[16];
            if (Gm.none) {
#pragma unroll
              for (int j = 0; j < 16; ++j) dpk[j] = 0u;
            } else {
              uint32_t rp2[32];
              tmem_ld32(tcol, rp2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 d = make_float2(keep_if_bit(__uint_as_float(rp2[2 * j]), Gm.vis, 2 * j),
                                             keep_if_bit(__uint_as_float(rp2[2 * j + 1]), Gm.vis, 2 * j + 1));
                d2 = add2(d2, d);
                dpk[j] = pack_bf16(d.x, d.y);
              }
            }
            tmem_st16(tcol, dpk);
            sd += d2.x + d2.y;
          }
          tmem_st_wait();
          tc_fence_before_sync();
          warp_arrive(bars + B_DDONE + s, lane);
        }
        G += nt;
        // this tile's staging slot in the main ring: behind Wt half 0 (first tile only), Wt half 1, nt K, 4 KV, nt V
        // and the next tile's Wt half 0
        rp.advance(5 + 2 * nt + (it == 0 ? 1 : 0) + (it + 1 < n_it ? 1 : 0));
        const uint32_t oslot = rp.slot;
        rp.advance();
        ph.wait(bars, B_OUTREADY, a.status, 183);
        // ---- combine the column halves of each row (the two threads of a row meet in the staging slot) ----
        // L + max(Z - dps, c) = max(Z + sum D, L + c), with sum D = L - dps
        float* s_sd = reinterpret_cast<float*>(smem + OFF_RING + oslot * SLOT);   // [2 column halves][128 rows]
        s_sd[cq * 128 + row] = sd;
        asm volatile("bar.sync 3, %0;" ::"n"(32 * WGRP) : "memory");
        ph.wait(bars, B_LZFULL, a.status, 181);
        const float L = s_lz[row] + s_lz[128 + row];
        const float Zrow = s_lz[256 + row] + s_lz[384 + row];
        const float ZD = Zrow + (s_sd[row] + s_sd[128 + row]);
        warp_arrive(bars + B_LZFREE, lane);
        // every thread has read the exchange before any output line is staged over it
        asm volatile("bar.sync 3, %0;" ::"n"(32 * WGRP) : "memory");
        ph.wait(bars, B_DONE, a.status, 182);
        tc_fence_after_sync();
        // The reference clamps Z - dps at 1e-24 in ITS feature units; ours are smaller by the slack of the bound
        // stabilisers, so the constant here is the smallest that still keeps the division finite.
        const float inv = 1.f / fmaxf(ZD, L + 1e-37f);
        // Nothing is ever rescaled: for inputs far above unit-variance logits the exponentials leave the fp32
        // range, or every feature of a row falls under it.  Record either instead of returning it silently.
        if (!(L < 1e30f) || !(fabsf(ZD) < 1e30f) || (Zrow == 0.f && T.len_b > 0)) a.status[1] = 1;
        // Precision: the in-window low-rank estimate (dps = L - sum D) more than 16 times the exact in-window mass L makes
        // D a small difference of large bf16-rounded terms; the row's error is about that ratio times 2^-8.
        if (ZD - Zrow < -15.f * L) a.status[2] = 1;
        // This thread's 64 outputs = one 128-byte line of block cq of the staged tile, laid out as the output
        // tensor map expects: 16-byte chunks XORed with row % 8.
        uint8_t* srow = smem + OFF_RING + oslot * SLOT + cq * 16384 + row * 128;
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t ro[32];
          tmem_ld32(lane_base + T_O + 64 * cq + 32 * hf, ro);
          tmem_ld_wait();
          if (hf == 1) {
            // O has been read: the next tile's first low-rank product may overwrite it
            tc_fence_before_sync();
            warp_arrive(bars + B_OFREE, lane);
          }
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o[j] = pack_bf16(__uint_as_float(ro[2 * j]) * inv, __uint_as_float(ro[2 * j + 1]) * inv);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(srow + (((4 * hf + c) ^ (row & 7)) << 4)) =
                make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        fence_async_smem();
        // every thread of the group has staged its line: one thread stores the tile, which clips rows past the
        // end of the sequence, and releases the slot once the store has read it
        asm volatile("bar.sync 3, %0;" ::"n"(32 * WGRP) : "memory");
        if (gtid == 0) {
          tma_store_4d(&a.tm_out, smem + OFF_RING + oslot * SLOT, 0, T.i0, T.h, T.b);
          tma_store_4d(&a.tm_out, smem + OFF_RING + oslot * SLOT + 16384, 64, T.i0, T.h, T.b);
          tma_store_commit();
          tma_store_wait_read0();
          mbar_arrive(bars + B_EMPTY + oslot);
        }
        __syncwarp();
      }
      if (gtid == 0) tma_store_wait_all();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == W_LOAD) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// feature sums in the internal order (the tensor path has no log-normalisation section)
float* ksum_slots(const Workspace& ws, char* base) { return reinterpret_cast<float*>(base + ws.lognorm); }

bool map_phik128(CUtensorMap* m, const __nv_bfloat16* phik, int S, int BH) {
  const uint64_t dims[3] = {(uint64_t)kM, (uint64_t)S, (uint64_t)BH};
  const uint64_t str[2] = {(uint64_t)kM * 2, (uint64_t)S * kM * 2};
  const uint32_t box[3] = {64, 128, 1};
  return cached_tmap(m, phik, 3, dims, str, box);
}

}  // namespace

bool tc128_shape(const SblParams& p) { return p.E == kE && p.D == kE && p.r == kR; }

cudaError_t tc128_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* beta, float* kv,
                              float* ksum, cudaStream_t st, bool also_bf16) {
  const TcLayout l = tc_layout(ws, base);
  Keys128Args a{};
  if (!map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, kE, p.k_stride_b, p.k_stride_s, p.k_stride_h, 128) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, kE, p.v_stride_b, p.v_stride_s, p.v_stride_h, 128))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 64};      // one block of 64 columns of one projection quarter per load
    if (!cached_tmap(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  if (!map_phik128(&a.tm_phik, l.phik, p.S, p.B * p.H)) return cudaErrorInvalidValue;
  a.lengths = p.key_lengths;
  a.beta = beta;
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
  DeviceInfo* dev = nullptr;
  cudaError_t e = device_info(&dev);
  if (e != cudaSuccess) return e;
  if (!dev->attr_keys128) {
    e = cudaFuncSetAttribute(tc128_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)keys128::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dev->attr_keys128 = true;
  }
  const int bh = p.B * p.H;
  dim3 grid((unsigned)(4 * ws.nsplit), (unsigned)bh);
  tc128_keys_kernel<<<grid, keys128::NTHREADS, keys128::SMEM_BYTES, st>>>(a);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const int64_t n = (int64_t)bh * kM * (kPitch / 4);
  tc128_combine_kernel<<<(unsigned)div_up(n, 256), 256, 0, st>>>(l.partial, ws.nsplit, bh, kv, ksum,
                                                                also_bf16 ? l.kv16 : nullptr, ksum_slots(ws, base));
  return cudaGetLastError();
}

cudaError_t tc128_band(const SblParams& p, const Workspace& ws, char* base, const float* beta, const float* kv,
                       const float* ksum, cudaStream_t st, bool kv16_ready) {
  const TcLayout l = tc_layout(ws, base);
  cudaError_t e = cudaSuccess;
  if (!kv16_ready) {
    const int64_t nkv = (int64_t)p.B * p.H * kM * kE;
    tc128_kv_to_bf16_kernel<<<(unsigned)div_up(nkv, 256), 256, 0, st>>>(kv, l.kv16, nkv, ksum, ksum_slots(ws, base));
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  Band128Args a{};
  if (!map_bthe(&a.tm_q, p.q, p.B, p.T, p.H, kE, p.q_stride_b, p.q_stride_t, p.q_stride_h, 128) ||
      !map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, kE, p.k_stride_b, p.k_stride_s, p.k_stride_h, 128) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, kE, p.v_stride_b, p.v_stride_s, p.v_stride_h, 128) ||
      !map_bthe(&a.tm_out, p.out, p.B, p.T, p.H, kE, p.o_stride_b, p.o_stride_t, p.o_stride_h, 128))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 128};     // one block of 64 columns of one projection half per load
    if (!cached_tmap(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  if (!map_phik128(&a.tm_phik, l.phik, p.S, p.B * p.H)) return cudaErrorInvalidValue;
  {
    const uint64_t dims[3] = {(uint64_t)kE, (uint64_t)kM, (uint64_t)(p.B * p.H)};
    const uint64_t str[2] = {(uint64_t)kE * 2, (uint64_t)kM * kE * 2};
    const uint32_t box[3] = {64, 128, 1};  // 128 features x one block of 64 columns per load
    if (!cached_tmap(&a.tm_kv, l.kv16, 3, dims, str, box)) return cudaErrorInvalidValue;
  }
  a.p = p;
  a.beta = beta;
  a.ksum = ksum_slots(ws, base);
  a.wmax = l.wmax;
  a.status = l.status;
  a.ntq = (int)div_up(p.T, band128::BQ);
  a.ntiles = a.ntq * p.B * p.H;
  DeviceInfo* dev = nullptr;
  if ((e = device_info(&dev)) != cudaSuccess) return e;
  if (!dev->attr_band128) {
    e = cudaFuncSetAttribute(tc128_band_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)band128::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dev->attr_band128 = true;
  }
  // persistent: one CTA per SM (shared and tensor memory allow no more), each walking its share of the query tiles
  const unsigned grid = (unsigned)(a.ntiles < dev->sms ? a.ntiles : dev->sms);
  tc128_band_kernel<<<grid, band128::NTHREADS, band128::SMEM_BYTES, st>>>(a);
  return cudaGetLastError();
}

}  // namespace sbl
