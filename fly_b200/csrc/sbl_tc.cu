// bf16 tensor-core path of the SBLocal forward for sm_100a: TMA tile loads,
// tcgen05.mma with accumulators (and the phi(Q) / packed-weight operands) in
// tensor memory, warp-specialised pipelines with mbarriers whose waits are
// bounded.  Shapes: E = D = 64, r = 128 (m = 256), eps = 0, any T, S, w, key
// lengths (this file), and E = D = 128, r = 256 (m = 512), whose keys and band
// kernels are in sbl_tc128.cu.  Everything else takes the generic kernels of
// sbl_f32.cu.
//
// Kernels
//   prep      sqrt(tau)*W -> bf16 (and fp32), clears the status words (and, for the fused forward, the log-scales)
//   key_bound beta = upper bound of the key log-scale from the key norms (fused forward)
//   keys<MAX> per (split, b*h): streams 128-key tiles; U = K Wt^T on tensor
//             cores; MAX: running max of (|u| - tau|k|^2/2) -> beta (atomic);
//             else phi(K) -> bf16 to the workspace and, MN-major, to shared
//             memory for KV += phi(K)^T [V | 1] (accumulators in tensor memory),
//             then one partial summary per CTA
//   combine   sums the split partials -> KV (fp32, and bf16 for the band kernel), sum phi(K)
//   band      persistent, one CTA per SM walking a run of 128-query tiles.  The
//             projection U = Q Wt^T is computed in two halves of 64 projections,
//             each into a 64-column slot of tensor memory, where the softmax
//             warps turn it IN PLACE into 128 bf16 features (the A operand of
//             every phi(Q) product); three such slots rotate, so the features of
//             the next query tile are formed while the current tile still uses
//             its own.  Per 128-key tile: S = Q K^T into one of two buffers, the
//             softmax warps write E = exp(tau S - pls) (masked to the window and
//             key length) back over S in fp32, the tensor core subtracts
//             P = phi(Q) phi(K)^T from it (same MMA, A operand negated, one
//             product per feature half), the softmax warps pack D = E - P to
//             bf16 over the first half of their own columns, O += D V;
//             O also receives phi(Q) KV; finally out = O / max(Z + sum D, L + 1e-24),
//             staged in shared memory and written by one bulk tensor store per tile.
//   Everything is kept in "feature units" (divided by e^{pls}, pls = query
//   log-scale + beta), so the exact and the low-rank terms share one
//   accumulator and no accumulator is ever rescaled.
//
// Feature order.  Inside this path the 256 features are ordered so that the
// 32 features a softmax thread forms from its 16 projections sit in the 16
// tensor-memory columns it read those projections from: slot
// kp = 128*h + 32*c + 16*s + j holds feature exp((-1)^s u_p ...) of projection
// p = 64*h + 16*c + j (reference index p + 128*s).  phi(K) in the workspace, the
// split partials and the bf16 KV use this order; the fp32 kv / ksum the API
// exchanges with callers use the reference's.
#include <mutex>

#include "sbl_common.cuh"
#include "sbl_tc_dev.cuh"
#include "sbl_tc_host.cuh"

namespace sbl {
namespace tch {

std::mutex g_dev_mu;
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Encoded tensor maps are cached by what they describe: a forward issues eleven of them, and in a serving
// loop over fixed buffers every one repeats.  Small, linear-probed, guarded by a mutex.
struct TmapKey {
  const void* base;
  int rank;
  uint64_t dims[4], strides[3];
  uint32_t box[4];
  bool operator==(const TmapKey& o) const {
    if (base != o.base || rank != o.rank) return false;
    for (int i = 0; i < rank; ++i)
      if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
    for (int i = 0; i + 1 < rank; ++i)
      if (strides[i] != o.strides[i]) return false;
    return true;
  }
};
struct TmapCache {
  static constexpr int N = 64;
  std::mutex mu;
  TmapKey keys[N];
  CUtensorMap maps[N];
  int used = 0, next = 0;
};
TmapCache g_tmaps;

bool cached_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                 const uint32_t* box) {
  TmapKey k{};
  k.base = base;
  k.rank = rank;
  for (int i = 0; i < rank; ++i) {
    k.dims[i] = dims[i];
    k.box[i] = box[i];
    if (i + 1 < rank) k.strides[i] = strides[i];
  }
  std::lock_guard<std::mutex> lock(g_tmaps.mu);
  for (int i = 0; i < g_tmaps.used; ++i)
    if (g_tmaps.keys[i] == k) {
      *out = g_tmaps.maps[i];
      return true;
    }
  if (!encode_tmap_bf16(out, base, rank, dims, strides, box)) return false;
  const int slot = g_tmaps.used < TmapCache::N ? g_tmaps.used++ : (g_tmaps.next++ % TmapCache::N);
  g_tmaps.keys[slot] = k;
  g_tmaps.maps[slot] = *out;
  return true;
}

bool map_bthe(CUtensorMap* m, const void* base, int B, int rows, int H, int E, int64_t sb, int64_t ss, int64_t sh,
              uint32_t box_rows) {
  const uint64_t dims[4] = {(uint64_t)E, (uint64_t)rows, (uint64_t)H, (uint64_t)B};
  // a size-1 axis may carry any stride in torch; give the encoder a legal one
  const uint64_t str[3] = {(uint64_t)ss * 2, (uint64_t)(H > 1 ? sh : E) * 2, (uint64_t)(B > 1 ? sb : E) * 2};
  const uint32_t box[4] = {64, box_rows, 1, 1};
  return cached_tmap(m, base, 4, dims, str, box);
}


DeviceInfo g_dev[64];

cudaError_t device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_dev_mu);
  DeviceInfo& d = g_dev[dev];
  if (d.sms == 0) {
    if ((e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  }
  *out = &d;
  return cudaSuccess;
}


TcLayout tc_layout(const Workspace& ws, char* base) {
  TcLayout l;
  l.wt32 = reinterpret_cast<float*>(base + ws.wt);
  l.wt16 = reinterpret_cast<__nv_bfloat16*>(base + ws.phiq);  // the tensor path has no phi(Q) section
  l.phik = reinterpret_cast<__nv_bfloat16*>(base + ws.phik);
  l.kv16 = reinterpret_cast<__nv_bfloat16*>(base + ws.qls);   // nor query log-scales
  l.partial = reinterpret_cast<float*>(base + ws.partial);
  l.status = reinterpret_cast<int*>(base + ws.status);
  l.wmax = reinterpret_cast<float*>(base + ws.status + 16);
  return l;
}

}  // namespace tch

namespace {

using namespace ptx;
using namespace tcdev;
using namespace tch;

constexpr int kE = 64;    // head dim (qk and v)
constexpr int kR = 128;   // projection rows
constexpr int kM = 256;   // features
constexpr int kPartialLd = 80;   // row pitch (floats) of a split-partial summary: 64 KV columns, the feature sum, padding

// ---------------------------------------------------------------------------
// One block of 1024 threads, 8 per projection row: sqrt(tau)*W in fp32 and bf16, the largest row
// norm of the bf16 copy (bound on |u_f| / |x| used as the query feature stabiliser), status reset.
__global__ void __launch_bounds__(1024) tc_prep_kernel(const float* W, float c, float* wt32, __nv_bfloat16* wt16,
                                                       int r, int E, int* status, float* wmax, int reset_status,
                                                       float* beta_fill, int n_beta) {
  __shared__ float red[32];
  // the fused forward lets this launch also reset the key log-scales (they are formed by atomic max)
  for (int i = threadIdx.x; i < n_beta; i += blockDim.x) beta_fill[i] = -INFINITY;
  float mx = 0.f;
  for (int f0 = 0; f0 < r; f0 += 128) {
    const int f = f0 + threadIdx.x / 8, part = threadIdx.x % 8;
    float s = 0.f;
    if (f < r)
      for (int e = part; e < E; e += 8) {
        const float v = c * W[f * E + e];
        const __nv_bfloat16 b = __float2bfloat16_rn(v);
        wt32[f * E + e] = v;
        wt16[f * E + e] = b;
        const float vb = __bfloat162float(b);
        s = fmaf(vb, vb, s);
      }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    mx = fmaxf(mx, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 32; ++i) mx = fmaxf(mx, red[i]);
    *wmax = sqrtf(mx) * 1.0005f;
  }
  if (reset_status && threadIdx.x < 4) status[threadIdx.x] = 0;
}

// Upper bound on the key log-scale from row norms alone: every feature exponent
// +-u_f - tau|k|^2/2 - ln(m)/2 is at most wmax|k| - tau|k|^2/2 - ln(m)/2 (Cauchy-Schwarz, wmax = largest row norm
// of the scaled projection).  With eps = 0 any stabiliser >= the true maximum gives the same output, so the
// fused forward uses this one-pass, memory-bound bound instead of the exact maximum over all m features.
// LPR lanes per key row (16 bytes each: LPR = E / 8), 16 * 256 / LPR rows per block.
template <int LPR>
__global__ void __launch_bounds__(256) tc_key_bound_kernel(const __nv_bfloat16* k, int64_t sb, int64_t ss, int64_t sh,
                                                           int H, int row_lo, int row_hi, float tau, float half_log_m,
                                                           const float* wmax, float* beta) {
  __shared__ float red[8];
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const __nv_bfloat16* base = k + b * sb + h * sh;
  const float wm = __ldg(wmax);
  constexpr int RPI = 256 / LPR;   // rows per iteration
  const int sub = threadIdx.x % LPR;
  float best = -INFINITY;
  // four rows per thread in flight at a time: the pass is a pure stream over K and one load per thread and
  // iteration leaves it latency-bound
#pragma unroll 1
  for (int it = 0; it < 16; it += 4) {
    uint4 v[4];
    int rows[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      rows[u] = row_lo + blockIdx.x * (16 * RPI) + (it + u) * RPI + threadIdx.x / LPR;
      v[u] = make_uint4(0, 0, 0, 0);
      if (rows[u] < row_hi) v[u] = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)rows[u] * ss) + sub);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float x = bf16_lo(w[j]), y = bf16_hi(w[j]);
        s = fmaf(x, x, s);
        s = fmaf(y, y, s);
      }
#pragma unroll
      for (int o = 1; o < LPR; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (rows[u] < row_hi) best = fmaxf(best, wm * sqrtf(s) - 0.5f * tau * s - half_log_m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) best = fmaxf(best, red[i]);
    if (best > -INFINITY) atomic_max_float(beta + bh, best);
  }
}

// Reference feature index of internal slot kp (see "Feature order" at the top of the file).
__host__ __device__ constexpr int feat_of_slot(int kp) {
  return 64 * (kp >> 7) + 16 * ((kp >> 5) & 3) + (kp & 15) + 128 * ((kp >> 4) & 1);
}

// kv (BH,256,64), ksum (BH,256) = sum over the splits of the per-CTA partial summaries.  The partials and
// kv16 (the band kernel's bf16 operand) are in the internal feature order, kv and ksum in the reference's.
__global__ void tc_combine_kernel(const float* partial, int nsplit, int BH, float* kv, float* ksum,
                                  __nv_bfloat16* kv16) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // over BH * 256 * 20 float4 groups
  if (i >= (int64_t)BH * kM * (kPartialLd / 4)) return;
  const int g = (int)(i % (kPartialLd / 4));
  const int64_t bf = i / (kPartialLd / 4);        // bh * 256 + slot
  if (g > 16) return;
  const int64_t bh = bf / kM;
  const int kp = (int)(bf % kM);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < nsplit; ++k) {
    const float4 v = *reinterpret_cast<const float4*>(partial + ((bh * nsplit + k) * kM + kp) * kPartialLd + 4 * g);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const int64_t out_row = bh * kM + feat_of_slot(kp);
  if (g < 16) {
    *reinterpret_cast<float4*>(kv + out_row * kE + 4 * g) = acc;
    if (kv16) {   // the band kernel's bf16 operand, when the caller goes straight on to the band stage
      const uint2 h = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
      *reinterpret_cast<uint2*>(kv16 + bf * kE + 4 * g) = h;
    }
  } else {
    ksum[out_row] = acc.x;
  }
}

// kv (BH,256,64) fp32 in the reference's feature order -> bf16 in the internal order
__global__ void tc_kv_to_bf16_kernel(const float* kv, __nv_bfloat16* kv16, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // over output elements
  if (i >= n) return;
  const int d = (int)(i % kE);
  const int64_t row = i / kE;
  const int64_t bh = row / kM;
  const int kp = (int)(row % kM);
  kv16[i] = __float2bfloat16_rn(kv[(bh * kM + feat_of_slot(kp)) * kE + d]);
}

// ---------------------------------------------------------------------------

// keys kernel
struct KeysArgs {
  CUtensorMap tm_k, tm_v, tm_w, tm_phik;
  const int64_t* lengths;
  const float* beta_in;   // !MAX
  float* beta_out;        // MAX
  __nv_bfloat16* phik;    // (BH, S, 256), internal feature order
  float* partial;         // (BH, nsplit, 256, 80)
  int* status;
  int S, H, sum_lo, sum_hi, nsplit;
  int64_t k_pos0, S_total;
  float tau, half_log_m;
};

namespace keys {
constexpr int TILE = 128;
constexpr int NFQ = 4;                     // projection groups per key row: a feature thread owns 128/NFQ projections
constexpr int NFEAT = 128 * NFQ;           // feature threads: warp w owns key rows 32*(w%4).., projection group w/4
constexpr int CHK = 4 / NFQ;               // 32-projection chunks per thread
constexpr int WPK = NFEAT / 32;            // producer warp; WPK+1: MMA warp
constexpr int NTHREADS = NFEAT + 64;
constexpr uint32_t OFF_W = 0;                    // 16 KB  [128 r][64 e]
constexpr uint32_t OFF_K = 16384;                // ring of [128 keys][64 e] tiles, 16 KB each: 2 deep (4 deep in the beta pass)
constexpr uint32_t OFF_V = 49152;                // 2 x 16 KB V tiles; [V | 1] is one MN-major operand (N = 80) whose second
constexpr uint32_t OFF_ONES = OFF_V + 32768;     // 64-column block is this 16 KB block of ones (leading offset per V slot)
constexpr uint32_t OFF_A = OFF_ONES + 16384;     // 2 x 64 KB: 4 blocks [128 keys][64 f] = phi(K) tile, MN-major A operand
constexpr uint32_t OFF_BAR = OFF_A + 2 * 65536;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 512 + 1024;    // + alignment slack
// tensor memory columns
constexpr uint32_t T_UK = 0;      // 2 x 128
constexpr uint32_t T_KV = 256;    // 2 x 128 (80 used): [KV (64) | sum phi(K) (16 identical columns)] for feature blocks 0-127, 128-255
}  // namespace keys

template <bool MAX_ONLY>
__global__ void __launch_bounds__(keys::NTHREADS) tc_keys_kernel(const __grid_constant__ KeysArgs a) {
  using namespace keys;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* bar_w = bars + 0;
  uint64_t* bar_done = bars + 1;
  uint64_t* v_full = bars + 2;    // [2] V tile landed
  uint64_t* v_empty = bars + 22;  // [2] V tile consumed by the summary MMAs
  uint64_t* k_full = bars + 4;    // [KD] K tile landed
  uint64_t* k_free = bars + 8;    // [KD] K tile consumed: U computed and every row norm read
  uint64_t* uk_full = bars + 12;  // [2] U = K Wt^T computed
  uint64_t* uk_free = bars + 14;  // [2] U read by all feature threads
  uint64_t* a_full = bars + 16;   // [2] phi(K) tile written to shared memory
  uint64_t* a_free = bars + 18;   // [2] phi(K) tile consumed (MMAs done + bulk store has read it)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  float* red = reinterpret_cast<float*>(bars + 24);  // [NFEAT / 32]
  constexpr int KD = MAX_ONLY ? 4 : 2;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int ntiles = (a.S + TILE - 1) / TILE;
  const int split = blockIdx.x;
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
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(k_full + i, 1);
      mbar_init(k_free + i, NFEAT / 32);   // one arrival per feature warp
    }
    for (int i = 0; i < 2; ++i) {
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
  if (!MAX_ONLY)
    for (int i = tid; i < 8192; i += NTHREADS)   // the "ones" block behind the V tile (16 KB of bf16 1.0)
      reinterpret_cast<__nv_bfloat16*>(smem + OFF_ONES)[i] = __float2bfloat16(1.0f);
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  constexpr uint32_t tb = 0;   // the CTA owns all 512 tensor-memory columns of its SM
  if (tid == 0 && *tmem_slot != 0) atomicCAS(a.status, 0, 41);

  // a tile whose rows all enter the summary and hold real keys is stored to the workspace by one bulk copy
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
      tma_load_2d(smem + OFF_W, &a.tm_w, bar_w, 0, 0);
    }
    for (int i = 0; i < nt; ++i) {
      const int ks = i % KD;
      const int row0 = (t_lo + i) * TILE;
      if (i >= KD) mbar_wait(k_free + ks, ((i / KD) - 1) & 1, a.status, 11);
      if (leader) {
        mbar_expect_tx(k_full + ks, 16384);
        tma_load_4d(smem + OFF_K + ks * 16384, &a.tm_k, k_full + ks, 0, row0, h, b);
      }
      if (!MAX_ONLY) {
        const int s = i & 1;
        if (i >= 2) mbar_wait(v_empty + s, ((i >> 1) - 1) & 1, a.status, 11);
        if (leader) {
          mbar_expect_tx(v_full + s, 16384);
          tma_load_4d(smem + OFF_V + s * 16384, &a.tm_v, v_full + s, 0, row0, h, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == WPK + 1) {
    // ---------------- MMA issuer ----------------
    const bool leader = elect_one();
    constexpr uint32_t id_uk = idesc_bf16(128, 128, false, false);
    constexpr uint32_t id_kv = idesc_bf16(128, 80, true, true);
    const uint64_t dW = smem_desc_sw128(smem_u32(smem + OFF_W), 16, 1024);
    const uint64_t dA0 = smem_desc_sw128(smem_u32(smem + OFF_A), 16384, 1024);
    const uint64_t dK0 = smem_desc_sw128(smem_u32(smem + OFF_K), 16, 1024);
    // second MN block of [V | 1] = the ones block: 32 KB behind V slot 0, 16 KB behind V slot 1
    const uint64_t dV0 = smem_desc_sw128(smem_u32(smem + OFF_V), 32768, 1024);
    const uint64_t dV1 = smem_desc_sw128(smem_u32(smem + OFF_V + 16384), 16384, 1024);
    auto issue_kv = [&](int u) {
      const int s = u & 1;
      mbar_wait(a_full + s, (u >> 1) & 1, a.status, 12);
      mbar_wait(v_full + s, (u >> 1) & 1, a.status, 14);
      tc_fence_after_sync();
      if (leader) {
        // bulk copy of the phi(K) tile to the workspace (an empty group keeps the group count uniform)
        if (tile_is_plain(u)) {
          const int row0 = (t_lo + u) * TILE;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            tma_store_3d(&a.tm_phik, smem + OFF_A + s * 65536 + j * 16384, j * 64, row0, bh);
        }
        tma_store_commit();
        const uint64_t dA = dA0 + (uint64_t)(s * (65536 >> 4));
        const uint64_t dV = s ? dV1 : dV0;
#pragma unroll
        for (int mb = 0; mb < 2; ++mb)
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ss(tb + T_KV + mb * 128, dA + (uint64_t)(mb * (32768 >> 4) + k * (2048 >> 4)),
                   dV + (uint64_t)(k * (2048 >> 4)), id_kv, (u > 0) || (k > 0));
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
    mbar_wait(bar_w, 0, a.status, 13);
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      mbar_wait(k_full + (i % KD), (i / KD) & 1, a.status, 14);
      if (i >= 2) mbar_wait(uk_free + s, ((i >> 1) - 1) & 1, a.status, 15);
      tc_fence_after_sync();
      if (leader) {
        const uint32_t td = tb + T_UK + s * 128;
        const uint64_t dK = dK0 + (uint64_t)((i % KD) * (16384 >> 4));
        mma_ss(td, dK, dW, id_uk, false);
        mma_ss(td, dK + 2, dW + 2, id_uk, true);
        mma_ss(td, dK + 4, dW + 4, id_uk, true);
        mma_ss(td, dK + 6, dW + 6, id_uk, true);
        mma_commit(uk_full + s);
      }
      __syncwarp();
      if (!MAX_ONLY && i >= 1) issue_kv(i - 1);
    }
    if (!MAX_ONLY && nt > 0) issue_kv(nt - 1);
    if (leader) {
      mma_commit(bar_done);
      if (!MAX_ONLY) tma_store_wait_all();
    }
    __syncwarp();
  } else {
    // ---------------- feature warps ----------------
    const int qd = warp & 3, cq = warp >> 2;
    constexpr int PWK = 128 / NFQ;                   // projections owned by this thread
    const int krow = qd * 32 + lane;                 // key row inside the tile
    const uint32_t lane_base = tb + ((uint32_t)(qd * 32) << 16);
    const float beta = MAX_ONLY ? 0.f : a.beta_in[bh];
    float run_max = -INFINITY;
    for (int i = 0; i < nt; ++i) {
      const int s = i & 1;
      const int row = (t_lo + i) * TILE + krow;
      mbar_wait(k_full + (i % KD), (i / KD) & 1, a.status, 19);
      const float g = 0.5f * a.tau * row_sumsq_sw128(smem + OFF_K + (i % KD) * 16384, krow);
      mbar_wait(uk_full + s, (i >> 1) & 1, a.status, 16);   // U computed: the tensor core is done with the K tile too
      tc_fence_after_sync();
      warp_arrive(k_free + (i % KD), lane);
      if (MAX_ONLY) {
        float mx = 0.f;
#pragma unroll
        for (int c = 0; c < CHK; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_base + T_UK + s * 128 + PWK * cq + 32 * c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, fabsf(__uint_as_float(r[j])));
        }
        if (row >= a.sum_lo && row < a.sum_hi) run_max = fmaxf(run_max, (mx - g) - a.half_log_m);
        tc_fence_before_sync();
        warp_arrive(uk_free + s, lane);
      } else {
        const bool live = row < a.S && (a.k_pos0 + row) < len_b;
        const bool in_sum = live && row >= a.sum_lo && row < a.sum_hi;
        const bool plain = tile_is_plain(i);
        const float off = ((-g - a.half_log_m) - beta) * kLog2e;
        __nv_bfloat16* grow = a.phik + ((int64_t)bh * a.S + row) * kM;
        uint8_t* sA = smem + OFF_A + s * 65536;
#pragma unroll
        for (int c = 0; c < CHK; ++c) {
          const int f0 = PWK * cq + 32 * c;          // first projection of this chunk
          uint32_t r[32];
          tmem_ld32(lane_base + T_UK + s * 128 + f0, r);
          tmem_ld_wait();
          uint32_t p1[16], p2[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            constexpr float2 lp = {kLog2e, kLog2e}, lm = {-kLog2e, -kLog2e};
            const float2 u = make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            const float2 ap = fma2(u, lp, make_float2(off, off)), am = fma2(u, lm, make_float2(off, off));
            const float2 ep = make_float2(ex2(ap.x), ex2(ap.y));
            const float2 em = make_float2(ex2(am.x), ex2(am.y));
            p1[j] = live ? pack_bf16(ep.x, ep.y) : 0u;
            p2[j] = live ? pack_bf16(em.x, em.y) : 0u;
          }
          // A chunk of 32 projections fills one 64-feature block of the internal order: per group of 16
          // projections (gi) two 16-byte pieces of the "+" features, then two of the "-" features.
          const int blk = f0 >> 5;
          if (!plain && row < a.S) {
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
              const uint32_t* src = ((q8 >> 1) & 1) ? p2 : p1;
              const int o = 8 * (q8 >> 2) + 4 * (q8 & 1);
              reinterpret_cast<uint4*>(grow + 64 * blk)[q8] = make_uint4(src[o], src[o + 1], src[o + 2], src[o + 3]);
            }
          }
          // the previous tile's MMAs and bulk store must be done with the shared phi(K) buffer
          if (c == 0 && i >= 2) mbar_wait(a_free + s, ((i >> 1) - 1) & 1, a.status, 17);
          // MN-major A operand: block = 64 features, 16-byte piece q8 of the key's 128-byte line, swizzled by key % 8
#pragma unroll
          for (int q8 = 0; q8 < 8; ++q8) {
            const uint32_t* src = ((q8 >> 1) & 1) ? p2 : p1;
            const int o = 8 * (q8 >> 2) + 4 * (q8 & 1);
            const uint32_t so = (uint32_t)krow * 128u + (uint32_t)((q8 ^ (krow & 7)) << 4);
            *reinterpret_cast<uint4*>(sA + blk * 16384 + so) =
                in_sum ? make_uint4(src[o], src[o + 1], src[o + 2], src[o + 3]) : make_uint4(0, 0, 0, 0);
          }
        }
        fence_async_smem();
        tc_fence_before_sync();
        warp_arrive(a_full + s, lane);
        warp_arrive(uk_free + s, lane);
      }
    }
    if (MAX_ONLY) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) run_max = fmaxf(run_max, __shfl_xor_sync(0xffffffffu, run_max, o));
      if (lane == 0) red[warp] = run_max;
      asm volatile("bar.sync 1, %0;" ::"n"(NFEAT) : "memory");
      if (tid == 0) {
        float v = red[0];
        for (int i = 1; i < NFEAT / 32; ++i) v = fmaxf(v, red[i]);
        if (v > -INFINITY) atomic_max_float(a.beta_out + bh, v);
      }
    } else {
      mbar_wait(bar_done, 0, a.status, 18);
      tc_fence_after_sync();
      // thread (feature row, group): writes 64/NFQ of the row's KV columns; the last group also the feature sum
      constexpr int CW = 64 / NFQ;
      float* part = a.partial + ((int64_t)bh * a.nsplit + split) * kM * kPartialLd;
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
        float* prow = part + (int64_t)(mb * 128 + krow) * kPartialLd;
        uint32_t q[16];
        tmem_ld16(lane_base + T_KV + mb * 128 + 64, q);
#pragma unroll
        for (int gq = 0; gq < CW / 16; ++gq) {
          uint32_t r[16];
          tmem_ld16(lane_base + T_KV + mb * 128 + CW * cq + 16 * gq, r);
          tmem_ld_wait();
          if (nt == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(prow + CW * cq + 16 * gq)[j] =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        tmem_ld_wait();
        if (cq == NFQ - 1) prow[64] = nt == 0 ? 0.f : __uint_as_float(q[0]);
      }
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
struct BandArgs {
  CUtensorMap tm_q, tm_k, tm_v, tm_w, tm_phik, tm_kv, tm_out;
  SblParams p;
  const float* beta;
  const float* ksum;     // (BH, 256) fp32, reference feature order
  const float* wmax;     // [1]: max_f |sqrt(tau) w_f| of the bf16 projection
  int* status;
  int ntq;               // query tiles per (b,h)
  int ntiles;            // ntq * B * H
};

namespace band {
constexpr int BQ = 128, KT = 128;
constexpr int NSOFT = 512;                 // softmax threads: two groups of 256, warp w owns rows 32*(w%4)..
constexpr int WSOFT = NSOFT / 32;          // softmax warps
constexpr int WGRP = WSOFT / 2;            // warps per softmax group (exponential group, packing group)
constexpr int W_LOADKV = WSOFT;            // producer: K, V, phi(K) tiles; output stores
constexpr int W_LOADQ = WSOFT + 1;         // producer: Q tiles, halves of Wt, halves of KV
constexpr int W_MMA_A = WSOFT + 2;         // MMA issuer: U halves, S
constexpr int W_MMA_B = WSOFT + 3;         // MMA issuer: P
constexpr int W_MMA_C = WSOFT + 4;         // MMA issuer: low-rank, O
constexpr int NTHREADS = NSOFT + 160;
constexpr uint32_t OFF_Q = 0;              // 2 x 16 KB [128 q][64 e]: current and next query tile
constexpr uint32_t OFF_W = 32768;          // 8 KB [64 r][64 e]: one half of Wt at a time
constexpr uint32_t OFF_KVH = 40960;        // 16 KB [128 f][64 d]: one feature half of KV at a time
constexpr uint32_t OFF_K = 57344;          // 16 KB [128 keys][64 e]
constexpr uint32_t OFF_V = OFF_K + 16384;  // 16 KB [128 keys][64 d]; also the staging buffer of the output tile
constexpr uint32_t OFF_PK = OFF_V + 16384; // 2 x 64 KB: phi(K) tiles, each 4 blocks [128 keys][64 f]
constexpr uint32_t OFF_MISC = OFF_PK + 2 * 65536;    // ksum fp32[256] + (L, Z) exchange fp32[2][2][256] + sum D fp32[2][256]
constexpr uint32_t OFF_BAR = OFF_MISC + 1024 + 12 * NSOFT;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 512 + 1024;
static_assert(SMEM_BYTES <= 232448, "dynamic shared memory of one CTA");
// tensor memory columns (512): three 64-column feature-half slots, two 128-column S/E/D buffers, O
__device__ __forceinline__ constexpr uint32_t hq_col(int slot) { return slot == 0 ? 0u : (slot == 1 ? 64u : 384u); }
constexpr uint32_t T_BUF = 128;    // 2 x 128: S of a key tile, then E, then D = E - P (fp32), then D packed bf16 in place
constexpr uint32_t T_O = 448;      // 64
// barrier indices
enum {
  B_QFULL = 0,                    // [2] Q tile landed                                   (by query tile parity)
  B_QFREE = B_QFULL + 2,          // [2] Q buffer reusable: last MMA reading it + one arrival per softmax warp
  B_WFULL = B_QFREE + 2,          // half of Wt landed                                   (per load)
  B_WFREE,                        // U half computed: the Wt buffer is reusable
  B_KVFULL,                       // half of KV landed                                   (per load)
  B_KVFREE,                       // low-rank product done with it
  B_UQFULL,                       // [3] U half computed into the slot
  B_PHIFULL = B_UQFULL + 3,       // [3] features formed in the slot (one arrival per softmax warp)
  B_HQFREE = B_PHIFULL + 3,       // [3] slot reusable: issuer A (low-rank) and issuer B (last P) both done
  B_KFULL = B_HQFREE + 3, B_KEMPTY, B_VFULL, B_VEMPTY,   // per key tile, single buffers
  B_PKFULL, B_PKEMPTY = B_PKFULL + 2,                    // [2] per key tile, by ring slot
  B_SFULL = B_PKEMPTY + 2,        // [2] by buffer
  B_ADONE = B_SFULL + 2,          // [2] one arrival per softmax warp
  B_PFULL = B_ADONE + 2,          // [2]
  B_BDONE = B_PFULL + 2,          // [2] one arrival per softmax warp
  B_BUFFREE = B_BDONE + 2,        // [2] O += D V done: the buffer may take the next S
  B_OFREE = B_BUFFREE + 2,        // O read by the epilogue (one arrival per softmax warp)
  B_DONE,                         // all MMAs of the query tile done
  B_OFULL,                        // output tile staged in shared memory (one arrival per softmax warp)
  B_OSTORED,                      // the bulk store of the staged tile has read the staging buffer
  B_LZFULL,                       // [2] L and Z of a query tile published by the exponential group (by tile parity)
  B_XFREE = B_LZFULL + 2,         // [2] ... and read by the packing group
  B_COUNT = B_XFREE + 2
};
static_assert(B_COUNT <= 60, "barriers and the tensor-memory slot share 512 bytes");
}  // namespace band

// Geometry of one 128-query tile: which key tiles it visits.
struct BandTile {
  int bh, b, h, i0, nq, len_b, j0, nt;
};
// A CTA walks consecutive tiles: (b*h, query tile) advance without dividing by the tile count.
struct TileCursor {
  int bh, qt;
  __device__ TileCursor(const BandArgs& a, int tile_id) : bh(tile_id / a.ntq), qt(tile_id % a.ntq) {}
  __device__ void next(const BandArgs& a) {
    if (++qt == a.ntq) {
      qt = 0;
      ++bh;
    }
  }
};
// Not inlined: every warp role needs it once per tile, and the kernel's instruction footprint is what limits it.
__device__ __noinline__ BandTile band_tile(const BandArgs& a, const TileCursor& c) {
  const SblParams& p = a.p;
  BandTile t;
  t.bh = c.bh;
  t.b = t.bh / p.H;
  t.h = t.bh - t.b * p.H;
  t.i0 = c.qt * band::BQ;
  t.nq = min(band::BQ, p.T - t.i0);
  t.len_b = (int)(p.key_lengths ? min(p.key_lengths[t.b], p.S_total) : p.S_total);
  const int hw = p.w / 2;
  // key buffer rows any query of this tile can see, clipped to the buffer and to the key length
  int lo = (int)(p.q_pos0 + t.i0 - hw - p.k_pos0);
  int hi = (int)(p.q_pos0 + t.i0 + t.nq - 1 - hw + p.w - 1 - p.k_pos0);
  lo = max(lo, 0);
  hi = min(hi, min(p.S - 1, t.len_b - 1 - (int)p.k_pos0));
  t.j0 = (lo / band::KT) * band::KT;
  t.nt = hi >= lo ? (hi - t.j0) / band::KT + 1 : 0;
  return t;
}

// Which phi(K) tile each of the two shared-memory slots holds.  Key tile kt of a (b,h) lives in slot
// kt & 1; consecutive query tiles of a run share two of their three key tiles, so only the new one is
// loaded.  The producer and the P-issuing warp walk the same sequence and keep identical copies.
struct PkTrack {
  int bh0 = -1, bh1 = -1, kt0 = -1, kt1 = -1;
  int fills0 = 0, fills1 = 0;   // completed or pending loads per slot
  int uses0 = 0, uses1 = 0;     // P products issued (or planned) per slot
  __device__ bool resident(int slot, int b, int k) const {
    return slot ? (bh1 == b && kt1 == k) : (bh0 == b && kt0 == k);
  }
  __device__ int fills(int slot) const { return slot ? fills1 : fills0; }
  __device__ int uses(int slot) const { return slot ? uses1 : uses0; }
  __device__ void filled(int slot, int b, int k) {
    if (slot) { bh1 = b; kt1 = k; ++fills1; } else { bh0 = b; kt0 = k; ++fills0; }
  }
  __device__ void used(int slot) {
    if (slot) ++uses1; else ++uses0;
  }
};

// Persistent: CTA c processes a run of consecutive query tiles.  Key tiles are numbered per CTA
// (g = 0, 1, ... across query tiles) and key tile g uses buffer g & 1; feature half h of the run's
// query tile `it` uses slot (2 it + h) % 3, use number (2 it + h) / 3 of that slot.  Both halves of
// tile it + 1 are formed while tile it is processed: half 0 in the slot tile it does not use, half 1
// in the slot of tile it's half 0 as soon as the last P product has read that.
__global__ void __launch_bounds__(band::NTHREADS, 1) tc_band_kernel(const __grid_constant__ BandArgs a) {
  using namespace band;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 62);
  float* s_ksum = reinterpret_cast<float*>(smem + OFF_MISC);   // [256], internal feature order
  float* s_lz = s_ksum + kM;        // [2 tile parities][L, Z][2 column halves][128 rows]
  float* s_sd = s_lz + 1024;        // [2 tile parities][2 column halves][128 rows]

  const SblParams& p = a.p;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hw = p.w / 2;
  // this CTA's run of consecutive query tiles: neighbours in a run share two of their three key tiles
  const int tile_lo = (int)((int64_t)a.ntiles * blockIdx.x / gridDim.x);
  const int n_it = (int)((int64_t)a.ntiles * (blockIdx.x + 1) / gridDim.x) - tile_lo;

  if (warp == W_MMA_A) {
    for (int i = lane; i < B_COUNT; i += 32) {
      const bool group = (i >= B_PHIFULL && i < B_PHIFULL + 3) || (i >= B_ADONE && i < B_ADONE + 2) ||
                         (i >= B_BDONE && i < B_BDONE + 2) || i == B_OFREE || i == B_OFULL ||
                         (i >= B_LZFULL && i < B_LZFULL + 2) || (i >= B_XFREE && i < B_XFREE + 2);
      int count = 1;
      if (group) count = WGRP;                                   // the warps of one softmax group arrive once per warp
      if (i >= B_QFREE && i < B_QFREE + 2) count = WGRP + 1;
      if (i >= B_HQFREE && i < B_HQFREE + 3) count = 2;
      mbar_init(bars + i, count);
    }
    fence_mbar_init();
  }
  if (warp == W_LOADKV) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // The CTA owns all 512 columns of its SM's tensor memory, so the allocation starts at
  // column 0; keeping the base a compile-time constant keeps every MMA operand uniform.
  constexpr uint32_t tb = 0;
  if (tid == 0 && *tmem_slot != 0) atomicCAS(a.status, 0, 40);

  if (warp == W_LOADKV) {
    // ---------------- producer 1: K, phi(K), V tiles, output stores (whole warp waits, one lane issues) ------
    const bool leader = elect_one();
    if (leader) {
      prefetch_tmap(&a.tm_k);
      prefetch_tmap(&a.tm_v);
      prefetch_tmap(&a.tm_phik);
      prefetch_tmap(&a.tm_out);
    }
    int gk = 0;   // key tiles loaded so far
    PkTrack pk;
    TileCursor cur_n(a, tile_lo);
    // The softmax warps stage a finished output tile in the V buffer (free once the tile's last O += D V has
    // run); one bulk store writes it out.  The next V load waits until the store has read the buffer.
    int o_i0 = 0, o_h = 0, o_b = 0;
    auto store_out = [&](int it2) {
      mbar_wait(bars + B_OFULL, it2 & 1, a.status, 45);
      if (leader) {
        tma_store_4d(&a.tm_out, smem + OFF_V, 0, o_i0, o_h, o_b);
        tma_store_commit();
        tma_store_wait_read0();
        mbar_arrive(bars + B_OSTORED);
      }
      __syncwarp();
    };
    BandTile T = band_tile(a, cur_n), Tn{};
    bool k0_done = false;     // K and phi(K) of this tile's first key tile were already loaded during the previous tile
    for (int it = 0; it < n_it; ++it) {
      cur_n.next(a);
      const bool have_next = it + 1 < n_it;
      if (have_next) Tn = band_tile(a, cur_n);
      // K and V are single-buffered, phi(K) double-buffered.  Issue order follows the order in which the tensor
      // core frees the buffers: K(g), phi(K)(g), then V(g-1); the first key tile of the NEXT query tile goes
      // ahead of this tile's last V, because the next tile's first S is issued that early.
      auto load_v = [&](int t) {
        const int g = gk + t;
        if (g >= 1) mbar_wait(bars + B_VEMPTY, (g - 1) & 1, a.status, 23);
        if (leader) {
          mbar_expect_tx(bars + B_VFULL, 16384);
          tma_load_4d(smem + OFF_V, &a.tm_v, bars + B_VFULL, 0, T.j0 + t * KT, T.h, T.b);
        }
      };
      auto load_k = [&](const BandTile& Tx, int t, int g) {
        const int row0 = Tx.j0 + t * KT;
        if (g >= 1) mbar_wait(bars + B_KEMPTY, (g - 1) & 1, a.status, 21);
        if (leader) {
          mbar_expect_tx(bars + B_KFULL, 16384);
          tma_load_4d(smem + OFF_K, &a.tm_k, bars + B_KFULL, 0, row0, Tx.h, Tx.b);
        }
        const int kt = row0 / KT, ps = kt & 1;
        if (!pk.resident(ps, Tx.bh, kt)) {
          // every P that read the slot's old tile must be done: wait for the latest of them
          if (pk.uses(ps) >= 1) mbar_wait(bars + B_PKEMPTY + ps, (pk.uses(ps) - 1) & 1, a.status, 22);
          if (leader) {
            mbar_expect_tx(bars + B_PKFULL + ps, 65536);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tma_load_3d(smem + OFF_PK + ps * 65536 + j * 16384, &a.tm_phik, bars + B_PKFULL + ps, j * 64, row0,
                          Tx.bh);
          }
          pk.filled(ps, Tx.bh, kt);
        }
        pk.used(ps);
      };
      // The last key tile of a query tile is the one no earlier tile of the run has touched, and its V is
      // loaded last, behind a single buffer: start pulling it into L2 now.
      if (leader && T.nt >= 2) tma_prefetch_4d(&a.tm_v, 0, T.j0 + (T.nt - 1) * KT, T.h, T.b);
      // Steps 0 .. nt: step t < nt loads K(t) (unless done) and then V(t-1), with the previous tile's output store
      // ahead of V(0); step nt loads the next tile's first K and this tile's last V.
#pragma unroll 1
      for (int t = 0; t <= T.nt; ++t) {
        if (t < T.nt) {
          if (!(t == 0 && k0_done)) load_k(T, t, gk + t);
        } else if (have_next && Tn.nt > 0) {
          load_k(Tn, 0, gk + T.nt);
        }
        // V(0) is not needed before the first O += D V; its buffer holds the previous tile's staged output
        // until that tile's epilogue, which must not hold up the K tile S(1) is waiting for
        if (t == 1 || (t == 0 && T.nt == 0)) {
          if (it >= 1) store_out(it - 1);
        }
        if (t >= 1) load_v(t - 1);
      }
      k0_done = have_next && Tn.nt > 0;
      o_i0 = T.i0;
      o_h = T.h;
      o_b = T.b;
      gk += T.nt;
      T = Tn;
    }
    store_out(n_it - 1);
    if (leader) tma_store_wait_all();
    __syncwarp();
  } else if (warp == W_LOADQ) {
    // ---------------- producer 2: Q tiles, halves of Wt, halves of KV ----------------
    // Load order = the order in which issuer A consumes them; every wait below is released by an MMA group
    // that issuer A reaches without needing a later load of this warp.
    const bool leader = elect_one();
    if (leader) {
      prefetch_tmap(&a.tm_q);
      prefetch_tmap(&a.tm_w);
      prefetch_tmap(&a.tm_kv);
    }
    // Per run tile `it` (it = -1 stands for "before the run"), in this order:
    //   0: Wt half 0 for U(it+1, 0)     1: KV half 1 for the low-rank product (it, 1)     2: Wt half 1 for U(it+1, 1)
    //   3: Q of tile it+2               4: KV half 0 for the low-rank product (it+1, 0)
    // plus Q of the first tile up front.  One loop, one copy of each load.
    TileCursor c1(a, tile_lo), c2(a, tile_lo);   // cursors of tiles it + 1 and it + 2
    c2.next(a);
    {
      const BandTile T0 = band_tile(a, c1);
      if (leader) {
        mbar_expect_tx(bars + B_QFULL, 16384);
        tma_load_4d(smem + OFF_Q, &a.tm_q, bars + B_QFULL, 0, T0.i0, T0.h, T0.b);
      }
    }
    int bh_cur = 0;
#pragma unroll 1
    for (int it = -1; it < n_it; ++it) {
      const bool have_next = it + 1 < n_it;
      const int bh_next = c1.bh;
#pragma unroll 1
      for (int step = 0; step < 5; ++step) {
        if (step == 0 || step == 2) {
          const int idx = 2 * it + 2 + (step >> 1);       // Wt load number = 2 * run tile + half
          if (!have_next) continue;
          if (idx >= 1) mbar_wait(bars + B_WFREE, (idx - 1) & 1, a.status, 50);
          if (leader) {
            mbar_expect_tx(bars + B_WFULL, 8192);
            tma_load_2d(smem + OFF_W, &a.tm_w, bars + B_WFULL, 0, 64 * (idx & 1));
          }
        } else if (step == 1 || step == 4) {
          const int idx = step == 1 ? 2 * it + 1 : 2 * it + 2;   // KV load number = 2 * run tile + half
          if (step == 1 ? it < 0 : !have_next) continue;
          if (idx >= 1) mbar_wait(bars + B_KVFREE, (idx - 1) & 1, a.status, 51);
          if (leader) {
            mbar_expect_tx(bars + B_KVFULL, 16384);
            tma_load_3d(smem + OFF_KVH, &a.tm_kv, bars + B_KVFULL, 0, 128 * (idx & 1), step == 1 ? bh_cur : bh_next);
          }
        } else {
          if (it + 2 >= n_it) continue;
          const BandTile T2 = band_tile(a, c2);
          if (it >= 0) mbar_wait(bars + B_QFREE + (it & 1), (it >> 1) & 1, a.status, 20);
          if (leader) {
            mbar_expect_tx(bars + B_QFULL + (it & 1), 16384);
            tma_load_4d(smem + OFF_Q + (it & 1) * 16384, &a.tm_q, bars + B_QFULL + (it & 1), 0, T2.i0, T2.h, T2.b);
          }
        }
      }
      bh_cur = bh_next;
      c1.next(a);
      c2.next(a);
    }
    __syncwarp();
  } else if (warp == W_MMA_A || warp == W_MMA_C) {
    // ---------------- MMA issuers A (U halves, S) and C (low-rank, O): whole warp waits, one lane issues ----------
    // Two warps, because one warp issues a group of 4-8 MMAs with its waits and commits in about a thousand
    // cycles and a query tile has eleven such groups besides the six of issuer B.  The order of a tile's groups
    // is written into a short op list first and then executed by a loop with a single copy of every group's
    // code (shared by both warps): the kernel is limited by instruction fetch as much as by anything else.
    const bool role_a = warp == W_MMA_A;
    const bool leader = elect_one();
    constexpr uint32_t id_s = idesc_bf16(128, 128, false, false);
    constexpr uint32_t id_u = idesc_bf16(128, 64, false, false);
    constexpr uint32_t id_o = idesc_bf16(128, 64, false, true);
    const uint64_t dQ0 = smem_desc_sw128(smem_u32(smem + OFF_Q), 16, 1024);
    const uint64_t dW = smem_desc_sw128(smem_u32(smem + OFF_W), 16, 1024);
    const uint64_t dKVH = smem_desc_sw128(smem_u32(smem + OFF_KVH), 16, 1024);
    const uint64_t dK0 = smem_desc_sw128(smem_u32(smem + OFF_K), 16, 1024);
    const uint64_t dV0 = smem_desc_sw128(smem_u32(smem + OFF_V), 16, 1024);
    enum { OP_S = 0, OP_U, OP_LR, OP_O, OP_QFREE, OP_DONE };
    // op word: kind | x << 4 (key tile g, or run tile) | y << 28 (Q buffer / feature half) | flag << 30
    auto mk = [](int kind, int x, int y, bool flag) {
      return (uint32_t)kind | ((uint32_t)x << 4) | ((uint32_t)y << 28) | ((uint32_t)flag << 30);
    };
    uint32_t ops[24];
    TileCursor cur_n(a, tile_lo);
    int gk = 0, nt_carry = 0;
    bool s0_issued = false;   // S(0) of the coming tile was issued during the previous tile
    // it = -1: the two projection halves of the run's first tile
    for (int it = -1; it < n_it; ++it) {
      int n = 0;
      const bool have_next = it + 1 < n_it;
      const int nt = nt_carry;
      int nt_n = 0;
      if (have_next) nt_n = band_tile(a, cur_n).nt;
      nt_carry = nt_n;
      const int qb = it & 1;
      if (role_a) {
        if (it < 0) {
          ops[n++] = mk(OP_U, 0, 0, true);                   // flag: wait for the tile's Q first
          ops[n++] = mk(OP_U, 0, 1, false);
          if (nt_n == 0) ops[n++] = mk(OP_QFREE, 0, 0, false);
        } else {
          if (nt > 0 && !s0_issued) ops[n++] = mk(OP_S, gk, qb, nt == 1);
          if (nt > 1) ops[n++] = mk(OP_S, gk + 1, qb, nt == 2);
          s0_issued = false;
          if (have_next) ops[n++] = mk(OP_U, it + 1, 0, true);
          // S(t+2) as soon as O += D(t) V has released its buffer; S(0) of the next tile the same way: the
          // exponential warps start that tile with it
          for (int t = 0; t + 2 < nt; ++t) ops[n++] = mk(OP_S, gk + t + 2, qb, t + 3 == nt);
          if (have_next && nt_n > 0) {
            ops[n++] = mk(OP_S, gk + nt, qb ^ 1, nt_n == 1);
            s0_issued = true;
          }
          // second feature half of the next tile: its slot is released by this tile's last P over half 0
          if (have_next) {
            ops[n++] = mk(OP_U, it + 1, 1, false);
            if (nt_n == 0) ops[n++] = mk(OP_QFREE, 0, qb ^ 1, false);
          }
        }
      } else if (it >= 0) {
        ops[n++] = mk(OP_LR, it, 0, false);
        // the second low-rank half goes ahead of the last O += D V, which waits longest
        for (int t = 0; t < nt; ++t) {
          if (t == nt - 1) ops[n++] = mk(OP_LR, it, 1, false);
          ops[n++] = mk(OP_O, gk + t, 0, false);
        }
        if (nt == 0) ops[n++] = mk(OP_LR, it, 1, false);
        ops[n++] = mk(OP_DONE, 0, 0, false);
      }
#pragma unroll 1
      for (int i = 0; i < n; ++i) {
        const uint32_t op = ops[i];
        const int kind = op & 15, x = (op >> 4) & 0xFFFFFF, y = (op >> 28) & 3;
        const bool flag = (op >> 30) & 1;
        if (kind == OP_S) {
          // S of key tile g = x (query tile in Q buffer y); flag: no later MMA reads that Q buffer
          const int g = x;
          mbar_wait(bars + B_KFULL, g & 1, a.status, 25);
          if (g >= 2) mbar_wait(bars + B_BUFFREE + (g & 1), ((g - 2) >> 1) & 1, a.status, 28);
          tc_fence_after_sync();
          if (leader) {
            const uint32_t td = tb + T_BUF + (g & 1) * 128;
            const uint64_t dQ = dQ0 + (uint64_t)(y * (16384 >> 4));
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_ss(td, dQ + 2 * k, dK0 + 2 * k, id_s, k > 0);
            mma_commit(bars + B_KEMPTY);
            mma_commit(bars + B_SFULL + (g & 1));
            if (flag) mma_commit(bars + B_QFREE + y);
          }
        } else if (kind == OP_U) {
          // U half y of run tile x into its slot
          const int idx = 2 * x + y, s = idx % 3, u = idx / 3;
          if (flag) mbar_wait(bars + B_QFULL + (x & 1), (x >> 1) & 1, a.status, 30);
          if (u >= 1) mbar_wait(bars + B_HQFREE + s, (u - 1) & 1, a.status, 52);
          mbar_wait(bars + B_WFULL, idx & 1, a.status, 53);
          tc_fence_after_sync();
          if (leader) {
            const uint32_t td = tb + hq_col(s);
            const uint64_t dQ = dQ0 + (uint64_t)((x & 1) * (16384 >> 4));
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_ss(td, dQ + 2 * k, dW + 2 * k, id_u, k > 0);
            mma_commit(bars + B_UQFULL + s);
            mma_commit(bars + B_WFREE);
          }
        } else if (kind == OP_LR) {
          // O (+)= phi(Q)[half y] KV[half y] of run tile x; half 0 comes first in a tile and initialises O
          const int idx = 2 * x + y, s = idx % 3, u = idx / 3;
          mbar_wait(bars + B_PHIFULL + s, u & 1, a.status, 31);
          mbar_wait(bars + B_KVFULL, idx & 1, a.status, 32);
          if (y == 0 && x >= 1) mbar_wait(bars + B_OFREE, (x - 1) & 1, a.status, 54);
          tc_fence_after_sync();
          if (leader) {
            const uint32_t ta = tb + hq_col(s);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              mma_ts(tb + T_O, ta + k * 8, dKVH + (uint64_t)(k * (2048 >> 4)), id_o, y != 0 || k > 0);
            mma_commit(bars + B_KVFREE);
            mma_commit(bars + B_HQFREE + s);
          }
        } else if (kind == OP_O) {
          // O += D V: D packed bf16 sits in the first 16 of every 32 columns of the buffer
          const int g = x;
          mbar_wait(bars + B_BDONE + (g & 1), (g >> 1) & 1, a.status, 29);
          mbar_wait(bars + B_VFULL, g & 1, a.status, 29);
          tc_fence_after_sync();
          if (leader) {
            const uint32_t ta = tb + T_BUF + (g & 1) * 128;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              mma_ts(tb + T_O, ta + 32 * (k >> 1) + 8 * (k & 1), dV0 + (uint64_t)(k * (2048 >> 4)), id_o, true);
            mma_commit(bars + B_VEMPTY);
            mma_commit(bars + B_BUFFREE + (g & 1));
          }
        } else if (kind == OP_QFREE) {
          if (leader) mma_commit(bars + B_QFREE + y);
        } else {
          if (leader) mma_commit(bars + B_DONE);
        }
        __syncwarp();
      }
      gk += nt;
      cur_n.next(a);
    }
  } else if (warp == W_MMA_B) {
    // ---------------- MMA issuer B: buffer(g) -= phi(Q) phi(K)^T, one product per feature half ----------------
    // The buffer holds E = exp(tau S - pls) written back by the softmax warps; the product is accumulated
    // with the A operand negated, which leaves D = E - P in fp32.
    // (its own warp, on another scheduler than issuer A: the two issue streams run in parallel)
    const bool leader = elect_one();
    constexpr uint32_t id_neg = idesc_bf16(128, 128, false, false) | (1u << 13);   // bit 13: negate A
    const uint64_t dPK0 = smem_desc_sw128(smem_u32(smem + OFF_PK), 16, 1024);
    int gk = 0;
    PkTrack pk;
    TileCursor cur(a, tile_lo);
    for (int it = 0; it < n_it; ++it, cur.next(a)) {
      const BandTile T = band_tile(a, cur);
      const int s0 = (2 * it) % 3, u0 = (2 * it) / 3, s1 = (2 * it + 1) % 3, u1 = (2 * it + 1) / 3;
      if (T.nt == 0) {
        // nothing to multiply: release both slots, but only once their features exist, so that this warp
        // can never be a whole use of a slot ahead of issuer A
        mbar_wait(bars + B_PHIFULL + s0, u0 & 1, a.status, 39);
        mbar_wait(bars + B_PHIFULL + s1, u1 & 1, a.status, 39);
        if (leader) {
          mbar_arrive(bars + B_HQFREE + s0);
          mbar_arrive(bars + B_HQFREE + s1);
        }
        __syncwarp();
        continue;
      }
      for (int t = 0; t < T.nt; ++t) {
        const int g = gk + t, s = g & 1;
        const int kt = T.j0 / KT + t, ps = kt & 1;
        const bool last = t == T.nt - 1;
        mbar_wait(bars + B_ADONE + s, (g >> 1) & 1, a.status, 26);
        if (!pk.resident(ps, T.bh, kt)) {   // a tile still resident from the previous query tile was waited for then
          mbar_wait(bars + B_PKFULL + ps, pk.fills(ps) & 1, a.status, 27);
          pk.filled(ps, T.bh, kt);
        }
        pk.used(ps);
        if (t == 0) mbar_wait(bars + B_PHIFULL + s0, u0 & 1, a.status, 39);
        tc_fence_after_sync();
        const uint64_t dPK = dPK0 + (uint64_t)(ps * (65536 >> 4));
        const uint32_t td = tb + T_BUF + s * 128;
        if (leader) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ts(td, tb + hq_col(s0) + k * 8, dPK + (uint64_t)((k >> 2) * (16384 >> 4) + (k & 3) * 2), id_neg, true);
          if (last) mma_commit(bars + B_HQFREE + s0);
        }
        __syncwarp();
        if (t == 0) {
          mbar_wait(bars + B_PHIFULL + s1, u1 & 1, a.status, 39);
          tc_fence_after_sync();
        }
        if (leader) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mma_ts(td, tb + hq_col(s1) + k * 8, dPK + (uint64_t)((2 + (k >> 2)) * (16384 >> 4) + (k & 3) * 2), id_neg,
                   true);
          if (last) mma_commit(bars + B_HQFREE + s1);
          mma_commit(bars + B_PKEMPTY + ps);
          mma_commit(bars + B_PFULL + s);
        }
        __syncwarp();
      }
      gk += T.nt;
    }
  } else {
    // ---------------- softmax warps: two groups that work on different phases at the same time ----------------
    // Exponential group (warps 0-7): E = exp(tau S - pls) of every key tile, the features of the query tiles, the
    //   row sums L and Z.  Its work is bound by the special-function unit.
    // Packing group (warps 8-15): D = E - P -> bf16 for every key tile, the row sum of D, the epilogue.  Its work
    //   is integer / conversion work and tensor-memory traffic, which runs beside the other group's exponentials.
    // A thread of either group owns one query row and 64 key columns of every key tile (two chunks of 32).
    const int qd = warp & 3, cq = (warp >> 2) & 1;   // lane quarter (rows), column half
    const bool exp_group = warp < WGRP;
    const int row = qd * 32 + lane;                  // query row of this thread
    const int gtid = tid & (32 * WGRP - 1);          // thread index inside the group
    const uint32_t lane_base = tb + ((uint32_t)(qd * 32) << 16);
    const int c0 = 64 * cq;                          // first key column (of every key tile) of this thread
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
    if (exp_group) {
      const float wmax = __ldg(a.wmax);
      const float half_log_m = 0.5f * logf((float)kM);
      const float sc = p.softmax_temp * kLog2e;
      int bh_smem = -1;
      // Row norm, stabiliser and key log-scale of run tile itx (its Q tile must be on its way), and the
      // summary row of its (b,h): gq = tau |q|^2 / 2, M = wmax |q| >= |u_f| for every projection (Cauchy-Schwarz).
      // Both threads of a row sum the whole row: no exchange is needed.
      auto prep_tile = [&](int itx, const BandTile& Tx, float& M, float& gq) {
        if (Tx.bh != bh_smem) {
          // every warp of the group is done with the old summary row before it is replaced
          asm volatile("bar.sync 2, %0;" ::"n"(32 * WGRP) : "memory");
          s_ksum[gtid] = __ldg(a.ksum + (int64_t)Tx.bh * kM + feat_of_slot(gtid));
          asm volatile("bar.sync 2, %0;" ::"n"(32 * WGRP) : "memory");
          bh_smem = Tx.bh;
        }
        mbar_wait(bars + B_QFULL + (itx & 1), (itx >> 1) & 1, a.status, 33);
        const float qn2 = row_sumsq_sw128(smem + OFF_Q + (itx & 1) * 16384, row);
        warp_arrive(bars + B_QFREE + (itx & 1), lane);
        gq = 0.5f * p.softmax_temp * qn2;
        M = sqrtf(qn2) * wmax;
      };
      // Features of one half, in place: this thread's 32 projections (two groups of 16 fp32 columns) become, per
      // group, 16 "+" and 16 "-" features (2 x 8 packed columns); z accumulates phi(Q) . sum phi(K) over them.
      auto form_half = [&](int itx, int half, float M) {
        const int idx = 2 * itx + half, s = idx % 3, u = idx / 3;
        mbar_wait(bars + B_UQFULL + s, u & 1, a.status, 34);
        tc_fence_after_sync();
        const float mo = -M * kLog2e;
        const float2 mo2 = make_float2(mo, mo);
        const float2 lp = make_float2(kLog2e, kLog2e), lm = make_float2(-kLog2e, -kLog2e);
        float2 zz = make_float2(0.f, 0.f);
#pragma unroll 1
        for (int g2 = 0; g2 < 2; ++g2) {
          const int c = 2 * cq + g2;               // group of 16 projections inside the half
          const uint32_t taddr = lane_base + hq_col(s) + 16 * c;
          const float* ks = s_ksum + 128 * half + 32 * c;
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
            zz = fma2(ep, *reinterpret_cast<const float2*>(ks + 2 * j), zz);
            zz = fma2(em, *reinterpret_cast<const float2*>(ks + 16 + 2 * j), zz);
          }
          tmem_st8(taddr, p1);
          tmem_st8(taddr + 8, p2);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        warp_arrive(bars + B_PHIFULL + s, lane);
        return zz.x + zz.y;
      };

      int gk = 0;
      TileCursor cur_n(a, tile_lo);
      BandTile T_carry{};
      float M_c = 0.f, gq_c = 0.f, beta_c = 0.f, z_c = 0.f;   // current tile: stabiliser, tau |q|^2 / 2, key log-scale, Z share
      float M_n = 0.f, gq_n = 0.f, beta_n = 0.f, z_n = 0.f;   // the same for the next tile
      // Tile it = -1 stands for "before the run": it only prepares the first tile.  Every phase below has a
      // single call site (the kernel is limited by instruction fetch; nothing is instantiated twice).
      for (int it = -1; it < n_it; ++it) {
        const BandTile T = T_carry;
        const int nt = T.nt;
        const bool have_next = it + 1 < n_it;
        // geometry and key log-scale of the next tile: fetched now, needed after the second key tile
        BandTile Tn{};
        if (have_next) {
          Tn = band_tile(a, cur_n);
          beta_n = __ldg(a.beta + Tn.bh);
        }
        T_carry = Tn;
        const int gi = (int)p.q_pos0 + T.i0 + row;     // global query position
        const float pls = (-gq_c + M_c - half_log_m) + beta_c;         // query log-scale + key log-scale
        const float2 sc2 = make_float2(sc, sc);
        const float2 co2 = make_float2(-pls * kLog2e, -pls * kLog2e);  // exp(tau s - pls) = ex2(s * sc + co)
        float L = 0.f;             // row sum of the exponentials over this thread's columns
        const int nsteps = nt > 2 ? nt : 2;
#pragma unroll 1
        for (int t = 0; t < nsteps; ++t) {
          if (t < nt) {
            // S(t) -> E = exp(tau S - pls) in place (fp32), zero outside the window; row sum
            const int gg = gk + t, s = gg & 1;
            mbar_wait(bars + B_SFULL + s, (gg >> 1) & 1, a.status, 35);
            tc_fence_after_sync();
#pragma unroll 1
            for (int ch = 0; ch < 2; ++ch) {
              const Geo G = geometry(gi, (int)p.k_pos0 + T.j0 + t * KT + c0 + 32 * ch, T.len_b);
              if (G.none) continue;   // a chunk nobody sees is left as it is: the packing group writes zeros for it
              const uint32_t tcol = lane_base + T_BUF + s * 128 + c0 + 32 * ch;
              uint32_t rs[32];
              tmem_ld32(tcol, rs);
              tmem_ld_wait();
              float2 l2 = make_float2(0.f, 0.f);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 x =
                    fma2(make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1])), sc2, co2);
                float2 e = make_float2(0.f, 0.f);
                if (G.vis & (1u << (2 * j))) e.x = ex2(x.x);          // predicated: hidden columns cost no exponential
                if (G.vis & (2u << (2 * j))) e.y = ex2(x.y);
                l2 = add2(l2, e);
                rs[2 * j] = __float_as_uint(e.x);
                rs[2 * j + 1] = __float_as_uint(e.y);
              }
              tmem_st32(tcol, rs);
              L += l2.x + l2.y;
            }
            tmem_st_wait();
            tc_fence_before_sync();
            warp_arrive(bars + B_ADONE + s, lane);
          }
          // Feature halves: after the first key tile the second half of THIS tile (its slot was released late in the
          // previous tile), after the second key tile the first half of the NEXT tile (its slot is free all along)
          const bool form_cur = t == 0 && it >= 0, form_next = t == 1 && have_next;
          if (form_cur || form_next) {
            if (form_next) {
              prep_tile(it + 1, Tn, M_n, gq_n);
              z_n = 0.f;
            }
            const float zadd = form_half(form_next ? it + 1 : it, form_next ? 0 : 1, form_next ? M_n : M_c);
            if (form_next) z_n += zadd; else z_c += zadd;
          }
        }
        if (it >= 0) {
          // hand L and Z of this tile to the packing group (double-buffered by tile parity)
          if (it >= 2) mbar_wait(bars + B_XFREE + (it & 1), ((it >> 1) - 1) & 1, a.status, 47);
          s_lz[(it & 1) * 512 + cq * 128 + row] = L;
          s_lz[(it & 1) * 512 + 256 + cq * 128 + row] = z_c;
          warp_arrive(bars + B_LZFULL + (it & 1), lane);
          gk += nt;
        }
        cur_n.next(a);
        M_c = M_n;
        gq_c = gq_n;
        beta_c = beta_n;
        z_c = z_n;
      }
    } else {
      int gk = 0;
      TileCursor cur(a, tile_lo);
      for (int it = 0; it < n_it; ++it, cur.next(a)) {
        const BandTile T = band_tile(a, cur);
        const int nt = T.nt;
        const int gi = (int)p.q_pos0 + T.i0 + row;
        float sd = 0.f;            // row sum of D = E - P over this thread's columns
        for (int t = 0; t < nt; ++t) {
          // D(t) = E - P (fp32, left by the tensor core) -> masked, packed bf16 over the first 16 of every 32
          // columns of this thread
          const int gg = gk + t, s = gg & 1;
          mbar_wait(bars + B_PFULL + s, (gg >> 1) & 1, a.status, 36);
          tc_fence_after_sync();
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            const Geo G = geometry(gi, (int)p.k_pos0 + T.j0 + t * KT + c0 + 32 * ch, T.len_b);
            const uint32_t tcol = lane_base + T_BUF + s * 128 + c0 + 32 * ch;
            float2 d2 = make_float2(0.f, 0.f);
            uint32_t dpk[16];
            if (G.none) {
#pragma unroll
              for (int j = 0; j < 16; ++j) dpk[j] = 0u;
            } else {
              uint32_t rp[32];
              tmem_ld32(tcol, rp);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 d = make_float2(keep_if_bit(__uint_as_float(rp[2 * j]), G.vis, 2 * j),
                                             keep_if_bit(__uint_as_float(rp[2 * j + 1]), G.vis, 2 * j + 1));
                d2 = add2(d2, d);
                dpk[j] = pack_bf16(d.x, d.y);
              }
            }
            tmem_st16(tcol, dpk);
            sd += d2.x + d2.y;
          }
          tmem_st_wait();
          tc_fence_before_sync();
          warp_arrive(bars + B_BDONE + s, lane);
        }
        // ---- combine the column halves of each row ----
        // L + max(Z - dps, c) = max(Z + sum D, L + c), with sum D = L - dps
        s_sd[(it & 1) * 256 + cq * 128 + row] = sd;
        asm volatile("bar.sync 3, %0;" ::"n"(32 * WGRP) : "memory");
        mbar_wait(bars + B_LZFULL + (it & 1), (it >> 1) & 1, a.status, 48);
        const float* lz = s_lz + (it & 1) * 512;
        const float L = lz[row] + lz[128 + row];
        const float Zrow = lz[256 + row] + lz[384 + row];
        const float ZD = Zrow + (s_sd[(it & 1) * 256 + row] + s_sd[(it & 1) * 256 + 128 + row]);
        warp_arrive(bars + B_XFREE + (it & 1), lane);
        // ---- epilogue: this thread writes half of the row's 64 outputs ----
        mbar_wait(bars + B_DONE, it & 1, a.status, 38);
        tc_fence_after_sync();
        // The reference clamps Z - dps at 1e-24 in ITS feature units; ours are smaller by the slack of the bound
        // stabilisers (e^-5 ... e^-50), so the constant here is the smallest that still keeps the division finite.
        const float inv = 1.f / fmaxf(ZD, L + 1e-37f);
        // Nothing here is ever rescaled, so for inputs far above unit-variance logits the exponentials leave the
        // fp32 range (queries and keys ~15 times the unit scale), or every feature of a row falls under it (the
        // bound stabilisers' slack grows with the norms): record either instead of returning it silently.
        if (!(L < 1e30f) || !(fabsf(ZD) < 1e30f) || (Zrow == 0.f && T.len_b > 0)) a.status[1] = 1;
        // Precision, not range: where the in-window low-rank estimate (dps = L - sum D) is more than 16 times the exact
        // in-window mass L, D = E - P is a small difference of large bf16-rounded terms and the row's error is about
        // that ratio times 2^-8 (inputs 3-4 times the unit logit scale do this to a few rows).  Report it.
        if (ZD - Zrow < -15.f * L) a.status[2] = 1;
        {
          // tensor-memory loads are warp-wide: every lane runs them
          uint32_t ro[32];
          tmem_ld32(lane_base + T_O + 32 * cq, ro);
          tmem_ld_wait();
          // O has been read: the next tile's first low-rank product may overwrite it
          tc_fence_before_sync();
          warp_arrive(bars + B_OFREE, lane);
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o[j] = pack_bf16(__uint_as_float(ro[2 * j]) * inv, __uint_as_float(ro[2 * j + 1]) * inv);
          // Stage the 64 bytes of this thread in the V buffer (the tile's last O += D V has run), laid out as
          // the output tensor map expects: 128-byte rows, 16-byte chunks XORed with row % 8.  The producer
          // warp writes the tile out with one bulk store, which clips rows past the end of the sequence.
          // (With key tiles, the V load this tile's products waited for was issued behind the previous tile's
          // store; without any, wait for that store here.)
          if (nt == 0 && it >= 1) mbar_wait(bars + B_OSTORED, (it - 1) & 1, a.status, 46);
          uint8_t* srow = smem + OFF_V + row * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(srow + (((4 * cq + c) ^ (row & 7)) << 4)) =
                make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
          fence_async_smem();
          warp_arrive(bars + B_OFULL, lane);
        }
        gk += nt;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == W_LOADKV) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------
// host side
bool map_phik(CUtensorMap* m, const __nv_bfloat16* phik, int S, int BH) {
  const uint64_t dims[3] = {(uint64_t)kM, (uint64_t)S, (uint64_t)BH};
  const uint64_t str[2] = {(uint64_t)kM * 2, (uint64_t)S * kM * 2};
  const uint32_t box[3] = {64, 128, 1};
  return cached_tmap(m, phik, 3, dims, str, box);
}

template <bool MAX_ONLY>
cudaError_t launch_keys(const SblParams& p, const Workspace& ws, char* base, const float* beta_in, float* beta_out,
                        cudaStream_t st) {
  const TcLayout l = tc_layout(ws, base);
  KeysArgs a{};
  if (!map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, kE, p.k_stride_b, p.k_stride_s, p.k_stride_h, 128) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, kE, p.v_stride_b, p.v_stride_s, p.v_stride_h, 128))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 128};
    if (!cached_tmap(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  if (!map_phik(&a.tm_phik, l.phik, p.S, p.B * p.H)) return cudaErrorInvalidValue;
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
  DeviceInfo* dev = nullptr;
  cudaError_t e = device_info(&dev);
  if (e != cudaSuccess) return e;
  if (!dev->attr_keys[MAX_ONLY ? 1 : 0]) {
    e = cudaFuncSetAttribute(tc_keys_kernel<MAX_ONLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)keys::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dev->attr_keys[MAX_ONLY ? 1 : 0] = true;
  }
  dim3 grid((unsigned)ws.nsplit, (unsigned)(p.B * p.H));
  tc_keys_kernel<MAX_ONLY><<<grid, keys::NTHREADS, keys::SMEM_BYTES, st>>>(a);
  return cudaGetLastError();
}

__global__ void tc_fill_kernel(float* p, float v, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

}  // namespace

bool tc_supported(const SblParams& p) {
  const bool shape64 = p.E == kE && p.D == kE && p.r == kR;
  if (p.dtype != SBL_DTYPE_BF16 || !(shape64 || tc128_shape(p))) return false;
  // the d = 64 band kernel writes a query tile's MMA groups into a fixed list (one entry per key tile and a
  // few more): windows that span more than 18 key tiles take the generic kernels
  if (shape64 && p.w > 2048) return false;
  if (p.softmax_eps != 0.f) return false;
  const int64_t strides[] = {p.q_stride_b, p.q_stride_t, p.q_stride_h, p.k_stride_b, p.k_stride_s, p.k_stride_h,
                             p.v_stride_b, p.v_stride_s, p.v_stride_h, p.o_stride_b, p.o_stride_t, p.o_stride_h};
  for (int64_t s : strides)
    if (s % 8 != 0 || s < 0) return false;
  if (p.q_stride_t < p.E || p.k_stride_s < p.E || p.v_stride_s < p.E || p.o_stride_t < p.E) return false;
  if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.out)) return false;
  if (p.S_total >= (1ll << 30) || p.q_pos0 + p.T >= (1ll << 30)) return false;
  return true;
}

cudaError_t tc_prepare_projection(const SblParams& p, const Workspace& ws, char* base, cudaStream_t st,
                                  bool reset_status, float* beta_fill) {
  const TcLayout l = tc_layout(ws, base);
  tc_prep_kernel<<<1, 1024, 0, st>>>(p.W, (float)sqrt((double)p.softmax_temp), l.wt32, l.wt16, p.r, p.E, l.status,
                                    l.wmax, reset_status ? 1 : 0, beta_fill, beta_fill ? p.B * p.H : 0);
  return cudaGetLastError();
}

cudaError_t tc_key_logscale(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st) {
  // head dim 128 has no exact-maximum pass: the one-pass bound is a valid stabiliser too (eps = 0)
  if (tc128_shape(p)) return tc_key_logscale_bound(p, ws, base, beta, st, false);
  const int bh = p.B * p.H;
  tc_fill_kernel<<<(unsigned)div_up(bh, 256), 256, 0, st>>>(beta, -INFINITY, bh);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_keys<true>(p, ws, base, nullptr, beta, st);
}

cudaError_t tc_key_logscale_bound(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st,
                                  bool beta_is_reset) {
  const TcLayout l = tc_layout(ws, base);
  const int bh = p.B * p.H;
  if (!beta_is_reset) {
    tc_fill_kernel<<<(unsigned)div_up(bh, 256), 256, 0, st>>>(beta, -INFINITY, bh);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  const int rows = p.sum_hi - p.sum_lo;
  if (rows <= 0) return cudaSuccess;
  const float half_log_m = (float)(log(2.0 * p.r) / 2.0);
  if (p.E == 128) {
    dim3 grid((unsigned)div_up(rows, 256), (unsigned)bh);
    tc_key_bound_kernel<16><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(p.k), p.k_stride_b,
                                                 p.k_stride_s, p.k_stride_h, p.H, p.sum_lo, p.sum_hi, p.softmax_temp,
                                                 half_log_m, l.wmax, beta);
  } else {
    dim3 grid((unsigned)div_up(rows, 512), (unsigned)bh);
    tc_key_bound_kernel<8><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(p.k), p.k_stride_b,
                                                p.k_stride_s, p.k_stride_h, p.H, p.sum_lo, p.sum_hi, p.softmax_temp,
                                                half_log_m, l.wmax, beta);
  }
  return cudaGetLastError();
}

cudaError_t tc_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* beta, float* kv,
                           float* ksum, cudaStream_t st, bool also_bf16) {
  if (tc128_shape(p)) return tc128_key_summary(p, ws, base, beta, kv, ksum, st, also_bf16);
  cudaError_t e = launch_keys<false>(p, ws, base, beta, nullptr, st);
  if (e != cudaSuccess) return e;
  const int bh = p.B * p.H;
  const int64_t n = (int64_t)bh * kM * (kPartialLd / 4);
  const TcLayout l = tc_layout(ws, base);
  tc_combine_kernel<<<(unsigned)div_up(n, 256), 256, 0, st>>>(l.partial, ws.nsplit, bh, kv, ksum,
                                                             also_bf16 ? l.kv16 : nullptr);
  return cudaGetLastError();
}

cudaError_t tc_band(const SblParams& p, const Workspace& ws, char* base, const float* beta, const float* kv,
                    const float* ksum, cudaStream_t st, bool kv16_ready) {
  if (tc128_shape(p)) return tc128_band(p, ws, base, beta, kv, ksum, st, kv16_ready);
  const TcLayout l = tc_layout(ws, base);
  cudaError_t e = cudaSuccess;
  if (!kv16_ready) {
    const int64_t nkv = (int64_t)p.B * p.H * kM * kE;
    tc_kv_to_bf16_kernel<<<(unsigned)div_up(nkv, 256), 256, 0, st>>>(kv, l.kv16, nkv);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  BandArgs a{};
  if (!map_bthe(&a.tm_q, p.q, p.B, p.T, p.H, kE, p.q_stride_b, p.q_stride_t, p.q_stride_h, 128) ||
      !map_bthe(&a.tm_k, p.k, p.B, p.S, p.H, kE, p.k_stride_b, p.k_stride_s, p.k_stride_h, 128) ||
      !map_bthe(&a.tm_v, p.v, p.B, p.S, p.H, kE, p.v_stride_b, p.v_stride_s, p.v_stride_h, 128) ||
      !map_bthe(&a.tm_out, p.out, p.B, p.T, p.H, kE, p.o_stride_b, p.o_stride_t, p.o_stride_h, 128))
    return cudaErrorInvalidValue;
  {
    const uint64_t dims[2] = {(uint64_t)kE, (uint64_t)kR};
    const uint64_t str[1] = {(uint64_t)kE * 2};
    const uint32_t box[2] = {64, 64};      // one half of the projection rows per load
    if (!cached_tmap(&a.tm_w, l.wt16, 2, dims, str, box)) return cudaErrorInvalidValue;
  }
  if (!map_phik(&a.tm_phik, l.phik, p.S, p.B * p.H)) return cudaErrorInvalidValue;
  {
    const uint64_t dims[3] = {(uint64_t)kE, (uint64_t)kM, (uint64_t)(p.B * p.H)};
    const uint64_t str[2] = {(uint64_t)kE * 2, (uint64_t)kM * kE * 2};
    const uint32_t box[3] = {64, 128, 1};  // one feature half per load
    if (!cached_tmap(&a.tm_kv, l.kv16, 3, dims, str, box)) return cudaErrorInvalidValue;
  }
  a.p = p;
  a.beta = beta;
  a.ksum = ksum;
  a.wmax = l.wmax;
  a.status = l.status;
  a.ntq = (int)div_up(p.T, band::BQ);
  a.ntiles = a.ntq * p.B * p.H;
  DeviceInfo* dev = nullptr;
  if ((e = device_info(&dev)) != cudaSuccess) return e;
  if (!dev->attr_band) {
    e = cudaFuncSetAttribute(tc_band_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)band::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    dev->attr_band = true;
  }
  // persistent: one CTA per SM (shared and tensor memory allow no more), each walking its share of the query tiles
  const unsigned grid = (unsigned)(a.ntiles < dev->sms ? a.ntiles : dev->sms);
  tc_band_kernel<<<grid, band::NTHREADS, band::SMEM_BYTES, st>>>(a);
  return cudaGetLastError();
}

// One warp waits on a barrier that nothing arrives on: the bounded wait must run out, record its site and
// let the kernel end normally (used to check the mechanism every other device-side wait relies on).
__global__ void tc_wait_selftest_kernel(int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    *status = 0;
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
  }
  __syncwarp();
  ptx::mbar_wait(&bar, 0, status, 99);
}

cudaError_t tc_wait_selftest(int* device_status, int* host_status, cudaStream_t st) {
  tc_wait_selftest_kernel<<<1, 32, 0, st>>>(device_status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(host_status, device_status, sizeof(int), cudaMemcpyDeviceToHost, st)) != cudaSuccess) return e;
  return cudaStreamSynchronize(st);
}

cudaError_t tc_read_status(const Workspace& ws, char* base, int* host_status, cudaStream_t st) {
  cudaError_t e = cudaMemcpyAsync(host_status, base + ws.status, 3 * sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return e;
  return cudaStreamSynchronize(st);
}

}  // namespace sbl
