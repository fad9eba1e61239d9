// Generic SIMT kernels of the SBLocal forward: any E, D, r, w, T != S, ragged
// key lengths, eps != 0; fp32 arithmetic on CUDA cores with fp32 or bf16
// storage.  This is the path that meets the 1e-4 bound against the fp32
// reference, and the one odd shapes fall to.  Intermediates phi(Q) and phi(K)
// live in the workspace in fp32, as (B*H, rows, m) row-major.
//
// All matrix products are register-tiled 64x64 block tiles (4x4 per thread,
// 256 threads) fed from shared memory in K-slices of 16 with the next slice
// prefetched into registers.
#include "sbl_common.cuh"

namespace sbl {
namespace {

constexpr int TILE = 64;       // block tile edge
constexpr int KS = 16;         // K slice
constexpr int LDT = TILE + 4;  // shared leading dimension (keeps float4 rows 16-byte aligned)
constexpr int NTHR = 256;
constexpr int PER_THR = TILE * KS / NTHR;  // slice elements per thread = 4

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float x) { *p = x; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// atomic max on a float through its ordered integer image
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// Fetches this thread's share of a TILE x KS slice (rows of a row-major
// matrix, K-contiguous) into registers; out-of-range elements read as 0.
template <typename T>
__device__ __forceinline__ void fetch_slice(float (&reg)[PER_THR], const T* base, int64_t ld, int nrows,
                                            int k0, int K) {
#pragma unroll
  for (int i = 0; i < PER_THR; ++i) {
    const int idx = threadIdx.x + i * NTHR;
    const int row = idx / KS, kk = idx % KS;
    reg[i] = (row < nrows && k0 + kk < K) ? ldf(base + (int64_t)row * ld + k0 + kk) : 0.f;
  }
}
__device__ __forceinline__ void stash_slice(float (*s)[LDT], const float (&reg)[PER_THR]) {
#pragma unroll
  for (int i = 0; i < PER_THR; ++i) {
    const int idx = threadIdx.x + i * NTHR;
    s[idx % KS][idx / KS] = reg[i];
  }
}

// acc(64x64) += A(64 x K) * B(64 x K)^T, both operands K-contiguous in global
// memory.  Thread (ty,tx) owns rows ty*4.., cols tx*4...
template <typename TA, typename TB>
__device__ __forceinline__ void tile_nt(float (&acc)[4][4], const TA* A, int64_t lda, int na, const TB* B,
                                        int64_t ldb, int nb, int K, float (*sA)[LDT], float (*sB)[LDT]) {
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  float ra[PER_THR], rb[PER_THR];
  fetch_slice(ra, A, lda, na, 0, K);
  fetch_slice(rb, B, ldb, nb, 0, K);
  for (int k0 = 0; k0 < K; k0 += KS) {
    __syncthreads();
    stash_slice(sA, ra);
    stash_slice(sB, rb);
    __syncthreads();
    if (k0 + KS < K) {
      fetch_slice(ra, A, lda, na, k0 + KS, K);
      fetch_slice(rb, B, ldb, nb, k0 + KS, K);
    }
    // two-level sum: one partial per K slice, so the rounding error grows with K/16, not K
    // (the feature dimension can be tens of thousands)
    float part[4][4] = {};
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      const float4 a = *reinterpret_cast<const float4*>(&sA[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&sB[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], bv[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
  }
}

__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------
// sqrt(tau) * W  (feature_maps_sb.py:62-64: the projection is scaled before
// the contraction)
__global__ void scale_projection_kernel(const float* W, float c, float* Wt, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Wt[i] = c * W[i];
}

__global__ void fill_kernel(float* p, float v, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// ---------------------------------------------------------------------------
// Feature map (feature_maps_sb.py:51-82).  One block = 64 rows of one (b,h).
enum { MODE_QUERY = 0, MODE_KEYMAX = 1, MODE_KEY = 2 };

struct FeatArgs {
  const void* x;
  int64_t sb, ss, sh;
  int rows, H, E, r;
  const float* Wt;
  float tau, half_log_m, eps_m;
  float* phi;             // (BH, rows, m): QUERY and KEY
  float* ls;              // QUERY: (BH, rows) log-scales; KEYMAX: beta out (BH); KEY: beta in (BH)
  const int64_t* lengths; // KEY
  int64_t pos0, S_total;  // KEY: global position of row 0, global key count
  int row_lo, row_hi;     // rows processed
};

template <typename T, int MODE>
__global__ void __launch_bounds__(NTHR) feat_kernel(FeatArgs a) {
  __shared__ __align__(16) float sA[KS][LDT];
  __shared__ __align__(16) float sB[KS][LDT];
  __shared__ float sG[TILE];
  __shared__ float sRed[NTHR / 32];
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int row0 = a.row_lo + blockIdx.x * TILE;
  const int nrows = min(TILE, a.row_hi - row0);
  const int m = 2 * a.r;
  const T* x = reinterpret_cast<const T*>(a.x) + b * a.sb + h * a.sh + (int64_t)row0 * a.ss;

  {  // diag = tau * |x|^2 / 2, four threads per row
    const int row = threadIdx.x / 4, part = threadIdx.x % 4;
    float s = 0.f;
    if (row < nrows)
      for (int e = part; e < a.E; e += 4) {
        const float xv = ldf(x + (int64_t)row * a.ss + e);
        s = fmaf(xv, xv, s);
      }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (part == 0) sG[row] = s / 2.f * a.tau;
  }
  __syncthreads();

  float run_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  float beta = 0.f;
  int64_t len_b = 0;
  if (MODE == MODE_KEY) {
    beta = a.ls[bh];
    len_b = a.lengths ? a.lengths[b] : a.S_total;
  }
  float* phi_rows = (MODE == MODE_KEYMAX) ? nullptr : a.phi + ((int64_t)bh * a.rows + row0) * m;

  for (int c0 = 0; c0 < a.r; c0 += TILE) {
    float acc[4][4] = {};
    tile_nt(acc, x, a.ss, nrows, a.Wt + (int64_t)c0 * a.E, (int64_t)a.E, a.r - c0, a.E, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = ty * 4 + i;
      if (row >= nrows) continue;
      const float g = sG[row];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = c0 + tx * 4 + j;
        if (col >= a.r) continue;
        const float u = acc[i][j];
        if (MODE == MODE_QUERY) {
          phi_rows[(int64_t)row * m + col] = u;
          run_max[i] = fmaxf(run_max[i], fabsf(u));
        } else if (MODE == MODE_KEYMAX) {
          run_max[i] = fmaxf(run_max[i], (fabsf(u) - g) - a.half_log_m);
        } else {
          float e1 = 0.f, e2 = 0.f;
          if (a.pos0 + row0 + row < len_b) {
            e1 = expf(((u - g) - a.half_log_m) - beta) + a.eps_m;
            e2 = expf(((-u - g) - a.half_log_m) - beta) + a.eps_m;
          }
          phi_rows[(int64_t)row * m + col] = e1;
          phi_rows[(int64_t)row * m + a.r + col] = e2;
        }
      }
    }
  }

  if (MODE == MODE_QUERY) {
#pragma unroll
    for (int i = 0; i < 4; ++i) run_max[i] = group16_max(run_max[i]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = ty * 4 + i;
      if (row >= nrows) continue;
      if (tx == 0) a.ls[(int64_t)bh * a.rows + row0 + row] = (-sG[row] + run_max[i]) - a.half_log_m;
      for (int c0 = 0; c0 < a.r; c0 += TILE)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = c0 + tx * 4 + j;
          if (col >= a.r) continue;
          const float u = phi_rows[(int64_t)row * m + col];  // written by this same thread above
          phi_rows[(int64_t)row * m + col] = expf(u - run_max[i]) + a.eps_m;
          phi_rows[(int64_t)row * m + a.r + col] = expf(-u - run_max[i]) + a.eps_m;
        }
    }
  } else if (MODE == MODE_KEYMAX) {
    float v = fmaxf(fmaxf(run_max[0], run_max[1]), fmaxf(run_max[2], run_max[3]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x % 32 == 0) sRed[threadIdx.x / 32] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < NTHR / 32; ++i) v = fmaxf(v, sRed[i]);
      if (v > -INFINITY) atomic_max_float(a.ls + bh, v);
    }
  }
}

// ---------------------------------------------------------------------------
// Summary: partial[bh][split] (m x (D+1)) = phi(K)[rows]^T [V | 1]
// (scatterbrain_utils.py:20,49).  The extra column carries sum_s phi(k_s).
template <typename T>
__global__ void __launch_bounds__(NTHR)
summary_partial_kernel(const float* phik, const void* vptr, int64_t sb, int64_t ss, int64_t sh, int S, int m,
                       int D, int H, int row_lo, int row_hi, int split_rows, int dtiles, float* partial) {
  __shared__ __align__(16) float sA[KS][LDT];
  __shared__ __align__(16) float sB[KS][LDT];
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const int f0 = (blockIdx.x / dtiles) * TILE, d0 = (blockIdx.x % dtiles) * TILE;
  const int s_begin = row_lo + blockIdx.y * split_rows;
  const int s_end = min(row_hi, s_begin + split_rows);
  const T* v = reinterpret_cast<const T*>(vptr) + b * sb + h * sh;
  const float* pk = phik + (int64_t)bh * S * m;
  const int D1 = D + 1;
  float acc[4][4] = {};
  for (int s0 = s_begin; s0 < s_end; s0 += KS) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < PER_THR; ++i) {
      const int idx = threadIdx.x + i * NTHR;
      const int kk = idx / TILE, c = idx % TILE;
      const int s = s0 + kk;
      const bool in = s < s_end;
      sA[kk][c] = (in && f0 + c < m) ? pk[(int64_t)s * m + f0 + c] : 0.f;
      const int d = d0 + c;
      sB[kk][c] = !in ? 0.f : (d < D ? ldf(v + (int64_t)s * ss + d) : (d == D ? 1.f : 0.f));
    }
    __syncthreads();
    float part[4][4] = {};   // two-level sum over the keys
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&sA[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&sB[kk][tx * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w};
      const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], bv[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
  }
  float* out = partial + ((int64_t)bh * gridDim.y + blockIdx.y) * m * D1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int f = f0 + ty * 4 + i;
    if (f >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = d0 + tx * 4 + j;
      if (d < D1) out[(int64_t)f * D1 + d] = acc[i][j];
    }
  }
}

__global__ void summary_combine_kernel(const float* partial, int nsplit, int m, int D, int BH, float* kv,
                                       float* ksum) {
  const int D1 = D + 1;
  const int64_t n = (int64_t)BH * m * D1;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = (int)(i % D1);
  const int64_t bf = i / D1;  // bh*m + f
  const int64_t bh = bf / m, f = bf % m;
  float s = 0.f;
  for (int k = 0; k < nsplit; ++k) s += partial[((bh * nsplit + k) * m + f) * D1 + d];
  if (d < D) kv[bf * D + d] = s;
  else ksum[bf] = s;
}

// ---------------------------------------------------------------------------
// Band kernel (sblocal_attention.py:87-122).  One block = 64 queries of one
// (b,h); keys of the union of their windows are visited in chunks of 64 with
// a running row stabiliser.  Per row it keeps
//   c    running max of tau*q.k over valid window keys
//   L    sum exp(tau*q.k - c)
//   dps  sum phi(q).phi(k) over valid window keys
//   oexp sum exp(tau*q.k - c) v           olr  phi(q)KV - sum phi(q).phi(k) v
// and finishes with the reference's formulas:
//   n = logaddexp(c + log L, log(max(Z - dps, 1e-24)) + pls)
//   out = exp(c - n) * oexp + exp(pls - n) * olr
template <typename T, int DV>
__global__ void __launch_bounds__(NTHR)
band_kernel(SblParams p, const float* phiq, const float* qls, const float* phik, const float* beta,
            const float* kv, const float* ksum, float* lognorm) {
  constexpr int DVW = DV * 16;
  extern __shared__ __align__(16) float smem[];
  float(*sA)[LDT] = reinterpret_cast<float(*)[LDT]>(smem);
  float(*sB)[LDT] = reinterpret_cast<float(*)[LDT]>(smem + KS * LDT);
  float(*sE)[TILE + 1] = reinterpret_cast<float(*)[TILE + 1]>(smem + 2 * KS * LDT);
  float(*sP)[TILE + 1] = reinterpret_cast<float(*)[TILE + 1]>(smem + 2 * KS * LDT + TILE * (TILE + 1));
  float* sV = smem + 2 * KS * LDT + 2 * TILE * (TILE + 1);  // [TILE][DVW]
  float* sKs = sV + TILE * DVW;                             // [KS]

  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int i0 = blockIdx.x * TILE;
  const int nq = min(TILE, p.T - i0);
  const int m = 2 * p.r;
  const int hw = p.w / 2;
  int64_t len_b = p.key_lengths ? p.key_lengths[b] : p.S_total;
  if (len_b > p.S_total) len_b = p.S_total;
  const int64_t gq0 = p.q_pos0 + i0;
  const T* q = reinterpret_cast<const T*>(p.q) + b * p.q_stride_b + h * p.q_stride_h + (int64_t)i0 * p.q_stride_t;
  const T* kbase = reinterpret_cast<const T*>(p.k) + b * p.k_stride_b + h * p.k_stride_h;
  const T* vbase = reinterpret_cast<const T*>(p.v) + b * p.v_stride_b + h * p.v_stride_h;
  const float* pq = phiq + ((int64_t)bh * p.T + i0) * m;
  const float* pk = phik + (int64_t)bh * p.S * m;

  // buffer rows of the keys any query of this block can see
  int64_t glo = gq0 - hw, ghi = gq0 + nq - 1 - hw + p.w - 1;
  if (glo < 0) glo = 0;
  if (ghi > len_b - 1) ghi = len_b - 1;
  int64_t blo = glo - p.k_pos0, bhi = ghi - p.k_pos0;
  if (blo < 0) blo = 0;
  if (bhi > p.S - 1) bhi = p.S - 1;

  float c[4], L[4], dps[4], oexp[4][DV], olr[4][DV];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    c[i] = -INFINITY;
    L[i] = 0.f;
    dps[i] = 0.f;
#pragma unroll
    for (int d = 0; d < DV; ++d) oexp[i][d] = olr[i][d] = 0.f;
  }

  for (int64_t kb = blo; kb <= bhi; kb += TILE) {
    const int nk = (int)min((int64_t)TILE, bhi - kb + 1);
    float sacc[4][4] = {}, pacc[4][4] = {};
    tile_nt(sacc, q, p.q_stride_t, nq, kbase + kb * p.k_stride_s, p.k_stride_s, nk, p.E, sA, sB);
    tile_nt(pacc, pq, (int64_t)m, nq, pk + kb * m, (int64_t)m, nk, m, sA, sB);
    for (int idx = threadIdx.x; idx < TILE * DVW; idx += NTHR) {
      const int kk = idx / DVW, d = idx % DVW;
      sV[idx] = (kk < nk && d < p.D) ? ldf(vbase + (kb + kk) * p.v_stride_s + d) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t gi = gq0 + ty * 4 + i;
      float qk[4];
      bool ok[4];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = tx * 4 + j;
        const int64_t gk = p.k_pos0 + kb + col;
        ok[j] = col < nk && gk >= gi - hw && gk <= gi - hw + p.w - 1 && gk >= 0 && gk < len_b;
        qk[j] = p.softmax_temp * sacc[i][j];
        if (ok[j]) mx = fmaxf(mx, qk[j]);
      }
      mx = group16_max(mx);
      const float cn = fmaxf(c[i], mx);
      if (cn > -INFINITY) {
        const float sc = expf(c[i] - cn);  // c = -inf -> 0
        L[i] *= sc;
#pragma unroll
        for (int d = 0; d < DV; ++d) oexp[i][d] *= sc;
        c[i] = cn;
      }
      float es = 0.f, ps = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = ok[j] ? expf(qk[j] - cn) : 0.f;
        const float pp = ok[j] ? pacc[i][j] : 0.f;
        es += e;
        ps += pp;
        sE[ty * 4 + i][tx * 4 + j] = e;
        sP[ty * 4 + i][tx * 4 + j] = pp;
      }
      L[i] += group16_sum(es);
      dps[i] += group16_sum(ps);
    }
    __syncthreads();
    for (int kk = 0; kk < nk; ++kk) {
      float vv[DV];
#pragma unroll
      for (int d = 0; d < DV; ++d) vv[d] = sV[kk * DVW + tx + 16 * d];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e = sE[ty * 4 + i][kk], pp = sP[ty * 4 + i][kk];
#pragma unroll
        for (int d = 0; d < DV; ++d) {
          oexp[i][d] = fmaf(e, vv[d], oexp[i][d]);
          olr[i][d] = fmaf(-pp, vv[d], olr[i][d]);
        }
      }
    }
  }

  // low-rank part: olr += phi(Q) KV, Z = phi(Q) . ksum
  float Z[4] = {0.f, 0.f, 0.f, 0.f};
  const float* kvb = kv + (int64_t)bh * m * p.D;
  const float* ksb = ksum + (int64_t)bh * m;
  for (int f0 = 0; f0 < m; f0 += KS) {
    __syncthreads();
    float ra[PER_THR];
    fetch_slice(ra, pq, (int64_t)m, nq, f0, m);
    stash_slice(sA, ra);
    for (int idx = threadIdx.x; idx < KS * DVW; idx += NTHR) {
      const int kk = idx / DVW, d = idx % DVW;
      sV[idx] = (f0 + kk < m && d < p.D) ? kvb[(int64_t)(f0 + kk) * p.D + d] : 0.f;
    }
    if (threadIdx.x < KS) sKs[threadIdx.x] = (f0 + threadIdx.x < m) ? ksb[f0 + threadIdx.x] : 0.f;
    __syncthreads();
    float zp[4] = {0.f, 0.f, 0.f, 0.f}, lp[4][DV];   // two-level sums over the features
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int d = 0; d < DV; ++d) lp[i][d] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&sA[kk][ty * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w};
      const float ks = sKs[kk];
      float vv[DV];
#pragma unroll
      for (int d = 0; d < DV; ++d) vv[d] = sV[kk * DVW + tx + 16 * d];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        zp[i] = fmaf(av[i], ks, zp[i]);
#pragma unroll
        for (int d = 0; d < DV; ++d) lp[i][d] = fmaf(av[i], vv[d], lp[i][d]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      Z[i] += zp[i];
#pragma unroll
      for (int d = 0; d < DV; ++d) olr[i][d] += lp[i][d];
    }
  }

  const float beta_bh = beta[bh];
  T* out = reinterpret_cast<T*>(p.out) + b * p.o_stride_b + h * p.o_stride_h + (int64_t)i0 * p.o_stride_t;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = ty * 4 + i;
    if (row >= nq) continue;
    const float pls = qls[(int64_t)bh * p.T + i0 + row] + beta_bh;
    const float lse = L[i] > 0.f ? c[i] + logf(L[i]) : -INFINITY;
    const float lrn = logf(fmaxf(Z[i] - dps[i], 1e-24f)) + pls;
    const float hi = fmaxf(lse, lrn), lo = fminf(lse, lrn);
    const float n = hi + log1pf(expf(lo - hi));  // logaddexp; lo = -inf gives hi
    const float ce = expf(c[i] - n), ps = expf(pls - n);
    if (tx == 0) lognorm[(int64_t)bh * p.T + i0 + row] = n;
#pragma unroll
    for (int d = 0; d < DV; ++d) {
      const int col = tx + 16 * d;
      if (col < p.D) stf(out + (int64_t)row * p.o_stride_t + col, ce * oexp[i][d] + ps * olr[i][d]);
    }
  }
}

// ---------------------------------------------------------------------------
// Dense attention matrices of the need_weights branch (sblocal_attention.py:124-136).  One block =
// 64 queries x 64 keys of one (b,h): low-rank part phi(q).phi(k) for every pair, exact part only
// inside the window and key length.
template <typename T>
__global__ void __launch_bounds__(NTHR)
weights_kernel(SblParams p, const float* phiq, const float* qls, const float* phik, const float* beta,
               const float* lognorm, float* attn, float* attn_un, float* attn_lr) {
  __shared__ __align__(16) float sA[KS][LDT];
  __shared__ __align__(16) float sB[KS][LDT];
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int bh = blockIdx.z, b = bh / p.H, h = bh % p.H;
  const int i0 = blockIdx.y * TILE, s0 = blockIdx.x * TILE;
  const int nq = min(TILE, p.T - i0), nk = min(TILE, p.S - s0);
  const int m = 2 * p.r, hw = p.w / 2;
  int64_t len_b = p.key_lengths ? p.key_lengths[b] : p.S_total;
  const T* q = reinterpret_cast<const T*>(p.q) + b * p.q_stride_b + h * p.q_stride_h + (int64_t)i0 * p.q_stride_t;
  const T* k = reinterpret_cast<const T*>(p.k) + b * p.k_stride_b + h * p.k_stride_h + (int64_t)s0 * p.k_stride_s;
  float sacc[4][4] = {}, pacc[4][4] = {};
  tile_nt(sacc, q, p.q_stride_t, nq, k, p.k_stride_s, nk, p.E, sA, sB);
  tile_nt(pacc, phiq + ((int64_t)bh * p.T + i0) * m, (int64_t)m, nq, phik + ((int64_t)bh * p.S + s0) * m, (int64_t)m,
          nk, m, sA, sB);
  const float beta_bh = beta[bh];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = ty * 4 + i;
    if (row >= nq) continue;
    const int gi = i0 + row;
    const float n = lognorm[(int64_t)bh * p.T + gi];
    const float pls = qls[(int64_t)bh * p.T + gi] + beta_bh;
    const float ps = expf(pls - n), en = expf(n), epls = expf(pls);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tx * 4 + j;
      if (col >= nk) continue;
      const int gk = s0 + col;
      const bool in_win = gk >= gi - hw && gk <= gi - hw + p.w - 1 && gk < len_b;
      const float lr = pacc[i][j];   // phi(K) is zero at padded keys already
      const float local = in_win ? expf(p.softmax_temp * sacc[i][j] - n) - lr * ps : 0.f;
      const float a = local + lr * ps;
      const int64_t o = (((int64_t)bh * p.T + gi) * p.S) + gk;
      attn[o] = a;
      if (attn_un) attn_un[o] = a * en;
      if (attn_lr) attn_lr[o] = lr * epls;
    }
  }
}

template <typename T, int DV>
cudaError_t launch_band(const SblParams& p, const float* phiq, const float* qls, const float* phik,
                        const float* beta, const float* kv, const float* ksum, float* lognorm, cudaStream_t st) {
  const size_t smem = sizeof(float) * (2 * KS * LDT + 2 * TILE * (TILE + 1) + TILE * DV * 16 + KS);
  cudaError_t e = cudaFuncSetAttribute(band_kernel<T, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)div_up(p.T, TILE), (unsigned)(p.B * p.H));
  band_kernel<T, DV><<<grid, NTHR, smem, st>>>(p, phiq, qls, phik, beta, kv, ksum, lognorm);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_band_t(const SblParams& p, const float* phiq, const float* qls, const float* phik,
                          const float* beta, const float* kv, const float* ksum, float* lognorm, cudaStream_t st) {
  const int dv = (int)div_up(p.D, 16);
  if (dv <= 1) return launch_band<T, 1>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
  if (dv <= 2) return launch_band<T, 2>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
  if (dv <= 4) return launch_band<T, 4>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
  return launch_band<T, 8>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
}

FeatArgs feat_args(const SblParams& p, const Workspace& ws, char* base, bool query) {
  FeatArgs a{};
  a.H = p.H;
  a.E = p.E;
  a.r = p.r;
  a.Wt = reinterpret_cast<const float*>(base + ws.wt);
  const double c = sqrt((double)p.softmax_temp);
  a.tau = (float)(c * c);
  a.half_log_m = (float)(log(2.0 * p.r) / 2.0);
  a.eps_m = (float)((double)p.softmax_eps / sqrt(2.0 * p.r));
  if (query) {
    a.x = p.q; a.sb = p.q_stride_b; a.ss = p.q_stride_t; a.sh = p.q_stride_h; a.rows = p.T;
  } else {
    a.x = p.k; a.sb = p.k_stride_b; a.ss = p.k_stride_s; a.sh = p.k_stride_h; a.rows = p.S;
  }
  a.row_lo = 0;
  a.row_hi = a.rows;
  a.lengths = p.key_lengths;
  a.pos0 = p.k_pos0;
  a.S_total = p.S_total;
  return a;
}

template <int MODE>
cudaError_t launch_feat(const SblParams& p, const FeatArgs& a, cudaStream_t st) {
  const int n = a.row_hi - a.row_lo;
  if (n <= 0) return cudaSuccess;
  dim3 grid((unsigned)div_up(n, TILE), (unsigned)(p.B * p.H));
  if (p.dtype == SBL_DTYPE_F32) feat_kernel<float, MODE><<<grid, NTHR, 0, st>>>(a);
  else feat_kernel<__nv_bfloat16, MODE><<<grid, NTHR, 0, st>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t f32_prepare_projection(const SblParams& p, const Workspace& ws, char* base, cudaStream_t st) {
  const int n = p.r * p.E;
  scale_projection_kernel<<<(unsigned)div_up(n, 256), 256, 0, st>>>(
      p.W, (float)sqrt((double)p.softmax_temp), reinterpret_cast<float*>(base + ws.wt), n);
  return cudaGetLastError();
}

cudaError_t f32_key_logscale(const SblParams& p, const Workspace& ws, char* base, float* beta, cudaStream_t st) {
  const int bh = p.B * p.H;
  fill_kernel<<<(unsigned)div_up(bh, 256), 256, 0, st>>>(beta, -INFINITY, bh);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  FeatArgs a = feat_args(p, ws, base, false);
  a.ls = beta;
  a.row_lo = p.sum_lo;
  a.row_hi = p.sum_hi;
  return launch_feat<MODE_KEYMAX>(p, a, st);
}

cudaError_t f32_key_features(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                             float* phik_out, cudaStream_t st) {
  FeatArgs a = feat_args(p, ws, base, false);
  a.ls = const_cast<float*>(beta);
  a.phi = phik_out;
  return launch_feat<MODE_KEY>(p, a, st);
}

cudaError_t f32_key_summary(const SblParams& p, const Workspace& ws, char* base, const float* phik, float* kv,
                            float* ksum, cudaStream_t st) {
  const int m = 2 * p.r, bh = p.B * p.H;
  const int dtiles = (int)div_up(p.D + 1, TILE), mtiles = (int)div_up(m, TILE);
  float* partial = reinterpret_cast<float*>(base + ws.partial);
  dim3 grid((unsigned)(mtiles * dtiles), (unsigned)ws.nsplit, (unsigned)bh);
  if (p.dtype == SBL_DTYPE_F32)
    summary_partial_kernel<float><<<grid, NTHR, 0, st>>>(phik, p.v, p.v_stride_b, p.v_stride_s, p.v_stride_h, p.S,
                                                         m, p.D, p.H, p.sum_lo, p.sum_hi, ws.split_rows, dtiles,
                                                         partial);
  else
    summary_partial_kernel<__nv_bfloat16><<<grid, NTHR, 0, st>>>(phik, p.v, p.v_stride_b, p.v_stride_s,
                                                                 p.v_stride_h, p.S, m, p.D, p.H, p.sum_lo, p.sum_hi,
                                                                 ws.split_rows, dtiles, partial);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return f32_combine_partials(p, ws, base, kv, ksum, st);
}

cudaError_t f32_combine_partials(const SblParams& p, const Workspace& ws, char* base, float* kv, float* ksum,
                                 cudaStream_t st) {
  const int m = 2 * p.r, bh = p.B * p.H;
  const float* partial = reinterpret_cast<const float*>(base + ws.partial);
  const int64_t n = (int64_t)bh * m * (p.D + 1);
  summary_combine_kernel<<<(unsigned)div_up(n, 256), 256, 0, st>>>(partial, ws.nsplit, m, p.D, bh, kv, ksum);
  return cudaGetLastError();
}

cudaError_t f32_query_features(const SblParams& p, const Workspace& ws, char* base, float* phiq_out,
                               float* qls_out, cudaStream_t st) {
  FeatArgs a = feat_args(p, ws, base, true);
  a.phi = phiq_out;
  a.ls = qls_out;
  return launch_feat<MODE_QUERY>(p, a, st);
}

cudaError_t f32_attention_weights(const SblParams& p, const Workspace& ws, char* base, const float* beta,
                                  float* attn, float* attn_un, float* attn_lr, cudaStream_t st) {
  const float* phiq = reinterpret_cast<const float*>(base + ws.phiq);
  const float* qls = reinterpret_cast<const float*>(base + ws.qls);
  const float* phik = reinterpret_cast<const float*>(base + ws.phik);
  const float* lognorm = reinterpret_cast<const float*>(base + ws.lognorm);
  dim3 grid((unsigned)div_up(p.S, TILE), (unsigned)div_up(p.T, TILE), (unsigned)(p.B * p.H));
  if (p.dtype == SBL_DTYPE_F32)
    weights_kernel<float><<<grid, NTHR, 0, st>>>(p, phiq, qls, phik, beta, lognorm, attn, attn_un, attn_lr);
  else
    weights_kernel<__nv_bfloat16><<<grid, NTHR, 0, st>>>(p, phiq, qls, phik, beta, lognorm, attn, attn_un, attn_lr);
  return cudaGetLastError();
}

cudaError_t f32_band(const SblParams& p, const Workspace& ws, char* base, const float* beta, const float* kv,
                     const float* ksum, cudaStream_t st) {
  const float* phiq = reinterpret_cast<const float*>(base + ws.phiq);
  const float* qls = reinterpret_cast<const float*>(base + ws.qls);
  const float* phik = reinterpret_cast<const float*>(base + ws.phik);
  float* lognorm = reinterpret_cast<float*>(base + ws.lognorm);
  if (p.dtype == SBL_DTYPE_F32) return launch_band_t<float>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
  return launch_band_t<__nv_bfloat16>(p, phiq, qls, phik, beta, kv, ksum, lognorm, st);
}

}  // namespace sbl
