// The fp32 CUDA-core tile shared by the flat scan, the k-means assignment, the IVF list scan and
// the int8 scan: a CTA of 256 threads computes a 128 x 128 block of pair values with the
// reference's direct per-pair formulas (accumulated in dimension order), each thread an 8 x 8
// micro-tile.  Operands are staged k-major in shared memory in slices of 16 dimensions, double
// buffered through registers.  What differs between users is only where the 128 "a" rows and the
// 128 "b" rows come from (row loaders) and what the epilogue does with the 64 values.
#pragma once
#include "common.cuh"

namespace vsk {
namespace tile {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256, PAD = 4;

struct Smem {
  float As[2][BK][BM + PAD];
  float Bs[2][BK][BN + PAD];
};

template <int METRIC>
__device__ __forceinline__ void accum(float& acc, float q, float x) {
  if (METRIC == VSK_METRIC_EUCLIDEAN) {
    float t = q - x;
    acc = fmaf(t, t, acc);
  } else if (METRIC == VSK_METRIC_MANHATTAN) {
    acc += fabsf(q - x);
  } else {
    acc = fmaf(q, x, acc);
  }
}

// fp32 row: 4 consecutive dimensions, zero beyond `dim` or for a missing row.
struct F32Row {
  const float* base;
  bool ok;
  bool vec;
  __device__ __forceinline__ float4 load(int k, int dim) const {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!ok) return v;
    if (vec && k + 3 < dim) return __ldg(reinterpret_cast<const float4*>(base + k));
    if (k + 0 < dim) v.x = __ldg(base + k + 0);
    if (k + 1 < dim) v.y = __ldg(base + k + 1);
    if (k + 2 < dim) v.z = __ldg(base + k + 2);
    if (k + 3 < dim) v.w = __ldg(base + k + 3);
    return v;
  }
};

// int8-coded row, dequantised while staging: x^ = (code - offset)/scale per dimension
// (ScalarQuantizer.swift:568-580), each operation rounded separately.
struct I8Row {
  const int8_t* base;
  const float* scale;
  const float* offset;
  bool ok;
  bool vec;
  __device__ __forceinline__ float deq(int c, int k) const {
    return __fdiv_rn(__fsub_rn((float)c, __ldg(offset + k)), __ldg(scale + k));
  }
  __device__ __forceinline__ float4 load(int k, int dim) const {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!ok) return v;
    if (vec && k + 3 < dim) {
      char4 c = __ldg(reinterpret_cast<const char4*>(base + k));
      v.x = deq(c.x, k); v.y = deq(c.y, k + 1); v.z = deq(c.z, k + 2); v.w = deq(c.w, k + 3);
      return v;
    }
    if (k + 0 < dim) v.x = deq(__ldg(base + k + 0), k + 0);
    if (k + 1 < dim) v.y = deq(__ldg(base + k + 1), k + 1);
    if (k + 2 < dim) v.z = deq(__ldg(base + k + 2), k + 2);
    if (k + 3 < dim) v.w = deq(__ldg(base + k + 3), k + 3);
    return v;
  }
};

// Row/column of the micro-tile element (i, j) of this thread inside the 128 x 128 block.
__device__ __forceinline__ int tile_row(int i) { return i < 4 ? (threadIdx.x >> 4) * 4 + i : 64 + (threadIdx.x >> 4) * 4 + (i - 4); }
__device__ __forceinline__ int tile_col(int j) { return j < 4 ? (threadIdx.x & 15) * 4 + j : 64 + (threadIdx.x & 15) * 4 + (j - 4); }
// The two block rows this thread stages (h = 0, 1) and the first of its 4 dimensions in a slice.
__device__ __forceinline__ int stage_row(int h) { return (threadIdx.x >> 2) + h * 64; }
__device__ __forceinline__ int stage_k() { return (threadIdx.x & 3) * 4; }

template <int METRIC, class ARow, class BRow>
__device__ __forceinline__ void mainloop(float (&acc)[8][8], const ARow (&ar)[2], const BRow (&br)[2], int dim,
                                         Smem& sm) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int lr = threadIdx.x >> 2, lk = stage_k();
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  const int nk = (dim + BK - 1) / BK;
  float4 ra[2], rb[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    ra[h] = ar[h].load(lk, dim);
    rb[h] = br[h].load(lk, dim);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = lr + h * 64;
    sm.As[0][lk + 0][r] = ra[h].x; sm.As[0][lk + 1][r] = ra[h].y; sm.As[0][lk + 2][r] = ra[h].z; sm.As[0][lk + 3][r] = ra[h].w;
    sm.Bs[0][lk + 0][r] = rb[h].x; sm.Bs[0][lk + 1][r] = rb[h].y; sm.Bs[0][lk + 2][r] = rb[h].z; sm.Bs[0][lk + 3][r] = rb[h].w;
  }
  __syncthreads();
  for (int kb = 0; kb < nk; ++kb) {
    const int s = kb & 1;
    if (kb + 1 < nk) {
      const int k = (kb + 1) * BK + lk;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        ra[h] = ar[h].load(k, dim);
        rb[h] = br[h].load(k, dim);
      }
    }
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&sm.As[s][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&sm.As[s][kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&sm.Bs[s][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&sm.Bs[s][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) accum<METRIC>(acc[i][j], av[i], bv[j]);
    }
    if (kb + 1 < nk) {
      const int s2 = s ^ 1;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = lr + h * 64;
        sm.As[s2][lk + 0][r] = ra[h].x; sm.As[s2][lk + 1][r] = ra[h].y; sm.As[s2][lk + 2][r] = ra[h].z; sm.As[s2][lk + 3][r] = ra[h].w;
        sm.Bs[s2][lk + 0][r] = rb[h].x; sm.Bs[s2][lk + 1][r] = rb[h].y; sm.Bs[s2][lk + 2][r] = rb[h].z; sm.Bs[s2][lk + 3][r] = rb[h].w;
      }
    }
    __syncthreads();
  }
}

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
__device__ __forceinline__ bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; }

}  // namespace tile
}  // namespace vsk

// ---- the same tile with a narrower "a" side ---------------------------------------------------
// BM_ = 32 or 64 "a" rows x 128 "b" rows per CTA (256 threads, BM_/16 x 8 values per thread).
// Used where the number of "a" rows that share a "b" block is small (IVF: the queries probing one list),
// so that a block's cost follows the rows it actually holds.
namespace vsk {
namespace tile {

template <int BM_>
struct SmemM {
  float As[2][BK][BM_ + PAD];
  float Bs[2][BK][BN + PAD];
};

template <int BM_>
__device__ __forceinline__ int mrow(int i) { return (threadIdx.x >> 4) * (BM_ / 16) + i; }

template <int METRIC, int BM_, class ARow, class BRow>
__device__ __forceinline__ void mainloop_m(float (&acc)[BM_ / 16][8], const ARow& ar, const BRow (&br)[2], int dim,
                                           SmemM<BM_>& sm) {
  static_assert(BM_ == 32 || BM_ == 64, "the narrow tile stages at most one \"a\" row per thread");
  constexpr int QM = BM_ / 16;
  // "a" staging: thread t stages dimensions lk..lk+3 of row t>>2 when that row exists (t>>2 < BM_)
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int lr = threadIdx.x >> 2, lk = stage_k();
  const bool a_stage = lr < BM_;
#pragma unroll
  for (int i = 0; i < QM; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  const int nk = (dim + BK - 1) / BK;
  float4 ra = make_float4(0.f, 0.f, 0.f, 0.f), rb[2];
  if (a_stage) ra = ar.load(lk, dim);
#pragma unroll
  for (int h = 0; h < 2; ++h) rb[h] = br[h].load(lk, dim);
  if (a_stage) { sm.As[0][lk + 0][lr] = ra.x; sm.As[0][lk + 1][lr] = ra.y; sm.As[0][lk + 2][lr] = ra.z; sm.As[0][lk + 3][lr] = ra.w; }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = lr + h * 64;
    sm.Bs[0][lk + 0][r] = rb[h].x; sm.Bs[0][lk + 1][r] = rb[h].y; sm.Bs[0][lk + 2][r] = rb[h].z; sm.Bs[0][lk + 3][r] = rb[h].w;
  }
  __syncthreads();
  for (int kb = 0; kb < nk; ++kb) {
    const int s = kb & 1;
    if (kb + 1 < nk) {
      const int k = (kb + 1) * BK + lk;
      if (a_stage) ra = ar.load(k, dim);
#pragma unroll
      for (int h = 0; h < 2; ++h) rb[h] = br[h].load(k, dim);
    }
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[QM];
#pragma unroll
      for (int i = 0; i < QM; ++i) av[i] = sm.As[s][kk][ty * QM + i];
      const float4 b0 = *reinterpret_cast<const float4*>(&sm.Bs[s][kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&sm.Bs[s][kk][64 + tx * 4]);
      const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < QM; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) accum<METRIC>(acc[i][j], av[i], bv[j]);
    }
    if (kb + 1 < nk) {
      const int s2 = s ^ 1;
      if (a_stage) { sm.As[s2][lk + 0][lr] = ra.x; sm.As[s2][lk + 1][lr] = ra.y; sm.As[s2][lk + 2][lr] = ra.z; sm.As[s2][lk + 3][lr] = ra.w; }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = lr + h * 64;
        sm.Bs[s2][lk + 0][r] = rb[h].x; sm.Bs[s2][lk + 1][r] = rb[h].y; sm.Bs[s2][lk + 2][r] = rb[h].z; sm.Bs[s2][lk + 3][r] = rb[h].w;
      }
    }
    __syncthreads();
  }
}

}  // namespace tile
}  // namespace vsk
