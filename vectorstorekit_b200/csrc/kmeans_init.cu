// k-means++ initialisation on the GPU: the reference's default way of choosing initial centroids
// (KMeansClustering.initializeKMeansPlusPlus, Clustering/KMeansClustering.swift:209-260; shader
// compute_min_distances, Acceleration/Metal/Shaders/ClusteringShaders.metal:205-238).
//
//   first centroid   a row drawn uniformly (Int.random(in: 0..<n) on the seeded generator)
//   each next one    every row's distance to its nearest chosen centroid is updated with the newest centroid
//                    (the minimum over all chosen centroids, as the reference recomputes it from scratch), then the
//                    reference's weighted draw: with d_i the un-squared distance, S = sum d_i, and u uniform in
//                    [0, 1), the first row whose running sum of d_i^2 / S exceeds u (the last row if none does).
//                    The weights divide squared distances by the sum of UN-squared ones - they do not sum to one -
//                    exactly as KMeansClustering.swift:236-252 computes them; that is kept.
//
// The reference seeds a fresh generator per draw (SeedableRNG(seed + number of centroids so far), :244), a 64-bit
// linear congruential generator (:480-491); Float.random / Int.random map its output as Swift's standard library
// does (24 random bits scaled by 2^-24; multiply-high with rejection).  The draws are therefore made on the host,
// one number per centroid, and the whole selection runs on the device without reading anything back.
// Running sums are taken in double precision by a two-level parallel scan, where the reference adds floats one
// after the other: a draw that lands within rounding of a row boundary may pick the neighbouring row.
#include <cmath>
#include <vector>

#include "common.cuh"

namespace vsk {
namespace {

constexpr int kPpBlock = 1024;   // rows per block of the two-level scan

// mind2[row] = min(mind2[row], |x_row - c|^2); one warp per row
__global__ void pp_update_kernel(const float* __restrict__ x, int64_t n, int dim, const float* __restrict__ cent,
                                 const int64_t* __restrict__ picked, int round, float* __restrict__ mind2) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float* c = cent + (int64_t)(round - 1) * dim;   // the newest centroid
  const float* p = x + row * dim;
  float s = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float d = __ldg(p + i) - __ldg(c + i);
    s = fmaf(d, d, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    if (row == picked[round - 1]) s = 0.f;   // a chosen row is at distance exactly 0 from itself
    mind2[row] = fminf(mind2[row], s);
  }
}

// per block of kPpBlock rows: sum of d^2 and sum of d
__global__ void __launch_bounds__(256) pp_block_sums_kernel(const float* __restrict__ mind2, int64_t n, double* __restrict__ s2,
                                                            double* __restrict__ s1) {
  __shared__ double a[256], b[256];
  const int64_t base = (int64_t)blockIdx.x * kPpBlock;
  double t2 = 0.0, t1 = 0.0;
  for (int i = threadIdx.x; i < kPpBlock; i += 256) {
    const int64_t r = base + i;
    if (r < n) {
      const float v = mind2[r];
      t2 += (double)v;
      t1 += (double)sqrtf(v);
    }
  }
  a[threadIdx.x] = t2;
  b[threadIdx.x] = t1;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      a[threadIdx.x] += a[threadIdx.x + o];
      b[threadIdx.x] += b[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    s2[blockIdx.x] = a[0];
    s1[blockIdx.x] = b[0];
  }
}

// One CTA: finds the drawn row and copies it into centroids[round].
__global__ void __launch_bounds__(1024) pp_pick_kernel(const float* __restrict__ x, int64_t n, int dim,
                                                       const float* __restrict__ mind2, const double* __restrict__ s2,
                                                       const double* __restrict__ s1, int nblocks, const float* __restrict__ u,
                                                       int round, float* __restrict__ cent, int64_t* __restrict__ picked,
                                                       int32_t* __restrict__ err) {
  __shared__ double sh[1024];
  __shared__ double s_total1, s_carry, s_before;
  __shared__ int s_block;
  __shared__ long long s_row;
  const int t = threadIdx.x;
  // S = sum of un-squared distances
  double acc = 0.0;
  for (int i = t; i < nblocks; i += 1024) acc += s1[i];
  sh[t] = acc;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (t < o) sh[t] += sh[t + o];
    __syncthreads();
  }
  if (t == 0) {
    s_total1 = sh[0];
    s_carry = 0.0;
    s_block = -1;
    s_row = -1;
  }
  __syncthreads();
  const double S = s_total1;
  if (!(S > 0.0)) {   // every row coincides with a chosen centroid: the reference throws degenerateData (:231-233)
    if (t == 0) atomicCAS(err, 0, 1);
    return;
  }
  const double target = (double)u[round] * S;   // u < cumulative(d^2 / S)  <=>  u * S < cumulative(d^2)
  // first block whose inclusive running sum of d^2 exceeds the target
  for (int base = 0; base < nblocks && s_block < 0; base += 1024) {
    const int i = base + t;
    sh[t] = i < nblocks ? s2[i] : 0.0;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const double v = t >= o ? sh[t - o] : 0.0;
      __syncthreads();
      sh[t] += v;
      __syncthreads();
    }
    const double incl = s_carry + sh[t];
    const double excl = incl - (i < nblocks ? s2[i] : 0.0);
    if (i < nblocks && incl > target && !(excl > target)) {   // exactly one thread: the first crossing
      s_block = i;
      s_before = excl;
    }
    __syncthreads();
    if (t == 1023) s_carry = incl;
    __syncthreads();
  }
  if (s_block >= 0) {
    const int64_t r = (int64_t)s_block * kPpBlock + t;
    const double v = (r < n && t < kPpBlock) ? (double)mind2[r] : 0.0;
    sh[t] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const double w = t >= o ? sh[t - o] : 0.0;
      __syncthreads();
      sh[t] += w;
      __syncthreads();
    }
    const double incl = s_before + sh[t];
    if (r < n && incl > target && !(incl - v > target)) s_row = r;
    __syncthreads();
    if (s_row < 0 && t == 0) s_row = min((long long)n - 1, (long long)s_block * kPpBlock + kPpBlock - 1);   // rounding fell between the two scans
  } else if (t == 0) {
    s_row = n - 1;   // the weights ran out before u was reached: the reference returns the last index (:446)
  }
  __syncthreads();
  const long long row = s_row;
  if (t == 0) picked[round] = row;
  for (int i = t; i < dim; i += 1024) cent[(int64_t)round * dim + i] = x[row * dim + i];
}

__global__ void pp_first_kernel(const float* __restrict__ x, int dim, int64_t first, float* __restrict__ cent,
                                int64_t* __restrict__ picked, float* __restrict__ mind2, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) mind2[i] = INFINITY;
  if (i < dim) cent[i] = x[first * dim + i];
  if (i == 0) picked[0] = first;
}

// ---- the reference's generator and Swift's mapping of its output ----------------------------------------
struct SeedableRng {   // KMeansClustering.swift:480-491
  uint64_t state;
  uint64_t next() {
    state = state * 2862933555777941757ull + 3037000493ull;
    return state;
  }
};
// Int.random(in: 0..<n, using:): multiply-high with rejection of the biased low range
uint64_t swift_random_below(SeedableRng& g, uint64_t n) {
  unsigned __int128 m = (unsigned __int128)g.next() * n;
  if ((uint64_t)m < n) {
    const uint64_t t = (0 - n) % n;
    while ((uint64_t)m < t) m = (unsigned __int128)g.next() * n;
  }
  return (uint64_t)(m >> 64);
}
// Float.random(in: 0..<1, using:): 24 random bits times 2^-24
float swift_random_unit_float(SeedableRng& g) {
  const uint32_t r = (uint32_t)g.next() & 0xffffffu;
  return (float)r * 5.9604645e-8f;
}

}  // namespace

int32_t kmeans_plusplus_dev(Ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k, uint64_t seed, float* centroids,
                            int64_t* picked_host) {
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty dataset");
  if (k <= 0 || k > n) return fail(ctx, VSK_ERR_INSUFFICIENT_TRAINING_DATA, "k = %d needs 1 <= k <= %lld rows", k, (long long)n);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !centroids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  // the draws: one generator per centroid, as the reference makes them
  std::vector<float> u((size_t)k, 0.f);
  SeedableRng g0{seed};
  const int64_t first = (int64_t)swift_random_below(g0, (uint64_t)n);
  for (int r = 1; r < k; ++r) {
    SeedableRng g{seed + (uint64_t)r};
    u[(size_t)r] = swift_random_unit_float(g);
  }
  const int nblocks = (int)ceil_div(n, kPpBlock);
  float *mind2 = nullptr, *du = nullptr;
  double* sums = nullptr;
  int64_t* picked = nullptr;
  int32_t* err = nullptr;
  auto body = [&]() -> int32_t {
    VSK_TRY(dev_alloc(ctx, (void**)&mind2, (size_t)n * 4));
    VSK_TRY(dev_alloc(ctx, (void**)&du, (size_t)k * 4));
    VSK_TRY(dev_alloc(ctx, (void**)&sums, (size_t)nblocks * 16));
    VSK_TRY(dev_alloc(ctx, (void**)&picked, (size_t)k * 8));
    VSK_TRY(dev_alloc(ctx, (void**)&err, 4));
    VSK_CUDA(ctx, cudaMemsetAsync(err, 0, 4, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(du, u.data(), (size_t)k * 4, cudaMemcpyHostToDevice, ctx->stream));
    pp_first_kernel<<<(unsigned)ceil_div(std::max<int64_t>(n, dim), 256), 256, 0, ctx->stream>>>(rows, dim, first, centroids, picked, mind2, n);
    ctx->stats.kernel_launches++;
    for (int r = 1; r < k; ++r) {
      pp_update_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(rows, n, dim, centroids, picked, r, mind2);
      pp_block_sums_kernel<<<(unsigned)nblocks, 256, 0, ctx->stream>>>(mind2, n, sums, sums + nblocks);
      pp_pick_kernel<<<1, 1024, 0, ctx->stream>>>(rows, n, dim, mind2, sums, sums + nblocks, nblocks, du, r, centroids, picked, err);
      ctx->stats.kernel_launches += 3;
    }
    VSK_CUDA(ctx, cudaGetLastError());
    int32_t herr = 0;
    VSK_CUDA(ctx, cudaMemcpyAsync(&herr, err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (picked_host) VSK_CUDA(ctx, cudaMemcpyAsync(picked_host, picked, (size_t)k * 8, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (herr != 0)
      return fail(ctx, VSK_ERR_INVALID_INPUT, "degenerate data: fewer distinct rows than centroids (k-means++ cannot draw)");
    return VSK_OK;
  };
  const int32_t st = body();
  if (st != VSK_OK) cudaStreamSynchronize(ctx->stream);
  dev_free(mind2);
  dev_free(du);
  dev_free(sums);
  dev_free(picked);
  dev_free(err);
  return st;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_kmeans_init_plusplus_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t k, uint64_t seed,
                                     float* centroids, int64_t* picked) {
  VSK_TRACE("vsk_kmeans_init_plusplus_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  return kmeans_plusplus_dev(ctx, rows, n, dim, k, seed, centroids, picked);
}

int32_t vsk_kmeans_init_plusplus(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t k, uint64_t seed,
                                 float* centroids, int64_t* picked) {
  VSK_TRACE("vsk_kmeans_init_plusplus");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty dataset");
  if (k <= 0 || k > n) return fail(ctx, VSK_ERR_INSUFFICIENT_TRAINING_DATA, "k = %d needs 1 <= k <= %lld rows", k, (long long)n);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !centroids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  float *dx = nullptr, *dc = nullptr;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&dx, (size_t)n * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dc, (size_t)k * dim * 4)) == VSK_OK) {
    cudaMemcpyAsync(dx, rows, (size_t)n * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    ctx->stats.h2d_bytes += n * (int64_t)dim * 4;
    st = kmeans_plusplus_dev(ctx, dx, n, dim, k, seed, dc, picked);
    if (st == VSK_OK) {
      const cudaError_t e = cudaMemcpy(centroids, dc, (size_t)k * dim * 4, cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "copy out failed: %s", cudaGetErrorString(e));
    }
  }
  dev_free(dx);
  dev_free(dc);
  return st;
}

}  // extern "C"
