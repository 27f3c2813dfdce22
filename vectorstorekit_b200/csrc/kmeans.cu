// Lloyd k-means on the GPU.  Replaces KMeansClustering.cluster
// (Clustering/KMeansClustering.swift:48-113) and the shader kernels assign_to_centroids,
// accumulate_centroids, finalize_centroids, compute_inertia
// (Acceleration/Metal/Shaders/ClusteringShaders.metal:29-177,317-331).
//
//   assignment  the fp32 tile kernel with an arg-min epilogue: per row the smallest
//               (squared distance, centroid index) key, so the lowest index wins ties exactly as
//               the reference's strict '<' scan does (KMeansClustering.swift:283-288)
//   update      rows are grouped by centroid with a stable counting sort, then one CTA per
//               centroid adds its rows IN ROW ORDER, one thread per dimension — the same fp32
//               summation order as KMeansClustering.updateCentroids (:342-380), with no float
//               atomics, so the result is deterministic
//   empty       an empty cluster keeps its previous centroid (ClusteringShaders.metal:171-176)
//   inertia     sum of the un-squared distances (KMeansClustering.swift:97), reduced in fp64
#include "common.cuh"
#include "tensor_scan.cuh"

namespace vsk {
namespace {

__global__ void decode_best_kernel(const unsigned long long* best, int64_t n, int32_t* assign, float* dist) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned long long b = best[i];
  assign[i] = (int32_t)(uint32_t)b;
  if (dist) dist[i] = sqrtf(ordered_to_float((uint32_t)(b >> 32)));
}

// Centroid update in two steps, both in a fixed order (deterministic, no float atomics).
// Rows are already grouped by centroid (`order`, row order inside a group).  A group is cut into segments of
// kSegRows rows; one CTA sums one segment, one thread per dimension, adding rows in row order; then one CTA per
// centroid adds its segments' partial sums in segment order and divides by the count.  A group of at most
// kSegRows rows is therefore summed exactly in the reference's order (KMeansClustering.swift:342-380).
constexpr int kSegRows = 256;

__global__ void segment_count_kernel(const int64_t* __restrict__ offsets, int k, int64_t* __restrict__ nseg) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < k) nseg[c] = (offsets[c + 1] - offsets[c] + kSegRows - 1) / kSegRows;
}

__global__ void segment_sum_kernel(const float* __restrict__ x, int dim, const int32_t* __restrict__ order,
                                   const int64_t* __restrict__ offsets, const int64_t* __restrict__ seg_off, int k,
                                   float* __restrict__ partial) {
  __shared__ int s_c;
  const int64_t seg = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = k;   // last centroid whose first segment is <= seg
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seg_off[mid] <= seg) lo = mid; else hi = mid;
    }
    s_c = lo;
  }
  __syncthreads();
  const int c = s_c;
  const int64_t begin = offsets[c] + (seg - seg_off[c]) * kSegRows;
  const int64_t end = min(offsets[c + 1], begin + kSegRows);
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float s = 0.f;
    int64_t r = begin;
    // eight rows' loads in flight per thread, added in row order (the sum's order is part of the result)
    for (; r + 8 <= end; r += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __ldg(x + (int64_t)order[r + j] * dim + d);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j];
    }
    for (; r + 4 <= end; r += 4) {
      const float v0 = __ldg(x + (int64_t)order[r + 0] * dim + d);
      const float v1 = __ldg(x + (int64_t)order[r + 1] * dim + d);
      const float v2 = __ldg(x + (int64_t)order[r + 2] * dim + d);
      const float v3 = __ldg(x + (int64_t)order[r + 3] * dim + d);
      s += v0; s += v1; s += v2; s += v3;
    }
    for (; r < end; ++r) s += __ldg(x + (int64_t)order[r] * dim + d);
    partial[seg * dim + d] = s;
  }
}

__global__ void centroid_finish_kernel(const float* __restrict__ partial, int dim, const int64_t* __restrict__ offsets,
                                       const int64_t* __restrict__ seg_off, const float* __restrict__ old_c,
                                       float* __restrict__ new_c) {
  const int c = blockIdx.x;
  const int64_t cnt = offsets[c + 1] - offsets[c];
  const int64_t s0 = seg_off[c], s1 = seg_off[c + 1];
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    if (cnt == 0) {
      new_c[(int64_t)c * dim + d] = old_c[(int64_t)c * dim + d];   // an empty cluster keeps its centroid
      continue;
    }
    float s = partial[s0 * dim + d];
    for (int64_t g = s0 + 1; g < s1; ++g) s += partial[g * dim + d];
    new_c[(int64_t)c * dim + d] = s / (float)cnt;
  }
}

// The same sum without the division, and the group's row count: one shard's contribution to a centroid when the
// rows are spread over several GPUs (the means are formed after the shards' sums have been added up).
__global__ void centroid_sum_kernel(const float* __restrict__ partial, int dim, const int64_t* __restrict__ offsets,
                                    const int64_t* __restrict__ seg_off, float* __restrict__ sums,
                                    float* __restrict__ counts) {
  const int c = blockIdx.x;
  const int64_t s0 = seg_off[c], s1 = seg_off[c + 1];
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float s = 0.f;
    for (int64_t g = s0; g < s1; ++g) s += partial[g * dim + d];
    sums[(int64_t)c * dim + d] = s;
  }
  if (threadIdx.x == 0) counts[c] = (float)(offsets[c + 1] - offsets[c]);   // exact below 2^24 rows per centroid and shard
}

// centroids from summed contributions: sum / count, an empty cluster keeps its centroid
__global__ void centroid_mean_kernel(const float* __restrict__ sums, const float* __restrict__ counts, int64_t total,
                                     int dim, const float* __restrict__ old_c, float* __restrict__ new_c) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float cnt = counts[i / dim];
  new_c[i] = cnt > 0.f ? sums[i] / cnt : old_c[i];
}

// fixed-shape fp64 reduction: 1024 partial sums, then one block
__global__ void sum_partial_kernel(const float* v, int64_t n, double* partial) {
  __shared__ double sh[256];
  const int64_t per = (n + gridDim.x - 1) / gridDim.x;
  const int64_t b = (int64_t)blockIdx.x * per, e = min(n, b + per);
  double s = 0.0;
  for (int64_t i = b + threadIdx.x; i < e; i += blockDim.x) s += (double)v[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
__global__ void sum_final_kernel(const double* partial, int np, float* out) {
  __shared__ double sh[1024];
  sh[threadIdx.x] = threadIdx.x < np ? partial[threadIdx.x] : 0.0;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = (float)sh[0];
}

}  // namespace

int32_t assign_rows_fp32(Ctx* ctx, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                         int32_t* assign, float* dist);

// Nearest centroid (and rooted distance) of every row.
static bool use_tensor_assign(const Ctx* ctx, int64_t n, int32_t k) {
  // the tensor path pays for making fp16 operands; tiny problems stay on the fp32 tile
  return ctx->search_path == VSK_PATH_TENSOR_RERANK && n * (int64_t)k >= (1ll << 22) && n >= 1024;
}

int32_t assign_rows(Ctx* ctx, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                    int32_t* assign, float* dist) {
  if (use_tensor_assign(ctx, n, k)) {
    TensorAssign ta;
    int32_t st = tensor_assign_prepare(ctx, rows, n, dim, &ta);
    if (st == VSK_OK) st = tensor_assign(ctx, &ta, rows, centroids, k, assign, dist, false);
    if (st == VSK_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = VSK_ERR_EXECUTION_FAILED;
    tensor_assign_release(&ta);
    return st;
  }
  return assign_rows_fp32(ctx, rows, n, dim, centroids, k, assign, dist);
}

int32_t assign_rows_fp32(Ctx* ctx, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                         int32_t* assign, float* dist) {
  void* best;
  VSK_TRY(scratch(ctx, SLOT_MISC4, (size_t)n * sizeof(unsigned long long), &best));
  VSK_CUDA(ctx, cudaMemsetAsync(best, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
  ExactScanArgs a{};
  a.metric = VSK_METRIC_EUCLIDEAN;
  a.mode = SCAN_ARGMIN;
  a.q = rows;
  a.nq = n;
  a.x = centroids;
  a.dim = dim;
  a.row_begin = 0;
  a.row_end = k;
  a.best = (unsigned long long*)best;
  VSK_TRY(launch_exact_scan(ctx, a));
  decode_best_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>((const unsigned long long*)best, n, assign, dist);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

// ---- nearest-centroid assignment without any allocation ------------------------------------
// Scratch for vsk_assign_static_dev: one 64-bit (distance, centroid) key per row.  The array is part
// of the library image, so every GPU that loads the library holds these 8 MB until the process exits.
constexpr int64_t kAssignStaticMaxRows = 1 << 20;
static __device__ __align__(256) unsigned long long g_assign_static_keys[kAssignStaticMaxRows];
// Device address of the array on each GPU, looked up once per device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use.
static unsigned long long* g_assign_static_ptr[64] = {};

int32_t assign_rows_static(Ctx* ctx, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                           int32_t* assign, float* dist) {
  if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, VSK_ERR_INVALID_INPUT, "device index out of range");
  unsigned long long* keys = g_assign_static_ptr[ctx->device];
  if (!keys) {
    // first call on this GPU (the context's device is current here)
    void* p = nullptr;
    VSK_CUDA(ctx, cudaGetSymbolAddress(&p, g_assign_static_keys));
    keys = g_assign_static_ptr[ctx->device] = static_cast<unsigned long long*>(p);
    chk_add(p, sizeof(g_assign_static_keys));   // checked build: the array is a legal target
  }
  // The array still holds the previous call's keys: every key this call reads must start as all ones.
  VSK_CUDA(ctx, cudaMemsetAsync(keys, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
  ExactScanArgs a{};
  a.metric = VSK_METRIC_EUCLIDEAN;
  a.mode = SCAN_ARGMIN;
  a.q = rows;
  a.nq = n;
  a.x = centroids;
  a.dim = dim;
  a.row_begin = 0;
  a.row_end = k;
  a.best = keys;
  const bool was_profiling = ctx->profile;   // timing events are created on demand: keep them out of this path
  ctx->profile = false;
  const int32_t st = launch_exact_scan(ctx, a);
  ctx->profile = was_profiling;
  VSK_TRY(st);
  decode_best_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(keys, n, assign, dist);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t kmeans_dev(Ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k, int32_t max_iters,
                   float tolerance, const float* init, float* centroids, int32_t* assign, float* inertia,
                   int32_t* iters_run) {
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty dataset");
  if (k <= 0 || k > n) return fail(ctx, VSK_ERR_INSUFFICIENT_TRAINING_DATA, "k = %d needs 1 <= k <= %lld rows", k, (long long)n);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "at most 2^31-1 rows");
  if (!rows || !init || !centroids || !assign) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  void *cur, *nxt, *dist, *order, *offsets, *partial, *inert;
  VSK_TRY(scratch(ctx, SLOT_MISC0, (size_t)k * dim * 4, &cur));
  VSK_TRY(scratch(ctx, SLOT_MISC1, (size_t)k * dim * 4, &nxt));
  VSK_TRY(scratch(ctx, SLOT_MISC2, (size_t)n * 4, &dist));
  VSK_TRY(scratch(ctx, SLOT_MISC3, (size_t)n * 4, &order));
  VSK_TRY(scratch(ctx, SLOT_X_TMP, (size_t)(k + 1) * 8, &offsets));
  VSK_TRY(scratch(ctx, SLOT_QAUX, 1024 * 8 + 16, &partial));
  inert = (char*)partial + 1024 * 8;
  VSK_CUDA(ctx, cudaMemcpyAsync(cur, init, (size_t)k * dim * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  float prev = INFINITY, last = INFINITY;
  int it = 0;
  bool converged = false;
  TensorAssign ta;
  const bool tc = use_tensor_assign(ctx, n, k);
  struct Release {
    TensorAssign* t;
    ~Release() { tensor_assign_release(t); }
  } release{&ta};
  if (tc) VSK_TRY(tensor_assign_prepare(ctx, rows, n, dim, &ta));
  while (it < max_iters && !converged) {
    if (tc) VSK_TRY(tensor_assign(ctx, &ta, rows, (const float*)cur, k, assign, (float*)dist, it > 0));
    else VSK_TRY(assign_rows_fp32(ctx, rows, n, dim, (const float*)cur, k, assign, (float*)dist));
    tl_mark(ctx, "assign_done");
    VSK_TRY(launch_stable_group(ctx, assign, n, k, (int32_t*)order, (int64_t*)offsets));
    tl_mark(ctx, "group_rows");
    {
      // segments per centroid -> first segment of each centroid -> partial sums -> means
      const int64_t max_segs = n / kSegRows + k + 1;
      void *nseg, *seg_off, *partial;
      VSK_TRY(scratch(ctx, SLOT_KM_NSEG, (size_t)(k + 1) * 8, &nseg));
      VSK_TRY(scratch(ctx, SLOT_KM_SEGOFF, (size_t)(k + 1) * 8, &seg_off));
      VSK_TRY(scratch(ctx, SLOT_KM_PARTIAL, (size_t)max_segs * dim * 4, &partial));
      segment_count_kernel<<<(unsigned)ceil_div(k, 256), 256, 0, ctx->stream>>>((const int64_t*)offsets, k, (int64_t*)nseg);
      VSK_TRY(launch_scan_i64(ctx, (const int64_t*)nseg, k, (int64_t*)seg_off));
      const int threads = std::min(256, (dim + 31) / 32 * 32);
      segment_sum_kernel<<<(unsigned)max_segs, threads, 0, ctx->stream>>>(rows, dim, (const int32_t*)order, (const int64_t*)offsets,
                                                                         (const int64_t*)seg_off, k, (float*)partial);
      centroid_finish_kernel<<<k, threads, 0, ctx->stream>>>((const float*)partial, dim, (const int64_t*)offsets,
                                                             (const int64_t*)seg_off, (const float*)cur, (float*)nxt);
      ctx->stats.kernel_launches += 2;
    }
    sum_partial_kernel<<<1024, 256, 0, ctx->stream>>>((const float*)dist, n, (double*)partial);
    sum_final_kernel<<<1, 1024, 0, ctx->stream>>>((const double*)partial, 1024, (float*)inert);
    tl_mark(ctx, "update_done");
    ctx->stats.kernel_launches += 3;
    VSK_CUDA(ctx, cudaGetLastError());
    std::swap(cur, nxt);
    ++it;
    if (tolerance >= 0.f || it == max_iters) {
      VSK_CUDA(ctx, cudaMemcpyAsync(&last, inert, 4, cudaMemcpyDeviceToHost, ctx->stream));
      VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      converged = tolerance >= 0.f && fabsf(last - prev) < tolerance;
      prev = last;
    }
  }
  VSK_CUDA(ctx, cudaMemcpyAsync(centroids, cur, (size_t)k * dim * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (inertia) *inertia = last;
  if (iters_run) *iters_run = it;
  return VSK_OK;
}

// ---- one Lloyd step over a shard of the rows (rows spread over several GPUs) -------------------------------
struct KMeansTrainer {
  Ctx* ctx = nullptr;
  const float* rows = nullptr;
  int64_t n = 0;
  int32_t dim = 0, k = 0;
  int32_t* assign = nullptr;   // [n]
  float* dist = nullptr;       // [n]
  int32_t* order = nullptr;    // [n]
  bool tc = false;
  TensorAssign ta;
  int steps = 0;
};

int32_t trainer_step(KMeansTrainer* t, const float* centroids, float* sums, float* counts, float* inertia) {
  Ctx* ctx = t->ctx;
  const int64_t n = t->n;
  const int dim = t->dim, k = t->k;
  if (t->tc) VSK_TRY(tensor_assign(ctx, &t->ta, t->rows, centroids, k, t->assign, t->dist, t->steps > 0));
  else VSK_TRY(assign_rows_fp32(ctx, t->rows, n, dim, centroids, k, t->assign, t->dist));
  void *offsets, *nseg, *seg_off, *partial, *red;
  VSK_TRY(scratch(ctx, SLOT_X_TMP, (size_t)(k + 1) * 8, &offsets));
  VSK_TRY(launch_stable_group(ctx, t->assign, n, k, t->order, (int64_t*)offsets));
  const int64_t max_segs = n / kSegRows + k + 1;
  VSK_TRY(scratch(ctx, SLOT_KM_NSEG, (size_t)(k + 1) * 8, &nseg));
  VSK_TRY(scratch(ctx, SLOT_KM_SEGOFF, (size_t)(k + 1) * 8, &seg_off));
  VSK_TRY(scratch(ctx, SLOT_KM_PARTIAL, (size_t)max_segs * dim * 4, &partial));
  VSK_TRY(scratch(ctx, SLOT_QAUX, 1024 * 8 + 16, &red));
  segment_count_kernel<<<(unsigned)ceil_div(k, 256), 256, 0, ctx->stream>>>((const int64_t*)offsets, k, (int64_t*)nseg);
  VSK_TRY(launch_scan_i64(ctx, (const int64_t*)nseg, k, (int64_t*)seg_off));
  const int threads = std::min(256, (dim + 31) / 32 * 32);
  segment_sum_kernel<<<(unsigned)max_segs, threads, 0, ctx->stream>>>(t->rows, dim, t->order, (const int64_t*)offsets,
                                                                     (const int64_t*)seg_off, k, (float*)partial);
  centroid_sum_kernel<<<k, threads, 0, ctx->stream>>>((const float*)partial, dim, (const int64_t*)offsets,
                                                      (const int64_t*)seg_off, sums, counts);
  sum_partial_kernel<<<1024, 256, 0, ctx->stream>>>(t->dist, n, (double*)red);
  sum_final_kernel<<<1, 1024, 0, ctx->stream>>>((const double*)red, 1024, inertia);
  ctx->stats.kernel_launches += 5;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  t->steps++;
  return VSK_OK;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_kmeans_trainer_create_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t k,
                                      vsk_kmeans_trainer** out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  *out = nullptr;
  if (n <= 0 || !rows) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty dataset");
  if (k <= 0) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be positive");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "at most 2^31-1 rows");
  KMeansTrainer* t = new KMeansTrainer();
  t->ctx = ctx;
  t->rows = rows;
  t->n = n;
  t->dim = dim;
  t->k = k;
  t->tc = use_tensor_assign(ctx, n, k);
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&t->assign, (size_t)n * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&t->dist, (size_t)n * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&t->order, (size_t)n * 4)) == VSK_OK && t->tc)
    st = tensor_assign_prepare(ctx, rows, n, dim, &t->ta);
  if (st != VSK_OK) {
    vsk_kmeans_trainer_destroy(reinterpret_cast<vsk_kmeans_trainer*>(t));
    return st;
  }
  *out = reinterpret_cast<vsk_kmeans_trainer*>(t);
  return VSK_OK;
}

int32_t vsk_kmeans_trainer_step_dev(vsk_kmeans_trainer* h, const float* centroids, float* sums, float* counts,
                                    float* inertia) {
  VSK_TRACE("vsk_kmeans_trainer_step_dev");
  KMeansTrainer* t = reinterpret_cast<KMeansTrainer*>(h);
  if (!t) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(t->ctx->device);
  if (!centroids || !sums || !counts || !inertia) return fail(t->ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  return trainer_step(t, centroids, sums, counts, inertia);
}

int32_t vsk_kmeans_trainer_assignments_dev(vsk_kmeans_trainer* h, int32_t* assign) {
  KMeansTrainer* t = reinterpret_cast<KMeansTrainer*>(h);
  if (!t || !assign) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(t->ctx->device);
  VSK_CUDA(t->ctx, cudaMemcpyAsync(assign, t->assign, (size_t)t->n * 4, cudaMemcpyDeviceToDevice, t->ctx->stream));
  VSK_CUDA(t->ctx, cudaStreamSynchronize(t->ctx->stream));
  return VSK_OK;
}

int32_t vsk_kmeans_trainer_destroy(vsk_kmeans_trainer* h) {
  KMeansTrainer* t = reinterpret_cast<KMeansTrainer*>(h);
  if (!t) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(t->ctx->device);
  cudaStreamSynchronize(t->ctx->stream);
  if (t->tc) tensor_assign_release(&t->ta);
  dev_free(t->assign);
  dev_free(t->dist);
  dev_free(t->order);
  delete t;
  return VSK_OK;
}

int32_t vsk_kmeans_finish_dev(vsk_ctx* c, const float* sums, const float* counts, const float* prev_centroids, int32_t k,
                              int32_t dim, float* centroids) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (k <= 0 || dim <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no centroids");
  if (!sums || !counts || !prev_centroids || !centroids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  const int64_t total = (int64_t)k * dim;
  centroid_mean_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, ctx->stream>>>(sums, counts, total, dim, prev_centroids, centroids);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_kmeans_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t k, int32_t max_iters,
                       float tolerance, const float* init, float* centroids, int32_t* assign, float* inertia,
                       int32_t* iters_run) {
  VSK_TRACE("vsk_kmeans_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  return kmeans_dev(ctx, rows, n, dim, k, max_iters, tolerance, init, centroids, assign, inertia, iters_run);
}

int32_t vsk_kmeans(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t k, int32_t max_iters,
                   float tolerance, const float* init, float* centroids, int32_t* assign, float* inertia,
                   int32_t* iters_run) {
  VSK_TRACE("vsk_kmeans");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty dataset");
  if (k <= 0 || k > n) return fail(ctx, VSK_ERR_INSUFFICIENT_TRAINING_DATA, "k = %d needs 1 <= k <= %lld rows", k, (long long)n);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !init || !centroids || !assign) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  float *dx = nullptr, *dinit = nullptr, *dcent = nullptr;
  int32_t* dassign = nullptr;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&dx, (size_t)n * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dinit, (size_t)k * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dcent, (size_t)k * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dassign, (size_t)n * 4)) == VSK_OK) {
    cudaMemcpyAsync(dx, rows, (size_t)n * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    cudaMemcpyAsync(dinit, init, (size_t)k * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    st = kmeans_dev(ctx, dx, n, dim, k, max_iters, tolerance, dinit, dcent, dassign, inertia, iters_run);
    if (st == VSK_OK) {
      cudaMemcpy(centroids, dcent, (size_t)k * dim * 4, cudaMemcpyDeviceToHost);
      cudaError_t e = cudaMemcpy(assign, dassign, (size_t)n * 4, cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "copy out failed: %s", cudaGetErrorString(e));
    }
  }
  dev_free(dx);
  dev_free(dinit);
  dev_free(dcent);
  dev_free(dassign);
  return st;
}

int32_t vsk_assign_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                       int32_t* assign, float* dist) {
  VSK_TRACE("vsk_assign_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (n <= 0 || k <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty rows or centroids");
  if (!rows || !centroids || !assign) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  VSK_TRY(assign_rows(ctx, rows, n, dim, centroids, k, assign, dist));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_assign_static_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, const float* centroids,
                              int32_t k, int32_t* assign, float* dist) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (n <= 0 || k <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty rows or centroids");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !centroids || !assign) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  if (n > kAssignStaticMaxRows)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE,
                "vsk_assign_static_dev handles at most %lld rows per call (got %lld): split the rows, or use "
                "vsk_assign_dev, which allocates its scratch",
                (long long)kAssignStaticMaxRows, (long long)n);
  VSK_TRY(assign_rows_static(ctx, rows, n, dim, centroids, k, assign, dist));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // extern "C"
