// Per-query selection over the candidate lists: one CTA per query sorts the list's 64-bit
// (value, row) keys in shared memory (bitonic network, at most 4096 keys = 32 KB), then either
// compacts the list to its best `keep` keys and tightens the query's threshold, or writes the
// final ascending top-k.  Replaces the reference's CPU-side `sorted().prefix(k)` per query
// (Acceleration/MetalAccelerationEngine.swift:465-471).
#include <math_constants.h>

#include "common.cuh"

namespace vsk {
namespace {

constexpr int SEL_THREADS = 512;

__device__ __forceinline__ void bitonic_sort(uint64_t* s, int P) {
  for (int size = 2; size <= P; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (P >> 1); t += blockDim.x) {
        int pos = 2 * t - (t & (stride - 1));
        int par = pos + stride;
        bool up = (pos & size) == 0;
        uint64_t x = s[pos], y = s[par];
        if ((x > y) == up) { s[pos] = y; s[par] = x; }
      }
      __syncthreads();
    }
  }
}

__device__ __forceinline__ int next_pow2(int c) {
  int p = 2;
  while (p < c) p <<= 1;
  return p;
}

__global__ void __launch_bounds__(SEL_THREADS) select_kernel(SelectArgs a) {
  extern __shared__ __align__(16) uint64_t s[];
  __shared__ int s_valid;
  const int64_t q = blockIdx.x;
  uint64_t* keys = a.cand.keys + q * kCandCap;
  int c;
  if (a.dense_count >= 0) {
    c = a.dense_count;
  } else {
    int raw = a.cand.count[q];
    c = min(raw, kCandCap);
    if (raw > kCandCap && threadIdx.x == 0) atomicOr(&a.cand.flags[q], 1);
  }
  const int P = next_pow2(c);
  for (int i = threadIdx.x; i < P; i += blockDim.x) s[i] = i < c ? keys[i] : kEmptyKey;
  if (threadIdx.x == 0) s_valid = 0;
  __syncthreads();
  bitonic_sort(s, P);
  for (int i = threadIdx.x; i < P; i += blockDim.x)
    if (s[i] != kEmptyKey && (i + 1 == P || s[i + 1] == kEmptyKey)) s_valid = i + 1;
  __syncthreads();
  const int valid = s_valid;

  if (a.cert_eps != nullptr) {
    // Last compaction of a coarse (bounded-error) scan.  Let c_k be the k-th smallest coarse value and
    // eps the query's error bound: a row of the true top-k has coarse value <= c_k + 2 eps, so those
    // rows are kept for the exact re-scoring.  The list is complete only below the threshold t that
    // filtered the scan, so the result can be certified only if c_k + 2 eps < t.
    int kept = valid;
    if (valid >= a.k) {
      const float bound = ordered_to_float((uint32_t)(s[a.k - 1] >> 32)) + 2.0f * a.cert_eps[q];
      // first index whose value exceeds the bound (the list is sorted)
      int lo = a.k, hi = valid;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (ordered_to_float((uint32_t)(s[mid] >> 32)) <= bound) lo = mid + 1; else hi = mid;
      }
      kept = lo;
      if (threadIdx.x == 0 && !(bound < a.cand.thr[q])) atomicOr(&a.cand.flags[q], 2);
    }
    for (int i = threadIdx.x; i < kept; i += blockDim.x) keys[i] = s[i];
    if (threadIdx.x == 0) a.cand.count[q] = kept;
  } else if (a.out_ids == nullptr) {
    const int kept = min(a.keep, valid);
    for (int i = threadIdx.x; i < kept; i += blockDim.x) keys[i] = s[i];
    if (threadIdx.x == 0) {
      a.cand.count[q] = kept;
      // The threshold only tightens once `keep` real candidates exist.
      if (valid >= a.keep) a.cand.thr[q] = ordered_to_float((uint32_t)(s[a.keep - 1] >> 32));
    }
  } else {
    const int64_t qo = a.q_subset ? (int64_t)a.q_subset[q] : q;
    for (int j = threadIdx.x; j < a.k; j += blockDim.x) {
      float d = CUDART_INF_F;
      int64_t id = -1;
      if (j < valid) {
        d = ordered_to_float((uint32_t)(s[j] >> 32));
        if (a.final_sqrt) d = sqrtf(d);
        id = (int64_t)(uint32_t)s[j] + a.id_base;
      }
      a.out_dist[qo * a.k + j] = d;
      a.out_ids[qo * a.k + j] = id;
    }
  }
}

__global__ void init_cand_kernel(CandLists c, int64_t nq) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nq) {
    c.count[i] = 0;
    c.thr[i] = CUDART_INF_F;
    c.flags[i] = 0;
  }
}

// Merge of g per-shard lists per query.  Shards are ordered by ascending first global row and
// each list is already (distance, id)-ascending, so (distance, shard, position) order equals
// (distance, global id) order.
__global__ void __launch_bounds__(SEL_THREADS) merge_kernel(const float* __restrict__ dist,
                                                           const int64_t* __restrict__ ids, int g,
                                                           int64_t nq, int k, float* out_dist,
                                                           int64_t* out_ids) {
  extern __shared__ __align__(16) uint64_t s[];
  const int64_t q = blockIdx.x;
  const int c = g * k;
  const int P = next_pow2(c);
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    uint64_t key = kEmptyKey;
    if (i < c) {
      int sh = i / k, j = i - sh * k;
      int64_t src = ((int64_t)sh * nq + q) * k + j;
      if (ids[src] >= 0) key = make_key(dist[src], (uint32_t)i);
    }
    s[i] = key;
  }
  __syncthreads();
  bitonic_sort(s, P);
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    float d = CUDART_INF_F;
    int64_t id = -1;
    if (j < P && s[j] != kEmptyKey) {
      int i = (int)(uint32_t)s[j];
      int sh = i / k, jj = i - sh * k;
      int64_t src = ((int64_t)sh * nq + q) * k + jj;
      d = dist[src];
      id = ids[src];
    }
    out_dist[q * k + j] = d;
    out_ids[q * k + j] = id;
  }
}

}  // namespace

int32_t launch_select(Ctx* ctx, const SelectArgs& a) {
  if (a.nq <= 0) return VSK_OK;
  select_kernel<<<(unsigned)a.nq, SEL_THREADS, kCandCap * sizeof(uint64_t), ctx->stream>>>(a);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_init_cand(Ctx* ctx, const CandLists& c, int64_t nq) {
  if (nq <= 0) return VSK_OK;
  init_cand_kernel<<<(unsigned)ceil_div(nq, 256), 256, 0, ctx->stream>>>(c, nq);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_merge_topk(Ctx* ctx, const float* dist, const int64_t* ids, int32_t g, int64_t nq,
                          int32_t k, float* out_dist, int64_t* out_ids) {
  if (nq <= 0) return VSK_OK;
  if ((int64_t)g * k > kCandCap)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "merge of %d lists of %d exceeds %d keys", g, k, kCandCap);
  int P = 2;
  while (P < g * k) P <<= 1;
  merge_kernel<<<(unsigned)nq, SEL_THREADS, P * sizeof(uint64_t), ctx->stream>>>(dist, ids, g, nq, k,
                                                                                   out_dist, out_ids);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

}  // namespace vsk
