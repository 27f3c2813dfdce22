// Per-query selection over the candidate lists, one CTA per query.
//   compaction  the list's 64-bit (value, row) keys are held in registers (8 per thread); a block-wide
//               radix select finds the key of rank `keep`, every key at or below it is written back
//               (unordered) and its value becomes the query's threshold
//   final       the short list left by the last compaction is sorted in shared memory (bitonic
//               network) and written out as the ascending top-k  Replaces the reference's CPU-side `sorted().prefix(k)` per query
// (Acceleration/MetalAccelerationEngine.swift:465-471).
#include <math_constants.h>

#include "common.cuh"

namespace vsk {
namespace {

constexpr int SEL_THREADS = 512;   // widest variant: 512 threads x 8 keys = the full list capacity

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

constexpr int SEL_ITEMS = 8;  // keys per thread, held in registers

// Block-wide radix select over the 64-bit keys each thread holds: returns the key of rank `rank`
// (1-based, ascending).  One pass per byte from the top; a pass histograms the byte among the keys that
// still match the decided prefix.  After the four value bytes, if the rest of the rank is made up of ALL
// keys with exactly that value, the id bytes need not be resolved and the pivot is (value, max id).
//
// Fast path first.  The values of one list sit in a narrow band (everything at or below the query's threshold), so the
// top bytes of the keys are the same for all of them and byte-wise passes from the top spend two of their four rounds
// learning nothing.  The fast path takes the smallest value v0 of the list, histograms the 8 most significant bits in
// which (value - v0) varies, and descends 8 bits at a time inside the bin that holds the rank until that bin has at
// most 32 keys; those go to shared memory and one warp finds the wanted one by counting, for every key, the keys
// below it.  Typical lists (a few hundred keys) need one histogram.  A bin of more than 32 keys that share their
// whole 32-bit value (bulk ties) falls back to the byte-wise passes below, which also resolve the row bits.
__device__ __forceinline__ uint64_t block_radix_select(const uint64_t (&key)[SEL_ITEMS], int rank, int* hist,
                                                       int* s_bin, int* s_less, int* s_in_bin) {
  __shared__ unsigned f_min, f_max;
  __shared__ int f_n;
  __shared__ unsigned long long f_small[32];
  __shared__ unsigned long long f_pivot;
  {
    unsigned lo = 0xffffffffu, hi = 0u;
#pragma unroll
    for (int i = 0; i < SEL_ITEMS; ++i)
      if (key[i] != kEmptyKey) {
        const unsigned v = (unsigned)(key[i] >> 32);
        lo = min(lo, v);
        hi = max(hi, v);
      }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    if (threadIdx.x == 0) { f_min = 0xffffffffu; f_max = 0u; f_n = 0; }
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { atomicMin(&f_min, lo); atomicMax(&f_max, hi); }
    __syncthreads();
    const unsigned v0 = f_min, range = f_max - v0;
    if (f_max >= v0 && range != 0u) {
      int shift = max(0, 32 - __clz(range) - 8);   // the digit of the first level: (u >> shift), at most 8 bits
      int width = 32 - __clz(range) - shift;
      unsigned prefix = 0u;                        // u >> (shift + width) of the keys still in play
      int r = rank;
      for (int level = 0;; ++level) {
        const unsigned dmask = (1u << width) - 1u;
#pragma unroll
        for (int i = 0; i < SEL_ITEMS; ++i)
          if (key[i] != kEmptyKey) {
            const unsigned u = (unsigned)(key[i] >> 32) - v0;
            if (level == 0 || (u >> (shift + width)) == prefix) atomicAdd(&hist[(u >> shift) & dmask], 1);
          }
        __syncthreads();
        if (threadIdx.x < 32) {
          int local[8], sum = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) { local[j] = hist[threadIdx.x * 8 + j]; sum += local[j]; }
          int incl = sum;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)threadIdx.x >= o) incl += t;
          }
          int before = incl - sum;
          if (before < r && r <= incl) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (before < r && r <= before + local[j]) {
                *s_bin = threadIdx.x * 8 + j;
                *s_less = before;
                *s_in_bin = local[j];
              }
              before += local[j];
            }
          }
        }
        __syncthreads();
        const int bin = *s_bin, less = *s_less, in_bin = *s_in_bin;
        r -= less;
        const unsigned want = (level == 0 ? 0u : (prefix << width)) | (unsigned)bin;   // u >> shift of the bin's keys
        if (in_bin <= 32) {
#pragma unroll
          for (int i = 0; i < SEL_ITEMS; ++i)
            if (key[i] != kEmptyKey && (((unsigned)(key[i] >> 32) - v0) >> shift) == want)
              f_small[atomicAdd(&f_n, 1)] = key[i];
          __syncthreads();
          if (threadIdx.x < 32) {
            const unsigned long long mine = (int)threadIdx.x < in_bin ? f_small[threadIdx.x] : kEmptyKey;
            int below = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) below += __shfl_sync(0xffffffffu, mine, j) < mine;
            if ((int)threadIdx.x < in_bin && below == r - 1) f_pivot = mine;
          }
          __syncthreads();
          return f_pivot;
        }
        if (shift == 0) break;   // more than 32 keys with one and the same value: the byte-wise passes resolve the rows
        prefix = want;
        width = min(8, shift);
        shift -= width;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
      }
    }
  }
  uint64_t prefix = 0, mask = 0;
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < SEL_ITEMS; ++i)
      if ((key[i] & mask) == prefix) atomicAdd(&hist[(int)((key[i] >> shift) & 255)], 1);
    __syncthreads();
    if (threadIdx.x < 32) {
      // lane l owns bins 8l .. 8l+7
      int local[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { local[j] = hist[threadIdx.x * 8 + j]; sum += local[j]; }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)threadIdx.x >= o) incl += t;
      }
      int before = incl - sum;
      if (before < rank && rank <= incl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (before < rank && rank <= before + local[j]) {
            *s_bin = threadIdx.x * 8 + j;
            *s_less = before;
            *s_in_bin = local[j];
          }
          before += local[j];
        }
      }
    }
    __syncthreads();
    const int bin = *s_bin, less = *s_less, in_bin = *s_in_bin;
    __syncthreads();
    rank -= less;
    prefix |= (uint64_t)bin << shift;
    mask |= (uint64_t)255 << shift;
    if (shift == 32 && in_bin == rank) return prefix | 0xffffffffull;  // every key with this value is taken
  }
  return prefix;
}

// NT threads handle a list of at most NT * 8 keys.  The host picks NT from an upper bound on the list
// lengths of the launch (SelectArgs::max_count); a list that is longer all the same is flagged like an
// overflowed list and its query is re-run.
template <int NT>
__global__ void __launch_bounds__(NT, NT == 128 ? 10 : 2) select_kernel(SelectArgs a) {
  extern __shared__ __align__(16) uint64_t s[];
  constexpr int CAPACITY = NT * SEL_ITEMS;
  __shared__ int hist[256];
  __shared__ int s_valid, s_bin, s_less, s_in_bin, s_out;
  const int64_t q = blockIdx.x;
  uint64_t* keys = a.cand.keys + q * kCandCap;
  int c;
  if (a.dense_count >= 0) {
    c = a.dense_count;
  } else {
    const int raw = a.cand.count[q];
    c = min(raw, CAPACITY);
    if (raw > CAPACITY && threadIdx.x == 0) atomicOr(&a.cand.flags[q], 1);
  }
  c = min(c, CAPACITY);

  if (a.out_ids != nullptr) {
    // ---- final order: sort the (short) list in shared memory and write the ascending top-k ----
    const int P = next_pow2(c);
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
      uint64_t key = i < c ? keys[i] : kEmptyKey;
      if (a.id_remap != nullptr && key != kEmptyKey)
        key = (key & 0xffffffff00000000ull) | (uint32_t)a.id_remap[(uint32_t)key];
      s[i] = key;
    }
    if (threadIdx.x == 0) s_valid = 0;
    __syncthreads();
    bitonic_sort(s, P);
    for (int i = threadIdx.x; i < P; i += blockDim.x)
      if (s[i] != kEmptyKey && (i + 1 == P || s[i + 1] == kEmptyKey)) s_valid = i + 1;
    __syncthreads();
    const int valid = s_valid;
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
    return;
  }

  // ---- compaction: keys in registers, radix select of the pivot, keep everything at or below it ----
  uint64_t key[SEL_ITEMS];
  int nvalid = 0;
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i) {
    const int idx = threadIdx.x + i * NT;
    key[i] = idx < c ? keys[idx] : kEmptyKey;
    nvalid += key[i] != kEmptyKey;
  }
  if (threadIdx.x == 0) { s_valid = 0; s_out = 0; }
  __syncthreads();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) nvalid += __shfl_xor_sync(0xffffffffu, nvalid, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_valid, nvalid);
  __syncthreads();
  const int valid = s_valid;

  if (a.bound_out != nullptr) {
    // Measure only (a shard's half-way point): c_j + eps bounds the exact value of this shard's j best rows from
    // above.  The list stays as it is; a dense list gets its count written for the compaction that follows.
    float b = CUDART_INF_F;
    if (valid >= a.bound_rank) {
      const uint64_t jth = block_radix_select(key, a.bound_rank, hist, &s_bin, &s_less, &s_in_bin);
      b = ordered_to_float((uint32_t)(jth >> 32)) + a.bound_eps[q];
    }
    if (threadIdx.x == 0) {
      a.bound_out[q] = b;
      if (a.dense_count >= 0) a.cand.count[q] = c;
    }
    return;
  }

  uint64_t pivot = kEmptyKey - 1;  // keep every real key
  if (a.cert_eps != nullptr) {
    // Last compaction of a coarse (bounded-error) scan.  Let c_k be the k-th smallest coarse value and
    // eps the query's error bound: a row of the true top-k has coarse value <= c_k + 2 eps, so those
    // rows are kept for the exact re-scoring.  The list is complete only below the threshold t that
    // filtered the scan, so the result can be certified only if c_k + 2 eps < t.
    // A sharded search also knows a value g that at least k rows over all shards do not exceed (exactly): rows of
    // the overall top-k then have coarse value <= g + eps, and only those are kept.
    float bound = CUDART_INF_F;
    bool have = false;
    if (valid >= a.k) {
      const uint64_t kth = block_radix_select(key, a.k, hist, &s_bin, &s_less, &s_in_bin);
      bound = ordered_to_float((uint32_t)(kth >> 32)) + 2.0f * a.cert_eps[q];
      have = true;
    }
    if (a.ext_bound != nullptr && a.ext_bound[q] < CUDART_INF_F) {
      bound = fminf(bound, a.ext_bound[q] + a.cert_eps[q]);
      have = true;
    }
    if (have) {
      pivot = ((uint64_t)float_to_ordered(bound) << 32) | 0xffffffffull;
      if (pivot == kEmptyKey) pivot = kEmptyKey - 1;
      if (threadIdx.x == 0 && !(bound < a.cand.thr[q])) atomicOr(&a.cand.flags[q], 2);
    }
  } else if (valid > a.keep) {
    pivot = block_radix_select(key, a.keep, hist, &s_bin, &s_less, &s_in_bin);
    // the keep-th smallest value becomes the query's threshold
    if (threadIdx.x == 0) a.cand.thr[q] = ordered_to_float((uint32_t)(pivot >> 32));
  } else if (valid == a.keep && a.keep > 0) {
    // exactly `keep` real keys: nothing to drop, but the threshold may tighten to their largest value
    const uint64_t last = block_radix_select(key, a.keep, hist, &s_bin, &s_less, &s_in_bin);
    if (threadIdx.x == 0) a.cand.thr[q] = ordered_to_float((uint32_t)(last >> 32));
  }
  // every thread has loaded its keys (barriers above), so the list can be rewritten in place
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i) {
    if (key[i] <= pivot && key[i] != kEmptyKey) {
      const int pos = atomicAdd(&s_out, 1);
      keys[pos] = key[i];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) a.cand.count[q] = s_out;
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

// The same merge for at most 1024 gathered keys per query: the keys stay in registers (128 threads x 8), a
// radix select finds the k-th, and only the k survivors are sorted — instead of sorting all g*k keys.
__global__ void __launch_bounds__(128) merge_select_kernel(const float* __restrict__ dist, const int64_t* __restrict__ ids,
                                                           int g, int64_t nq, int k, float* out_dist, int64_t* out_ids) {
  __shared__ __align__(16) uint64_t s[128 * SEL_ITEMS];
  __shared__ int hist[256];
  __shared__ int s_valid, s_bin, s_less, s_in_bin, s_out;
  const int64_t q = blockIdx.x;
  const int c = g * k;
  uint64_t key[SEL_ITEMS];
  int nvalid = 0;
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i) {
    const int idx = threadIdx.x + i * 128;
    key[i] = kEmptyKey;
    if (idx < c) {
      const int sh = idx / k, j = idx - sh * k;
      const int64_t src = ((int64_t)sh * nq + q) * k + j;
      if (ids[src] >= 0) key[i] = make_key(dist[src], (uint32_t)idx);
    }
    nvalid += key[i] != kEmptyKey;
  }
  if (threadIdx.x == 0) { s_valid = 0; s_out = 0; }
  __syncthreads();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) nvalid += __shfl_xor_sync(0xffffffffu, nvalid, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_valid, nvalid);
  __syncthreads();
  const int valid = s_valid;
  uint64_t pivot = kEmptyKey - 1;
  if (valid > k) pivot = block_radix_select(key, k, hist, &s_bin, &s_less, &s_in_bin);
  const int P = next_pow2(min(valid, 128 * SEL_ITEMS));
  for (int i = threadIdx.x; i < P; i += blockDim.x) s[i] = kEmptyKey;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i)
    if (key[i] <= pivot && key[i] != kEmptyKey) s[atomicAdd(&s_out, 1)] = key[i];
  __syncthreads();
  const int kept = s_out;          // k, or more when the k-th value is tied across keys that were all taken
  const int PS = next_pow2(kept);
  bitonic_sort(s, PS);
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    float d = CUDART_INF_F;
    int64_t id = -1;
    if (j < kept) {
      const int i = (int)(uint32_t)s[j];
      const int sh = i / k, jj = i - sh * k;
      const int64_t src = ((int64_t)sh * nq + q) * k + jj;
      d = dist[src];
      id = ids[src];
    }
    out_dist[q * k + j] = d;
    out_ids[q * k + j] = id;
  }
}

// ---- packed (distance, global row) keys: what shards exchange -----------------------------------------------
// A result entry as one 64-bit word, ordered(distance) << 32 | global row, so that unsigned order is (distance,
// global row) order - the order an unsharded search returns - whatever shard an entry came from.  A missing entry
// (id -1) is the all-ones key.  Rows beyond `nq` (padding to whole slices) are filled with missing entries.
__global__ void pack_keys_kernel(const float* __restrict__ dist, const int64_t* __restrict__ ids, int64_t nq, int64_t rows,
                                 int k, uint64_t* __restrict__ keys) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * k) return;
  uint64_t key = kEmptyKey;
  if (i < nq * k) {
    const int64_t id = ids[i];
    if (id >= 0) key = make_key(dist[i], (uint32_t)id);
  }
  keys[i] = key;
}

__global__ void unpack_keys_kernel(const uint64_t* __restrict__ keys, int64_t count, float* __restrict__ dist,
                                   int64_t* __restrict__ ids) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint64_t key = keys[i];
  dist[i] = key == kEmptyKey ? CUDART_INF_F : ordered_to_float((uint32_t)(key >> 32));
  ids[i] = key == kEmptyKey ? -1 : (int64_t)(uint32_t)key;
}

// Merge of g lists of k keys per query ([g][stride_q][k], query q of this launch at row q): the k smallest keys,
// ascending, to out[q][k].  One CTA per query: the keys stay in registers, a radix select finds the k-th, only the
// survivors are sorted.
template <int NT>
__global__ void __launch_bounds__(NT) merge_keys_kernel(const uint64_t* __restrict__ in, int g, int64_t stride_q, int k,
                                                        uint64_t* __restrict__ out) {
  __shared__ __align__(16) uint64_t s[NT * SEL_ITEMS];
  __shared__ int hist[256];
  __shared__ int s_valid, s_bin, s_less, s_in_bin, s_out;
  const int64_t q = blockIdx.x;
  const int c = g * k;
  uint64_t key[SEL_ITEMS];
  int nvalid = 0;
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i) {
    const int idx = threadIdx.x + i * NT;
    key[i] = kEmptyKey;
    if (idx < c) {
      const int sh = idx / k, j = idx - sh * k;
      key[i] = in[((int64_t)sh * stride_q + q) * k + j];
    }
    nvalid += key[i] != kEmptyKey;
  }
  if (threadIdx.x == 0) { s_valid = 0; s_out = 0; }
  __syncthreads();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) nvalid += __shfl_xor_sync(0xffffffffu, nvalid, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_valid, nvalid);
  __syncthreads();
  const int valid = s_valid;
  uint64_t pivot = kEmptyKey - 1;
  // keys are distinct (a global row appears once), so the select resolves all 64 bits and exactly k survive
  if (valid > k) pivot = block_radix_select(key, k, hist, &s_bin, &s_less, &s_in_bin);
  const int P = next_pow2(max(min(valid, k), 1));
  for (int i = threadIdx.x; i < P; i += blockDim.x) s[i] = kEmptyKey;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < SEL_ITEMS; ++i)
    if (key[i] <= pivot && key[i] != kEmptyKey) {
      const int pos = atomicAdd(&s_out, 1);
      if (pos < P) s[pos] = key[i];
    }
  __syncthreads();
  bitonic_sort(s, P);
  for (int j = threadIdx.x; j < k; j += blockDim.x) out[q * k + j] = j < P ? s[j] : kEmptyKey;
}

}  // namespace

int32_t launch_pack_keys(Ctx* ctx, const float* dist, const int64_t* ids, int64_t nq, int64_t rows, int32_t k,
                         uint64_t* keys) {
  if (rows <= 0) return VSK_OK;
  pack_keys_kernel<<<(unsigned)ceil_div(rows * k, 256), 256, 0, ctx->stream>>>(dist, ids, nq, rows, k, keys);
  tl_mark(ctx, "pack_keys");
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_unpack_keys(Ctx* ctx, const uint64_t* keys, int64_t count, float* dist, int64_t* ids) {
  if (count <= 0) return VSK_OK;
  unpack_keys_kernel<<<(unsigned)ceil_div(count, 256), 256, 0, ctx->stream>>>(keys, count, dist, ids);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_merge_keys(Ctx* ctx, const uint64_t* in, int32_t g, int64_t stride_q, int64_t nq, int32_t k, uint64_t* out) {
  if (nq <= 0) return VSK_OK;
  if ((int64_t)g * k > kCandCap)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "merge of %d lists of %d exceeds %d keys", g, k, kCandCap);
  if (g * k <= 128 * SEL_ITEMS)
    merge_keys_kernel<128><<<(unsigned)nq, 128, 0, ctx->stream>>>(in, g, stride_q, k, out);
  else
    merge_keys_kernel<SEL_THREADS><<<(unsigned)nq, SEL_THREADS, 0, ctx->stream>>>(in, g, stride_q, k, out);
  tl_mark(ctx, "merge_keys");
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_select(Ctx* ctx, const SelectArgs& a) {
  if (a.nq <= 0) return VSK_OK;
  // lists known to hold at most 1024 keys take the 128-thread variant (four times as many CTAs per SM);
  // only the final ordering sorts in shared memory
  const bool small = a.max_count > 0 && a.max_count <= 128 * SEL_ITEMS && (a.dense_count < 0 || a.dense_count <= 128 * SEL_ITEMS);
  static bool carveout_done = false;
  if (!carveout_done) {
    prefer_shared_carveout(select_kernel<128>);
    prefer_shared_carveout(select_kernel<SEL_THREADS>);
    prefer_shared_carveout(init_cand_kernel);
    prefer_shared_carveout(pack_keys_kernel);
    prefer_shared_carveout(unpack_keys_kernel);
    prefer_shared_carveout(merge_keys_kernel<128>);
    prefer_shared_carveout(merge_keys_kernel<SEL_THREADS>);
    carveout_done = true;
  }
  if (small) {
    const size_t smem = a.out_ids ? 128 * SEL_ITEMS * sizeof(uint64_t) : 0;
    select_kernel<128><<<(unsigned)a.nq, 128, smem, ctx->stream>>>(a);
  } else {
    const size_t smem = a.out_ids ? kCandCap * sizeof(uint64_t) : 0;
    select_kernel<SEL_THREADS><<<(unsigned)a.nq, SEL_THREADS, smem, ctx->stream>>>(a);
  }
  tl_mark(ctx, a.out_ids ? "final_order" : (a.bound_out ? "bound_select" : (a.cert_eps ? "certify_select" : "select")));
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
  if (g * k <= 128 * SEL_ITEMS)
    merge_select_kernel<<<(unsigned)nq, 128, 0, ctx->stream>>>(dist, ids, g, nq, k, out_dist, out_ids);
  else
    merge_kernel<<<(unsigned)nq, SEL_THREADS, P * sizeof(uint64_t), ctx->stream>>>(dist, ids, g, nq, k, out_dist, out_ids);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

}  // namespace vsk
