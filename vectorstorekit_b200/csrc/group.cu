// Stable grouping (counting sort) of items by a small integer key, used to turn row -> cluster
// assignments into cluster-major row lists (k-means update in row order, inverted lists in
// insertion order, probe tables grouped by list).  Deterministic: no floating point, and the only
// atomics are absent — every counter has a single writer.
//
// Items are cut into segments; one warp walks one segment in item order.  Pass 1 counts keys per
// segment, pass 2 turns the per-segment counts into starting positions (scan over segments, then
// over keys), pass 3 walks the segment again and hands out positions in item order.
#include "common.cuh"

namespace vsk {
namespace {

__device__ __forceinline__ void seg_walk(const int32_t* __restrict__ keys, int64_t begin, int64_t end,
                                         int32_t* __restrict__ row, const int64_t* __restrict__ offsets,
                                         int32_t* __restrict__ order) {
  const int lane = threadIdx.x & 31;
  for (int64_t base = begin; base < end; base += 32) {
    const int64_t i = base + lane;
    const bool valid = i < end;
    const int key = valid ? keys[i] : (int)(0x80000000u | lane);
    const unsigned mask = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(mask & ((1u << lane) - 1));
    const bool leader = rank == 0;
    if (valid) {
      const int cur = row[key];
      if (order) order[offsets[key] + cur + rank] = (int32_t)i;
      __syncwarp(mask);
      if (leader) row[key] = cur + __popc(mask);
    }
    __syncwarp();
  }
}

__global__ void seg_count_kernel(const int32_t* keys, int64_t n, int64_t seg_len, int32_t nkeys, int32_t* table) {
  const int64_t seg = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t begin = seg * seg_len;
  if (begin >= n) return;
  seg_walk(keys, begin, min(n, begin + seg_len), table + seg * nkeys, nullptr, nullptr);
}

__global__ void seg_scatter_kernel(const int32_t* keys, int64_t n, int64_t seg_len, int32_t nkeys, int32_t* table,
                                   const int64_t* offsets, int32_t* order) {
  const int64_t seg = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t begin = seg * seg_len;
  if (begin >= n) return;
  seg_walk(keys, begin, min(n, begin + seg_len), table + seg * nkeys, offsets, order);
}

// per key: exclusive scan of the segment counts; totals[key] = items with that key.  Eight segments per step so
// that the loads of a step are independent (the walk is otherwise one memory latency per segment).
__global__ void seg_scan_kernel(int32_t* table, int64_t nseg, int32_t nkeys, int64_t* totals) {
  const int key = blockIdx.x * blockDim.x + threadIdx.x;
  if (key >= nkeys) return;
  int64_t run = 0;
  int64_t s = 0;
  for (; s + 8 <= nseg; s += 8) {
    int32_t t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = table[(s + u) * nkeys + key];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      table[(s + u) * nkeys + key] = (int32_t)run;
      run += t[u];
    }
  }
  for (; s < nseg; ++s) {
    const int32_t t = table[s * nkeys + key];
    table[s * nkeys + key] = (int32_t)run;
    run += t;
  }
  totals[key] = run;
}

// offsets[0..nkeys] = exclusive scan of totals (single block; nkeys is small)
__global__ void key_scan_kernel(const int64_t* totals, int32_t nkeys, int64_t* offsets) {
  __shared__ int64_t carry;
  __shared__ int64_t buf[1024];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < nkeys; base += 1024) {
    const int i = base + threadIdx.x;
    const int64_t v = i < nkeys ? totals[i] : 0;
    buf[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int64_t t = threadIdx.x >= o ? buf[threadIdx.x - o] : 0;
      __syncthreads();
      buf[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < nkeys) offsets[i] = carry + buf[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += buf[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[nkeys] = carry;
}

}  // namespace

int32_t launch_scan_i64(Ctx* ctx, const int64_t* totals, int32_t n, int64_t* offsets) {
  key_scan_kernel<<<1, 1024, 0, ctx->stream>>>(totals, n, offsets);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t launch_stable_group(Ctx* ctx, const int32_t* keys, int64_t n, int32_t nkeys, int32_t* order,
                            int64_t* offsets) {
  if (n <= 0 || nkeys <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "nothing to group");
  // Segment length: a warp walks its segment 32 items per step, each step one dependent read-modify-write of its
  // counters, so short segments (many warps) are what makes a small grouping fast; the count table (segments x keys)
  // bounds them from below: at most 8 M entries for the sake of the scan over it, 1 024 to 4 096 items otherwise
  // (about 1 000 segments when there are enough items).
  int64_t seg_len = std::min<int64_t>(4096, std::max<int64_t>(1024, ceil_div(n, 1024)));
  seg_len = std::max<int64_t>(seg_len, ceil_div(n * (int64_t)nkeys, 8ll << 20));
  seg_len = ceil_div(seg_len, 32) * 32;
  const int64_t nseg = ceil_div(n, seg_len);
  void *table, *totals;
  VSK_TRY(scratch(ctx, SLOT_MISC5, (size_t)nseg * nkeys * sizeof(int32_t), &table));
  VSK_TRY(scratch(ctx, SLOT_MISC6, (size_t)nkeys * sizeof(int64_t), &totals));
  VSK_CUDA(ctx, cudaMemsetAsync(table, 0, (size_t)nseg * nkeys * sizeof(int32_t), ctx->stream));
  const int warps = 4;
  const unsigned blocks = (unsigned)ceil_div(nseg, warps);
  seg_count_kernel<<<blocks, warps * 32, 0, ctx->stream>>>(keys, n, seg_len, nkeys, (int32_t*)table);
  seg_scan_kernel<<<(unsigned)ceil_div(nkeys, 128), 128, 0, ctx->stream>>>((int32_t*)table, nseg, nkeys, (int64_t*)totals);
  key_scan_kernel<<<1, 1024, 0, ctx->stream>>>((const int64_t*)totals, nkeys, offsets);
  seg_scatter_kernel<<<blocks, warps * 32, 0, ctx->stream>>>(keys, n, seg_len, nkeys, (int32_t*)table, offsets, order);
  ctx->stats.kernel_launches += 4;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

}  // namespace vsk
