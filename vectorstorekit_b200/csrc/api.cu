// C ABI: context, flat fp32 index, stateless distances, merge.  The search schedule lives here:
// how a batch of queries walks the resident database in chunks, with per-query thresholds that
// tighten between chunks so that only a few thousand of the N values per query ever leave the
// scan kernels.
#include <cstdarg>
#include <cstdio>
#include <cmath>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <functional>
#include <math_constants.h>

#include "common.cuh"
#include "tensor_scan.cuh"

namespace vsk {

int32_t fail(Ctx* ctx, int32_t status, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return status;
}

int32_t dev_alloc(Ctx* ctx, void** p, size_t bytes) {
  *p = nullptr;
  if (bytes == 0) return VSK_OK;
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) {
    size_t fr = 0, tot = 0;
    cudaMemGetInfo(&fr, &tot);
    cudaGetLastError();
    return fail(ctx, VSK_ERR_OUT_OF_MEMORY, "device out of memory: required %zu bytes, available %zu", bytes, fr);
  }
  chk_add(*p, bytes);
  return VSK_OK;
}
void dev_free(void* p) {
  if (!p) return;
  chk_remove(p);
  const cudaError_t e = cudaFree(p);
  if (e != cudaSuccess) {
    // nothing to hand the error to (frees happen on clean-up paths): say so once, and do not leave it behind for the
    // next cudaGetLastError of an unrelated call to find
    static bool told = false;
    if (!told) fprintf(stderr, "vsk: cudaFree(%p) failed: %s\n", p, cudaGetErrorString(e));
    told = true;
    cudaGetLastError();
  }
}

int32_t lanes_fork(Ctx* ctx) {
  VSK_CUDA(ctx, cudaEventRecord(ctx->ev_fork, ctx->stream_main));
  VSK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream_aux, ctx->ev_fork, 0));
  return VSK_OK;
}
int32_t lanes_join(Ctx* ctx) {
  VSK_CUDA(ctx, cudaEventRecord(ctx->ev_join, ctx->stream_aux));
  VSK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream_main, ctx->ev_join, 0));
  return VSK_OK;
}

int32_t pinned_reserve(Ctx* ctx, PinnedBuf* b, size_t bytes) {
  if (b->bytes >= bytes) return VSK_OK;
  // the old buffer may still be the target of a copy in flight
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream_main));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream_aux));
  if (b->p) cudaFreeHost(b->p);
  b->p = nullptr;
  b->bytes = 0;
  const size_t want = bytes + bytes / 4 + 4096;
  if (cudaHostAlloc(&b->p, want, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    b->p = nullptr;
    return fail(ctx, VSK_ERR_OUT_OF_MEMORY, "pinned host memory: %zu bytes not available", want);
  }
  b->bytes = want;
  return VSK_OK;
}

int32_t scratch(Ctx* ctx, int slot, size_t bytes, void** out) {
  slot += ctx->lane * 64;   // each lane has its own set of buffers
  if (ctx->scratch_bytes[slot] < bytes) {
    // in-flight work may still use the old buffer
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    dev_free(ctx->scratch[slot]);
    ctx->scratch[slot] = nullptr;
    ctx->scratch_bytes[slot] = 0;
#ifdef VSK_CHECKED
    size_t want = (bytes + 15) & ~(size_t)15;   // no slack: the announced range is the largest request so far
#else
    size_t want = bytes + bytes / 8 + 256;
#endif
    VSK_TRY(dev_alloc(ctx, &ctx->scratch[slot], want));
    ctx->scratch_bytes[slot] = want;
  }
  *out = ctx->scratch[slot];
  return VSK_OK;
}

void tl_mark(Ctx* ctx, const char* name) {
  if (!ctx->timeline) return;
  if (ctx->marks_used == ctx->marks.size()) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
    ctx->marks.push_back(Ctx::Mark{name, ctx->lane, e});
  }
  Ctx::Mark& m = ctx->marks[ctx->marks_used++];
  m.name = name;
  m.lane = ctx->lane;
  cudaEventRecord(m.ev, ctx->stream);
}

void prof_begin(Ctx* ctx) {
  if (!ctx->profile) return;
  if (ctx->prof_used + 2 > ctx->prof_events.size()) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    ctx->prof_events.push_back(a);
    ctx->prof_events.push_back(b);
  }
  cudaEventRecord(ctx->prof_events[ctx->prof_used], ctx->stream);
}
void prof_end(Ctx* ctx) {
  if (!ctx->profile || ctx->prof_used + 2 > ctx->prof_events.size()) return;
  cudaEventRecord(ctx->prof_events[ctx->prof_used + 1], ctx->stream);
  ctx->prof_used += 2;
  ctx->stats.scan_kernel_launches++;
}
void prof_collect(Ctx* ctx) {
  for (size_t i = 0; i + 1 < ctx->prof_used; i += 2) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ctx->prof_events[i], ctx->prof_events[i + 1]) == cudaSuccess)
      ctx->stats.scan_kernel_ms += ms;
  }
  ctx->prof_used = 0;
}

vsk_tuning default_tuning() {
  vsk_tuning t{};
  t.fold_row_term = 1;
  t.chunk_growth = 3;
  t.dense_rows = 0;
  t.ivf_pilot_tiles = 4;
  t.stream_scan = 1;
  t.overlap_min_queries = 0;   // measured: on one GPU the halves take turns at a power-capped device, no gain
  t.stage_kblocks = 2;   // measured: C2 -3 %, int8 shard -7 %, IVF and the 100 k flat case unchanged
  return t;
}

static bool metric_ok(int32_t m) { return m >= VSK_METRIC_EUCLIDEAN && m <= VSK_METRIC_MANHATTAN; }

// Candidate-list workspace for `nq` queries.
static int32_t cand_workspace(Ctx* ctx, int64_t nq, CandLists* c) {
  void* p;
  VSK_TRY(scratch(ctx, SLOT_CAND_KEYS, (size_t)nq * kCandCap * sizeof(uint64_t), &p));
  c->keys = (uint64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_COUNT, (size_t)nq * sizeof(int32_t), &p));
  c->count = (int32_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_THR, (size_t)nq * sizeof(float), &p));
  c->thr = (float*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_FLAGS, (size_t)nq * sizeof(int32_t), &p));
  c->flags = (int32_t*)p;
  c->nq = nq;
  return VSK_OK;
}

// scan(mode, row_begin, row_end): appends to the lists.

// Rows per chunk after `seen` rows, for lists compacted to `keep` keys.  A chunk of g * seen rows appends
// about keep * g keys to a list, with a relative spread of 1/sqrt(keep) (the threshold is the keep-th order
// statistic of the rows seen); g is chosen so that the mean plus six such deviations still fits the free
// room of a list.  level 1 divides g by 8 (for the rare query whose list overflowed all the same), level 2
// uses chunks no larger than the free room, which cannot overflow whatever the row order.
int64_t schedule_chunk(int64_t seen, int32_t keep, int level) {
  const int64_t room = kCandCap - keep;
  if (level >= 2) return room;
  double g = (double)room / ((double)keep * (1.0 + 6.0 / sqrt((double)keep)));
  if (level == 1) g /= 8.0;
  return std::max<int64_t>(room, (int64_t)(g * (double)seen));
}

int64_t schedule_dense_rows(const Ctx* ctx, int32_t keep) {
  if (ctx->tuning.dense_rows > 0) return std::min<int64_t>(kCandCap, ctx->tuning.dense_rows);
  return std::min<int64_t>(kCandCap, std::max<int64_t>(1024, ceil_div(8 * (int64_t)keep, 256) * 256));
}

int32_t schedule_max_count(int64_t seen, int64_t chunk, int32_t keep) {
  const double mean = (double)keep * (double)chunk / (double)std::max<int64_t>(seen, 1);
  const double bound = (double)keep + mean * (1.0 + 8.0 / sqrt((double)keep)) + 8.0;
  return (int32_t)std::min<double>(bound, 1e9);
}

// Walks rows [0, n) in chunks.  The first chunk (schedule_dense_rows) is written densely, one slot per
// row; it is compacted to the best `keep`, whose worst value becomes the threshold.  Each later chunk appends
// only rows at or below the threshold (see schedule_chunk for its size).  A list that overflows is flagged
// and its query is re-run at the next level.
static int32_t run_schedule(Ctx* ctx, const ScanFn& scan, int64_t n, int64_t nq, int32_t keep,
                            const CandLists& cand, int level) {
  // a list must have room beyond the keys it keeps, or the walk below would never advance
  if (keep <= 0 || keep > kCandCap / 2)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "a search keeps between 1 and %d rows per query (asked for %d)", kCandCap / 2, keep);
  VSK_TRY(launch_init_cand(ctx, cand, nq));
  SelectArgs sel{};
  sel.cand = cand;
  sel.nq = nq;
  sel.keep = keep;
  int64_t seen = std::min<int64_t>(n, schedule_dense_rows(ctx, keep));
  VSK_TRY(scan(SCAN_DENSE, 0, seen));
  sel.dense_count = (int32_t)seen;
  sel.max_count = (int32_t)seen;
  VSK_TRY(launch_select(ctx, sel));
  sel.dense_count = -1;
  while (seen < n) {
    const int64_t chunk = std::min(schedule_chunk(seen, keep, level), n - seen);
    if (chunk <= 0) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "search schedule: empty chunk after %lld rows", (long long)seen);
    VSK_TRY(scan(SCAN_THRESHOLD, seen, seen + chunk));
    sel.max_count = level >= 2 ? kCandCap : schedule_max_count(seen, chunk, keep);
    VSK_TRY(launch_select(ctx, sel));
    seen += chunk;
  }
  return VSK_OK;
}

// Indices of flagged queries, gathered on the host (a few bytes per query, once per batch).
static int32_t flagged_queries(Ctx* ctx, const CandLists& cand, int64_t nq, std::vector<int32_t>* out) {
  std::vector<int32_t> flags((size_t)nq);
  VSK_CUDA(ctx, cudaMemcpyAsync(flags.data(), cand.flags, nq * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  out->clear();
  for (int64_t i = 0; i < nq; ++i)
    if (flags[i]) out->push_back((int32_t)i);
  return VSK_OK;
}

// fp32 scan of `nq` queries (optionally the subset `sub_dev` of a larger batch) over n rows
// described by `proto` (metric, operands, norms, masks), with final output.
static int pick_query_tile(int64_t g);

// Exact top-k of nq queries (optionally the subset `sub_dev` of a larger batch) over n rows with any scan that
// follows the candidate-list protocol: `make_scan` binds the lists (and the subset) to a scan function; queries
// whose list overflowed are re-run at the next level of the schedule.
int32_t scan_topk(Ctx* ctx, const ScanBinder& make_scan, int64_t n, int64_t nq, const int32_t* sub_dev, int32_t k,
                  int64_t id_base, int final_sqrt, float* out_dist, int64_t* out_ids, int level, const int32_t* id_remap) {
  CandLists cand;
  VSK_TRY(cand_workspace(ctx, nq, &cand));
  const ScanFn scan = make_scan(cand, nq, sub_dev);
  VSK_TRY(run_schedule(ctx, scan, n, nq, k, cand, level));
  SelectArgs fin{};
  fin.cand = cand;
  fin.nq = nq;
  fin.dense_count = -1;
  fin.keep = k;
  fin.out_dist = out_dist;
  fin.out_ids = out_ids;
  fin.k = k;
  fin.id_base = id_base;
  fin.q_subset = sub_dev;
  fin.final_sqrt = final_sqrt;
  fin.max_count = k;
  fin.id_remap = id_remap;
  VSK_TRY(launch_select(ctx, fin));
  if (level < 2) {
    std::vector<int32_t> bad;
    VSK_TRY(flagged_queries(ctx, cand, nq, &bad));
    if (!bad.empty()) {
      // map list positions back to query indices of the caller's batch
      if (sub_dev) {
        std::vector<int32_t> sub_h((size_t)nq);
        VSK_CUDA(ctx, cudaMemcpy(sub_h.data(), sub_dev, nq * sizeof(int32_t), cudaMemcpyDeviceToHost));
        for (auto& b : bad) b = sub_h[b];
      }
      void* p;
      VSK_TRY(scratch(ctx, level == 0 ? SLOT_MISC0 : SLOT_MISC1, bad.size() * sizeof(int32_t), &p));
      VSK_CUDA(ctx, cudaMemcpyAsync(p, bad.data(), bad.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
      VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      ctx->stats.fallback_queries += (int64_t)bad.size();
      VSK_TRY(scan_topk(ctx, make_scan, n, (int64_t)bad.size(), (const int32_t*)p, k, id_base, final_sqrt, out_dist,
                        out_ids, level + 1, id_remap));
    }
  }
  return VSK_OK;
}

int32_t fp32_topk(Ctx* ctx, const ExactScanArgs& proto, int64_t n, int64_t nq, const int32_t* sub_dev, int32_t k,
                  int64_t id_base, float* out_dist, int64_t* out_ids, int level) {
  const ScanBinder bind = [ctx, &proto](const CandLists& cand, int64_t bn, const int32_t* sub) -> ScanFn {
    ExactScanArgs a = proto;
    a.nq = bn;
    // a small batch (a few queries, or the handful of queries a fallback re-runs): narrow query tiles
    if (a.bm_hint == 0 && bn < 128) {
      const int bm = pick_query_tile(bn);
      if (bm < 128) a.bm_hint = bm;
    }
    a.q_subset = sub;
    a.cand = cand;
    return [ctx, a](int mode, int64_t b, int64_t e) mutable {
      a.mode = mode;
      a.row_begin = b;
      a.row_end = e;
      return launch_exact_scan(ctx, a);
    };
  };
  return scan_topk(ctx, bind, n, nq, sub_dev, k, id_base, proto.metric == VSK_METRIC_EUCLIDEAN, out_dist, out_ids, level,
                   proto.final_id_remap);
}

static int32_t fp32_search(Index* ix, const float* q, int64_t nq, const int32_t* sub_dev, int32_t k,
                           const float* qnorm, const uint64_t* qmasks, float* out_dist, int64_t* out_ids,
                           int level) {
  ExactScanArgs a{};
  a.metric = ix->metric;
  a.q = q;
  a.x = ix->rows;
  if (ix->kind == INDEX_FLAT_I8) {
    a.x = nullptr;
    a.x_codes = ix->codes;
    a.sq_scale = ix->sq_scale;
    a.sq_offset = ix->sq_offset;
  }
  a.dim = ix->dim;
  a.qnorm = qnorm;
  a.xnorm = ix->row_norm;
  a.row_masks = (qmasks && ix->has_masks) ? ix->masks : nullptr;
  a.q_masks = a.row_masks ? qmasks : nullptr;
  return fp32_topk(ix->ctx, a, ix->n, nq, sub_dev, k, ix->id_base, out_dist, out_ids, level);
}

// ---- filtered search, grouped by mask ---------------------------------------------------------
// Queries that carry the same filter mask share one set of eligible rows.  When a batch has few distinct
// masks, each group of queries is scanned only against its eligible rows (a list of row numbers made by one
// compaction pass over the 8-byte row masks), instead of computing every (query, row) value and discarding the
// ineligible ones afterwards: the FP32 work drops by the share of rows the filter rejects.
__global__ void mask_compact_kernel(const uint64_t* __restrict__ masks, int64_t n, uint64_t qmask,
                                    int32_t* __restrict__ rows, int32_t* counter) {
  __shared__ int warp_base[8];
  __shared__ int block_base;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool pass = i < n && (masks[i] & qmask) != 0;
  const unsigned bal = __ballot_sync(0xffffffffu, pass);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_base[warp] = __popc(bal);
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < 8; ++w) { const int c = warp_base[w]; warp_base[w] = tot; tot += c; }
    block_base = tot ? atomicAdd(counter, tot) : 0;
  }
  __syncthreads();
  if (pass) rows[block_base + warp_base[warp] + __popc(bal & ((1u << lane) - 1u))] = (int32_t)i;
}

// counts[g] = rows eligible under group mask g (at most 64 groups; one pass over the row masks)
__global__ void mask_count_kernel(const uint64_t* __restrict__ masks, int64_t n, const uint64_t* __restrict__ gmasks,
                                  int groups, unsigned long long* __restrict__ counts) {
  __shared__ uint64_t gm[64];
  __shared__ unsigned int local[64];
  if (threadIdx.x < 64) {
    gm[threadIdx.x] = threadIdx.x < groups ? gmasks[threadIdx.x] : 0ull;
    local[threadIdx.x] = 0u;
  }
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t m = masks[i];
    for (int g = 0; g < groups; ++g)
      if ((m & gm[g]) != 0ull) atomicAdd(&local[g], 1u);
  }
  __syncthreads();
  if (threadIdx.x < groups && local[threadIdx.x]) atomicAdd(&counts[threadIdx.x], (unsigned long long)local[threadIdx.x]);
}

__global__ void fill_empty_results_kernel(const int32_t* __restrict__ qpos, int64_t m, int k, float* out_dist,
                                          int64_t* out_ids) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m * k) return;
  const int64_t q = qpos[i / k];
  out_dist[q * k + i % k] = INFINITY;
  out_ids[q * k + i % k] = -1;
}

static int pick_query_tile(int64_t g) {
  auto pad = [&](int bm) { return ceil_div(g, bm) * bm; };
  const double best = (double)pad(32);
  if ((double)pad(128) <= 1.1 * best) return 128;
  if ((double)pad(64) <= 1.1 * best) return 64;
  return 32;
}

// Returns *handled = false (and does nothing) when the batch has too many distinct masks to profit.
// max_fraction >= 0: the caller has a faster scan for the unfiltered pairs (the tensor path, about thirty times the
// fp32 tile's rate) and this path is taken only when the filters leave less than that share of the (query, row)
// pairs eligible - then scanning only eligible rows wins all the same.
static int32_t filtered_grouped_search(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm,
                                       const uint64_t* qmasks, float* out_dist, int64_t* out_ids, bool* handled,
                                       double max_fraction = -1.0) {
  Ctx* ctx = ix->ctx;
  *handled = false;
  std::vector<uint64_t> hm((size_t)nq);
  VSK_CUDA(ctx, cudaMemcpyAsync(hm.data(), qmasks, (size_t)nq * 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::vector<int32_t> perm((size_t)nq);
  for (int64_t i = 0; i < nq; ++i) perm[(size_t)i] = (int32_t)i;
  std::stable_sort(perm.begin(), perm.end(), [&](int32_t a, int32_t b) { return hm[(size_t)a] < hm[(size_t)b]; });
  std::vector<int64_t> starts;
  for (int64_t i = 0; i < nq; ++i)
    if (i == 0 || hm[(size_t)perm[(size_t)i]] != hm[(size_t)perm[(size_t)i - 1]]) starts.push_back(i);
  starts.push_back(nq);
  const int64_t groups = (int64_t)starts.size() - 1;
  // Worth it?  Cost is proportional to (padded queries) x (rows scanned).  Grouped: each group's queries padded
  // to its query tile, over its eligible rows (assumed to be at most 60 % of the rows); ungrouped: all queries
  // padded to 128, over all rows.
  int64_t padded = 0;
  for (int64_t g = 0; g < groups; ++g) {
    const int64_t sz = starts[(size_t)g + 1] - starts[(size_t)g];
    padded += ceil_div(sz, pick_query_tile(sz)) * pick_query_tile(sz);
  }
  if (groups > 256 || (double)padded * 0.6 > (double)(ceil_div(nq, 128) * 128)) return VSK_OK;
  // A batch small enough for the streaming scan is bound by the bytes it reads: one pass over all rows (rows that
  // no query may see are skipped there too) beats one pass over the eligible rows per group, unless there is
  // only one group.
  if (nq <= kStreamScanMaxQueries && groups > 1) return VSK_OK;
  void *dperm, *drows, *dcount;
  if (max_fraction >= 0.0) {
    if (groups > 64) return VSK_OK;
    std::vector<uint64_t> gm((size_t)groups);
    for (int64_t g = 0; g < groups; ++g) gm[(size_t)g] = hm[(size_t)perm[(size_t)starts[(size_t)g]]];
    VSK_TRY(scratch(ctx, SLOT_FILTER_COUNT, 64 * 16, &dcount));
    unsigned long long* dcnt = (unsigned long long*)dcount;
    uint64_t* dgm = (uint64_t*)dcount + 64;
    VSK_CUDA(ctx, cudaMemsetAsync(dcnt, 0, 64 * 8, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(dgm, gm.data(), (size_t)groups * 8, cudaMemcpyHostToDevice, ctx->stream));
    mask_count_kernel<<<(unsigned)std::min<int64_t>(ceil_div(ix->n, 256), 1184), 256, 0, ctx->stream>>>(ix->masks, ix->n, dgm, (int)groups, dcnt);
    ctx->stats.kernel_launches++;
    std::vector<unsigned long long> cnt((size_t)groups);
    VSK_CUDA(ctx, cudaMemcpyAsync(cnt.data(), dcnt, (size_t)groups * 8, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double pairs = 0.0;
    for (int64_t g = 0; g < groups; ++g) pairs += (double)(starts[(size_t)g + 1] - starts[(size_t)g]) * (double)cnt[(size_t)g];
    if (pairs >= max_fraction * (double)nq * (double)ix->n) return VSK_OK;
  }
  *handled = true;
  VSK_TRY(scratch(ctx, SLOT_FILTER_PERM, (size_t)nq * 4, &dperm));
  VSK_TRY(scratch(ctx, SLOT_FILTER_ROWS, (size_t)ix->n * 4, &drows));
  VSK_TRY(scratch(ctx, SLOT_FILTER_COUNT, 16, &dcount));
  VSK_CUDA(ctx, cudaMemcpyAsync(dperm, perm.data(), (size_t)nq * 4, cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // perm is a local
  for (int64_t g = 0; g < groups; ++g) {
    const int64_t b = starts[(size_t)g], e = starts[(size_t)g + 1];
    const uint64_t m = hm[(size_t)perm[(size_t)b]];
    const int32_t* qpos = (const int32_t*)dperm + b;
    VSK_CUDA(ctx, cudaMemsetAsync(dcount, 0, 4, ctx->stream));
    mask_compact_kernel<<<(unsigned)ceil_div(ix->n, 256), 256, 0, ctx->stream>>>(ix->masks, ix->n, m, (int32_t*)drows, (int32_t*)dcount);
    ctx->stats.kernel_launches++;
    int32_t cnt = 0;
    VSK_CUDA(ctx, cudaMemcpyAsync(&cnt, dcount, 4, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (cnt == 0) {
      fill_empty_results_kernel<<<(unsigned)ceil_div((e - b) * k, 256), 256, 0, ctx->stream>>>(qpos, e - b, k, out_dist, out_ids);
      ctx->stats.kernel_launches++;
      continue;
    }
    ExactScanArgs a{};
    a.metric = ix->metric;
    a.q = q;
    a.x = ix->rows;
    a.x_rows = (const int32_t*)drows;
    a.bm_hint = pick_query_tile(e - b);
    a.dim = ix->dim;
    a.qnorm = qnorm;
    a.xnorm = ix->row_norm;
    VSK_TRY(fp32_topk(ctx, a, cnt, e - b, qpos, k, ix->id_base, out_dist, out_ids, 0));
  }
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

constexpr int64_t kQueryBatch = 16384;  // queries per pass: bounds the candidate workspace at 512 MB

static int32_t flat_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks,
                               float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_FLAT_F32) return fail(ctx, VSK_ERR_INVALID_INPUT, "not a flat fp32 index");
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  if (qmasks && !ix->has_masks) return fail(ctx, VSK_ERR_INVALID_INPUT, "query masks given but the index has no row masks");
  ctx->stats.searches++;
  ctx->stats.queries += nq;
  for (int64_t b = 0; b < nq; b += kQueryBatch) {
    const int64_t bn = std::min(kQueryBatch, nq - b);
    const float* qb = q + b * ix->dim;
    const uint64_t* mb = qmasks ? qmasks + b : nullptr;
    float* qnorm = nullptr;
    if (ix->metric == VSK_METRIC_COSINE) {
      void* p;
      VSK_TRY(scratch(ctx, SLOT_QNORM, bn * sizeof(float), &p));
      qnorm = (float*)p;
      VSK_TRY(launch_row_norms(ctx, qb, bn, ix->dim, 0, qnorm));
    }
    // Euclidean, cosine and dot-product batches take the tensor path, filtered or not (the filter is applied to the
    // hits in the contraction's epilogue).  A batch of a few queries is bound by the bytes it reads, not by the
    // contraction: the fp32 streaming scan reads each eligible fp32 row once.
    const bool tensor = ctx->search_path == VSK_PATH_TENSOR_RERANK && ix->metric != VSK_METRIC_MANHATTAN &&
                        !(mb && bn <= kStreamScanMaxQueries);
    bool grouped = false;
    if (mb && ix->has_masks)
      VSK_TRY(filtered_grouped_search(ix, qb, bn, k, qnorm, mb, out_dist + b * k, out_ids + b * k, &grouped,
                                      tensor ? 0.03 : -1.0));
    if (grouped) {
      // done: every group of equal masks was scanned against its own eligible rows
    } else if (tensor) {
      VSK_TRY(tensor_search(ix, qb, bn, k, qnorm, mb, out_dist + b * k, out_ids + b * k));
    } else {
      VSK_TRY(fp32_search(ix, qb, bn, nullptr, k, qnorm, mb, out_dist + b * k, out_ids + b * k, 0));
    }
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

// Entry used by the tensor path for queries whose certificate failed.
int32_t fp32_search_subset(Index* ix, const float* q, const std::vector<int32_t>& subset, int32_t k,
                           const float* qnorm, const uint64_t* qmasks, float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  if (subset.empty()) return VSK_OK;
  void* p;
  VSK_TRY(scratch(ctx, SLOT_SUBSET, subset.size() * sizeof(int32_t), &p));
  VSK_CUDA(ctx, cudaMemcpyAsync(p, subset.data(), subset.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.fallback_queries += (int64_t)subset.size();
  return fp32_search(ix, q, (int64_t)subset.size(), (const int32_t*)p, k, qnorm, qmasks, out_dist, out_ids, 0);
}

int32_t flat_reserve(Index* ix, int64_t need) {
  Ctx* ctx = ix->ctx;
  if (need <= ix->capacity) return VSK_OK;
  int64_t cap = std::max<int64_t>(need, ix->capacity + ix->capacity / 2);
  float* rows = nullptr;
  float* norm = nullptr;
  uint64_t* masks = nullptr;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&rows, (size_t)cap * ix->dim * sizeof(float))) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&norm, (size_t)cap * sizeof(float))) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&masks, (size_t)cap * sizeof(uint64_t))) != VSK_OK) {
    dev_free(rows);   // out of memory part-way: the index keeps what it had
    dev_free(norm);
    dev_free(masks);
    return st;
  }
  if (ix->n > 0) {
    VSK_CUDA(ctx, cudaMemcpyAsync(rows, ix->rows, (size_t)ix->n * ix->dim * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(norm, ix->row_norm, (size_t)ix->n * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    if (ix->has_masks)
      VSK_CUDA(ctx, cudaMemcpyAsync(masks, ix->masks, (size_t)ix->n * sizeof(uint64_t), cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  dev_free(ix->rows);
  dev_free(ix->row_norm);
  dev_free(ix->masks);
  ix->rows = rows;
  ix->row_norm = norm;
  ix->masks = masks;
  ix->capacity = cap;
  return VSK_OK;
}

// Rows (and masks) were written straight into the reserved storage (an index image being loaded): compute what
// an add computes and count them in.
int32_t flat_adopt_rows(Index* ix, int64_t n, bool has_masks) {
  Ctx* ctx = ix->ctx;
  if (n > ix->capacity) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "more rows than reserved");
  ix->has_masks = has_masks;
  if (ix->metric == VSK_METRIC_COSINE || ix->metric == VSK_METRIC_EUCLIDEAN)
    VSK_TRY(launch_row_norms(ctx, ix->rows, n, ix->dim, ix->metric == VSK_METRIC_EUCLIDEAN, ix->row_norm));
  ix->n = n;
  tensor_invalidate(ix);
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

static int32_t flat_add(Index* ix, const float* rows, int64_t n, const uint64_t* masks, bool on_device) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_FLAT_F32) return fail(ctx, VSK_ERR_INVALID_INPUT, "not a flat fp32 index");
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows to add");
  if (!rows) return fail(ctx, VSK_ERR_INVALID_INPUT, "null rows");
  if (ix->n + n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "a flat index holds at most 2^31-1 rows");
  if (ix->n > 0 && ((masks != nullptr) != ix->has_masks))
    return fail(ctx, VSK_ERR_INVALID_INPUT, "either every added block carries masks or none does");
  VSK_TRY(flat_reserve(ix, ix->n + n));
  if (masks) ix->has_masks = true;
  const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  VSK_CUDA(ctx, cudaMemcpyAsync(ix->rows + ix->n * ix->dim, rows, (size_t)n * ix->dim * sizeof(float), kind, ctx->stream));
  if (masks)
    VSK_CUDA(ctx, cudaMemcpyAsync(ix->masks + ix->n, masks, (size_t)n * sizeof(uint64_t), kind, ctx->stream));
  if (!on_device) ctx->stats.h2d_bytes += (int64_t)n * ix->dim * 4 + (masks ? n * 8 : 0);
  if (ix->metric == VSK_METRIC_COSINE || ix->metric == VSK_METRIC_EUCLIDEAN)
    VSK_TRY(launch_row_norms(ctx, ix->rows + ix->n * ix->dim, n, ix->dim, ix->metric == VSK_METRIC_EUCLIDEAN,
                             ix->row_norm + ix->n));
  ix->n += n;
  tensor_invalidate(ix);
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

const char* vsk_status_string(int32_t s) {
  switch (s) {
    case VSK_OK: return "ok";
    case VSK_ERR_DEVICE_NOT_AVAILABLE: return "device not available";
    case VSK_ERR_OUT_OF_MEMORY: return "device out of memory";
    case VSK_ERR_UNSUPPORTED_OPERATION: return "unsupported operation";
    case VSK_ERR_INVALID_BUFFER_SIZE: return "invalid buffer size";
    case VSK_ERR_EXECUTION_FAILED: return "execution failed";
    case VSK_ERR_TIMEOUT: return "timeout";
    case VSK_ERR_INVALID_INPUT: return "invalid input";
    case VSK_ERR_DIMENSION_MISMATCH: return "dimension mismatch";
    case VSK_ERR_EMPTY_INPUT: return "empty input";
    case VSK_ERR_NOT_TRAINED: return "index not trained";
    case VSK_ERR_INSUFFICIENT_TRAINING_DATA: return "insufficient training data";
    case VSK_ERR_IMPORT_FAILED: return "index image could not be imported";
    case VSK_ERR_EXPORT_FAILED: return "index image could not be exported";
    default: return "unknown status";
  }
}

int32_t vsk_open(int32_t device, vsk_ctx** out_ctx) {
  if (!out_ctx) return VSK_ERR_INVALID_INPUT;
  *out_ctx = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0 || device < 0 || device >= count) {
    cudaGetLastError();
    return VSK_ERR_DEVICE_NOT_AVAILABLE;
  }
  Ctx* ctx = new Ctx();
  ctx->device = device;
  if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&ctx->prop, device) != cudaSuccess) {
    delete ctx;
    return VSK_ERR_DEVICE_NOT_AVAILABLE;
  }
  if (ctx->prop.major != 10) {
    // the kernels are built for sm_100a only
    delete ctx;
    return VSK_ERR_DEVICE_NOT_AVAILABLE;
  }
  if (cudaStreamCreateWithFlags(&ctx->stream_main, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->stream_aux, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ctx->ev_join, cudaEventDisableTiming) != cudaSuccess) {
    if (ctx->stream_main) cudaStreamDestroy(ctx->stream_main);
    if (ctx->stream_aux) cudaStreamDestroy(ctx->stream_aux);
    if (ctx->ev_fork) cudaEventDestroy(ctx->ev_fork);
    cudaGetLastError();
    delete ctx;
    return VSK_ERR_DEVICE_NOT_AVAILABLE;
  }
  ctx->stream = ctx->stream_main;
  ctx->tuning = default_tuning();
  if (chk_open(ctx) != VSK_OK) {   // checked build: the range table of this GPU
    cudaStreamDestroy(ctx->stream_main);
    cudaStreamDestroy(ctx->stream_aux);
    cudaEventDestroy(ctx->ev_fork);
    cudaEventDestroy(ctx->ev_join);
    cudaGetLastError();
    delete ctx;
    return VSK_ERR_DEVICE_NOT_AVAILABLE;
  }
  *out_ctx = reinterpret_cast<vsk_ctx*>(ctx);
  return VSK_OK;
}

int32_t vsk_close(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  worker_release(ctx);   // runs what is still queued, then joins
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream_main);
  cudaStreamSynchronize(ctx->stream_aux);
  comm_release(ctx);
  for (auto& p : ctx->scratch) dev_free(p);
  for (auto& b : ctx->host_flags)
    if (b.p) cudaFreeHost(b.p);
  for (auto& e : ctx->prof_events) cudaEventDestroy(e);
  for (auto& m : ctx->marks) cudaEventDestroy(m.ev);
  if (ctx->tl_origin) cudaEventDestroy(ctx->tl_origin);
  cudaEventDestroy(ctx->ev_fork);
  cudaEventDestroy(ctx->ev_join);
  cudaStreamDestroy(ctx->stream_main);
  cudaStreamDestroy(ctx->stream_aux);
  delete ctx;
  return VSK_OK;
}

int32_t vsk_device_info_get(vsk_ctx* c, vsk_device_info* out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  memset(out, 0, sizeof(*out));
  out->device = ctx->device;
  out->sm_count = ctx->prop.multiProcessorCount;
  out->cc_major = ctx->prop.major;
  out->cc_minor = ctx->prop.minor;
  out->hbm_bytes = (int64_t)ctx->prop.totalGlobalMem;
  out->l2_bytes = ctx->prop.l2CacheSize;
  out->max_smem_per_block = (int32_t)ctx->prop.sharedMemPerBlockOptin;
  strncpy(out->name, ctx->prop.name, sizeof(out->name) - 1);
  return VSK_OK;
}

int32_t vsk_stats_get(vsk_ctx* c, vsk_stats* out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  if (ctx->profile) {
    cudaStreamSynchronize(ctx->stream);
    prof_collect(ctx);
  }
  *out = ctx->stats;
  return VSK_OK;
}

const char* vsk_last_error(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  return ctx ? ctx->err.c_str() : "null context";
}

int32_t vsk_set_search_path(vsk_ctx* c, int32_t path) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  if (path != VSK_PATH_TENSOR_RERANK && path != VSK_PATH_FP32_SCAN)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "unknown search path %d", path);
  ctx->search_path = path;
  return VSK_OK;
}

int64_t vsk_schedule_chunk(int64_t seen, int32_t keep, int32_t level) {
  if (seen < 0 || keep <= 0 || keep > kCandCap / 2) return -1;
  return schedule_chunk(seen, keep, level);
}

int32_t vsk_timeline(vsk_ctx* c, int32_t enable) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream_main);
  cudaStreamSynchronize(ctx->stream_aux);
  ctx->marks_used = 0;
  ctx->timeline = enable != 0;
  if (ctx->timeline) {
    if (!ctx->tl_origin && cudaEventCreate(&ctx->tl_origin) != cudaSuccess) {
      cudaGetLastError();
      ctx->timeline = false;
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "could not create the origin event");
    }
    cudaEventRecord(ctx->tl_origin, ctx->stream_main);
  }
  return VSK_OK;
}

int64_t vsk_timeline_read(vsk_ctx* c, char* text, int64_t capacity) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !text || capacity <= 0) return -1;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream_main);
  cudaStreamSynchronize(ctx->stream_aux);
  int64_t used = 0;
  text[0] = 0;
  for (size_t i = 0; i < ctx->marks_used; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ctx->tl_origin, ctx->marks[i].ev) != cudaSuccess) { cudaGetLastError(); continue; }
    const int w = snprintf(text + used, (size_t)(capacity - used), "%d %s %.4f\n", ctx->marks[i].lane, ctx->marks[i].name, ms);
    if (w < 0 || used + w >= capacity) break;
    used += w;
  }
  ctx->marks_used = 0;
  if (ctx->timeline) cudaEventRecord(ctx->tl_origin, ctx->stream_main);
  return used;
}

int32_t vsk_profile(vsk_ctx* c, int32_t enable) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaStreamSynchronize(ctx->stream);
  prof_collect(ctx);
  ctx->profile = enable != 0;
  return VSK_OK;
}

void* vsk_stream(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  return ctx ? (void*)ctx->stream_main : nullptr;
}

int32_t vsk_tuning_get(vsk_ctx* c, vsk_tuning* out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  *out = ctx->tuning;
  return VSK_OK;
}

int32_t vsk_tuning_set(vsk_ctx* c, const vsk_tuning* in) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !in) return VSK_ERR_INVALID_INPUT;
  if (in->chunk_growth < 1 || in->ivf_pilot_tiles < 1 || in->ivf_pilot_tiles > 16 || in->dense_rows < 0 ||
      in->dense_rows > kCandCap || in->overlap_min_queries < 0 || in->wait_limit_log2 < 0 || in->wait_limit_log2 > 30 ||
      in->assign_stages < 0 || in->assign_stages > 8 || in->stage_kblocks < 0 || in->stage_kblocks > 2)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "tuning value out of range");
  ctx->tuning = *in;
  return VSK_OK;
}

int32_t vsk_batch_distances_dev(vsk_ctx* c, int32_t metric, const float* q, int64_t nq, const float* x,
                                int64_t nx, int32_t dim, float* out) {
  VSK_TRACE("vsk_batch_distances_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (!metric_ok(metric)) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", metric);
  if (nq <= 0 || nx <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or candidates");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!q || !x || !out) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  ExactScanArgs a{};
  a.metric = metric;
  a.mode = SCAN_MATRIX;
  a.q = q;
  a.x = x;
  a.dim = dim;
  a.nq = nq;
  a.row_begin = 0;
  a.row_end = nx;
  a.out = out;
  a.ld_out = nx;
  if (metric == VSK_METRIC_COSINE) {
    void* p;
    VSK_TRY(scratch(ctx, SLOT_QNORM, nq * sizeof(float), &p));
    VSK_TRY(launch_row_norms(ctx, q, nq, dim, 0, (float*)p));
    a.qnorm = (float*)p;
    VSK_TRY(scratch(ctx, SLOT_X_TMP, nx * sizeof(float), &p));
    VSK_TRY(launch_row_norms(ctx, x, nx, dim, 0, (float*)p));
    a.xnorm = (float*)p;
  }
  VSK_TRY(launch_exact_scan(ctx, a));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_batch_distances(vsk_ctx* c, int32_t metric, const float* q, int64_t nq, const float* x, int64_t nx,
                            int32_t dim, float* out) {
  VSK_TRACE("vsk_batch_distances");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (!metric_ok(metric)) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", metric);
  if (nq <= 0 || nx <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or candidates");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!q || !x || !out) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  float *dq = nullptr, *dx = nullptr, *dout = nullptr;
  int32_t st = VSK_OK;
  if ((st = dev_alloc(ctx, (void**)&dq, (size_t)nq * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dx, (size_t)nx * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dout, (size_t)nq * nx * 4)) == VSK_OK) {
    cudaMemcpyAsync(dq, q, (size_t)nq * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    cudaMemcpyAsync(dx, x, (size_t)nx * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    st = vsk_batch_distances_dev(c, metric, dq, nq, dx, nx, dim, dout);
    if (st == VSK_OK) {
      cudaError_t e = cudaMemcpy(out, dout, (size_t)nq * nx * 4, cudaMemcpyDeviceToHost);
      if (e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "copy out failed: %s", cudaGetErrorString(e));
    }
    ctx->stats.h2d_bytes += (nq + nx) * dim * 4;
    ctx->stats.d2h_bytes += nq * nx * 4;
  }
  dev_free(dq);
  dev_free(dx);
  dev_free(dout);
  return st;
}

int32_t vsk_flat_create(vsk_ctx* c, int32_t metric, int32_t dim, vsk_index** out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  *out = nullptr;
  if (!metric_ok(metric)) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", metric);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  Index* ix = new Index();
  ix->ctx = ctx;
  ix->kind = INDEX_FLAT_F32;
  ix->metric = metric;
  ix->dim = dim;
  *out = reinterpret_cast<vsk_index*>(ix);
  return VSK_OK;
}

int32_t vsk_flat_add_f32(vsk_index* i, const float* rows, int64_t n, const uint64_t* masks) {
  VSK_TRACE("vsk_flat_add_f32");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  drain_stale_error("vsk_flat_add");
  return flat_add(ix, rows, n, masks, false);
}

int32_t vsk_flat_add_f32_dev(vsk_index* i, const float* rows, int64_t n, const uint64_t* masks) {
  VSK_TRACE("vsk_flat_add_f32_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  drain_stale_error("vsk_flat_add");
  return flat_add(ix, rows, n, masks, true);
}

int32_t vsk_index_destroy(vsk_index* i) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  cudaStreamSynchronize(ix->ctx->stream);
  dev_free(ix->rows);
  dev_free(ix->row_norm);
  dev_free(ix->masks);
  dev_free(ix->rows16);
  dev_free(ix->row_aux);
  dev_free(ix->codes);
  dev_free(ix->sq_scale);
  dev_free(ix->sq_offset);
  dev_free(ix->centroids);
  dev_free(ix->list_offsets);
  dev_free(ix->list_rows);
  dev_free(ix->assign);
  dev_free(ix->pq_codebooks);
  dev_free(ix->pq_codes);
  if (ix->coarse) {   // shares the centroids: only its derived buffers are its own
    dev_free(ix->coarse->row_norm);
    dev_free(ix->coarse->rows16);
    dev_free(ix->coarse->row_aux);
    delete ix->coarse;
  }
  delete ix;
  return VSK_OK;
}

int64_t vsk_index_size(vsk_index* i) {
  Index* ix = reinterpret_cast<Index*>(i);
  return ix ? ix->n : -1;
}

int32_t vsk_index_set_id_base(vsk_index* i, int64_t id_base) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  ix->id_base = id_base;
  return VSK_OK;
}

int32_t vsk_search_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks,
                       float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_search_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  drain_stale_error("vsk_search_dev");
  if (ix->kind == INDEX_FLAT_I8) return sq8_search_dev(ix, q, nq, k, out_dist, out_ids);
  if (ix->kind == INDEX_PQ) {
    if (qmasks) return fail(ix->ctx, VSK_ERR_UNSUPPORTED_OPERATION, "a product-quantised index carries no row masks");
    return pq_search_dev(ix, q, nq, k, out_dist, out_ids);
  }
  return flat_search_dev(ix, q, nq, k, qmasks, out_dist, out_ids);
}

}  // extern "C"

namespace vsk {
// vsk_search_dev for callers inside the library (the device is already selected)
int32_t flat_search_dev_entry(Index* ix, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, float* out_dist,
                              int64_t* out_ids) {
  if (ix->kind == INDEX_FLAT_I8) return sq8_search_dev(ix, q, nq, k, out_dist, out_ids);
  return flat_search_dev(ix, q, nq, k, qmasks, out_dist, out_ids);
}
}  // namespace vsk

extern "C" {

int32_t vsk_coarse_values_dev(vsk_index* i, const float* q, int64_t nq, int64_t rows, float* coarse, float* eps) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (ix->kind != INDEX_FLAT_F32) return fail(ctx, VSK_ERR_INVALID_INPUT, "not a flat fp32 index");
  if (ix->metric == VSK_METRIC_MANHATTAN) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "manhattan has no tensor path");
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (nq > kQueryBatch) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "at most %lld queries per call", (long long)kQueryBatch);
  if (!q || !coarse) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  return tensor_coarse_values(ix, q, nq, rows, coarse, eps);
}

__global__ void fill_inf_kernel(float* p, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = CUDART_INF_F;
}

int32_t vsk_search_shard_begin_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t shards, float* bound) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  ctx->pending[ctx->lane] = ShardPending{};
  if (ix->kind != INDEX_FLAT_F32) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "the two-half search covers flat fp32 indexes");
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (nq > kQueryBatch) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "at most %lld queries per two-half search", (long long)kQueryBatch);
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (shards <= 0) return fail(ctx, VSK_ERR_INVALID_INPUT, "shards must be positive");
  if (!q || !bound) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  const bool tensor = ctx->search_path == VSK_PATH_TENSOR_RERANK && ix->metric != VSK_METRIC_MANHATTAN;
  if (!tensor) {
    // no split form: nothing is known yet, the second half runs the whole search
    fill_inf_kernel<<<(unsigned)ceil_div(nq, 256), 256, 0, ctx->stream>>>(bound, nq);
    ctx->stats.kernel_launches++;
    VSK_CUDA(ctx, cudaGetLastError());
    ctx->pending[ctx->lane].active = true;
    ctx->pending[ctx->lane].ix = ix;
    ctx->pending[ctx->lane].q = q;
    ctx->pending[ctx->lane].nq = nq;
    ctx->pending[ctx->lane].k = k;
    return VSK_OK;
  }
  ctx->stats.searches++;
  ctx->stats.queries += nq;
  float* qnorm = nullptr;
  if (ix->metric == VSK_METRIC_COSINE) {
    void* p;
    VSK_TRY(scratch(ctx, SLOT_QNORM, nq * sizeof(float), &p));
    qnorm = (float*)p;
    VSK_TRY(launch_row_norms(ctx, q, nq, ix->dim, 0, qnorm));
  }
  return tensor_search_begin(ix, q, nq, k, qnorm, nullptr, shards, bound);
}

int32_t vsk_search_shard_finish_dev(vsk_index* i, const float* bound, float* out_dist, int64_t* out_ids) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (!bound || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  if (!ctx->pending[ctx->lane].active || ctx->pending[ctx->lane].ix != ix)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "no search is waiting for its second half on this index");
  if (!ctx->pending[ctx->lane].tensor) {
    const ShardPending pd = ctx->pending[ctx->lane];
    ctx->pending[ctx->lane] = ShardPending{};
    return flat_search_dev(ix, pd.q, pd.nq, pd.k, nullptr, out_dist, out_ids);
  }
  VSK_TRY(tensor_search_finish(ix, bound, out_dist, out_ids));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_search(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, float* out_dist,
                   int64_t* out_ids) {
  VSK_TRACE("vsk_search");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (nq <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no queries");
  if (k <= 0) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be positive");
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  void *dq, *dd, *di, *dm = nullptr;
  VSK_TRY(scratch(ctx, SLOT_Q, (size_t)nq * ix->dim * 4, &dq));
  VSK_TRY(scratch(ctx, SLOT_OUT_D, (size_t)nq * k * 4, &dd));
  VSK_TRY(scratch(ctx, SLOT_OUT_I, (size_t)nq * k * 8, &di));
  VSK_CUDA(ctx, cudaMemcpyAsync(dq, q, (size_t)nq * ix->dim * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (qmasks) {
    VSK_TRY(scratch(ctx, SLOT_QMASK, (size_t)nq * 8, &dm));
    VSK_CUDA(ctx, cudaMemcpyAsync(dm, qmasks, (size_t)nq * 8, cudaMemcpyHostToDevice, ctx->stream));
  }
  VSK_TRY(vsk_search_dev(i, (const float*)dq, nq, k, (const uint64_t*)dm, (float*)dd, (int64_t*)di));
  VSK_CUDA(ctx, cudaMemcpyAsync(out_dist, dd, (size_t)nq * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(out_ids, di, (size_t)nq * k * 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.h2d_bytes += nq * ix->dim * 4 + (qmasks ? nq * 8 : 0);
  ctx->stats.d2h_bytes += nq * k * 12;
  return VSK_OK;
}

int32_t vsk_merge_topk_dev(vsk_ctx* c, const float* dist, const int64_t* ids, int32_t g, int64_t nq, int32_t k,
                           float* out_dist, int64_t* out_ids) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (g <= 0 || nq <= 0 || k <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "nothing to merge");
  if (!dist || !ids || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  VSK_TRY(launch_merge_topk(ctx, dist, ids, g, nq, k, out_dist, out_ids));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // extern "C"
