// Inverted-file index: build (assign rows to trained centroids, store them list by list) and
// search (probe the nprobe nearest lists, exact rooted L2 over their rows, ascending top-k).
// Replaces IVFIndex.insert / IVFIndex.search (Indexes/IVFIndex.swift:80-122,124-202), which walk
// the probed lists one query at a time with scalar loops and a full sort.
//
// With the tensor search path selected, a batch of at least 256 queries is scanned on the tensor cores
// (ivf_tensor_search, tensor_scan.cu): coarse fp16 values filter the rows, every kept row is re-scored exactly, and
// only queries whose candidate list overflowed come back to the fp32 scan below.
//
// The fp32 search is LIST-major.  The (query, probe) pairs of a batch are grouped by list, so that the
// rows of a list are read once for all the queries that probe it: one CTA computes a block of
// 128 probing queries x 128 list rows with the fp32 tile, and appends the rows at or below each
// query's threshold to that query's candidate list.  Probes are processed in stages by probe rank
// (rank 0; 1; 2-3; 4-7; ...), compacting the candidate lists and tightening the thresholds between
// stages, so the number of appended rows per stage stays near k.
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "tile_core.cuh"
#include "tensor_scan.cuh"

namespace vsk {
namespace {

using namespace tile;


struct IvfScanArgs {
  const float* q;            // [nq][dim]
  const float* rows;         // list-major rows
  int32_t dim;
  const int64_t* list_off;   // [nlist+1] storage range of each list
  const int32_t* list_rows;  // [n] original row id of each stored row
  int32_t nlist;
  int32_t slots;             // items per query = nprobe + 1 (last slot: remainder of the rank-0 list)
  const int32_t* order;      // pair items grouped by (stage, list)
  const int64_t* pair_off;   // [nkeys+1]
  int32_t stage;
  const int64_t* item_off;   // [nlist+1] first CTA of each list in this launch
  int64_t win_lo, win_hi;    // row window inside every list for this launch
  int32_t remainder_lo;      // remainder items only take rows >= this (the pilot window of stage 0)
  int32_t bm;                // "a" rows per CTA for this launch: 32, 64 or 128
  const int32_t* q_subset;   // or null: list position -> query
  CandLists cand;
  // filter (or null): stored row s may be appended for query q iff (row_masks[s] & q_masks[q]) != 0, applied before
  // the distance can count - the reference filters the probed candidates first (IVFIndex.swift:162-165)
  const uint64_t* row_masks;
  const uint64_t* q_masks;
};

template <int BM_>
__global__ void __launch_bounds__(THREADS, 2) ivf_scan_kernel(IvfScanArgs a) {
  constexpr int QM = BM_ / 16;
  __shared__ __align__(16) typename std::conditional<BM_ == 128, Smem, SmemM<(BM_ == 128 ? 64 : BM_)>>::type sm;
  __shared__ int s_list;
  // which list does this CTA belong to: last l with item_off[l] <= blockIdx.x
  if (threadIdx.x == 0) {
    int lo = 0, hi = a.nlist;
    const int64_t b = blockIdx.x;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.item_off[mid] <= b) lo = mid; else hi = mid;
    }
    s_list = lo;
  }
  __syncthreads();
  const int l = s_list;
  const int64_t local = (int64_t)blockIdx.x - a.item_off[l];
  const int64_t lbeg = a.list_off[l], len = a.list_off[l + 1] - lbeg;
  const int64_t wlo = min(a.win_lo, len), whi = min(a.win_hi, len);
  const int64_t rtiles = (whi - wlo + BN - 1) / BN;
  const int64_t qt = local / rtiles, rt = local % rtiles;
  const int64_t pbeg = a.pair_off[(int64_t)a.stage * a.nlist + l] + qt * BM_;
  const int64_t pend = a.pair_off[(int64_t)a.stage * a.nlist + l + 1];
  const int64_t r0 = wlo + rt * BN;  // first row (inside the list) of this block
  const int dim = a.dim;

  auto query_row = [&](int64_t p) {
    F32Row r;
    r.ok = p < pend;
    int64_t q = 0;
    if (r.ok) {
      const int pos = a.order[p] / a.slots;
      q = a.q_subset ? a.q_subset[pos] : pos;
    }
    r.base = a.q + q * dim;
    r.vec = (dim % 4 == 0) && aligned16(a.q);
    return r;
  };
  F32Row br[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int64_t r = r0 + stage_row(h);
    br[h].ok = r < whi;
    br[h].base = a.rows + (lbeg + (br[h].ok ? r : 0)) * dim;
    br[h].vec = (dim % 4 == 0) && aligned16(a.rows);
  }
  float acc[QM][8];
  if constexpr (BM_ == 128) {
    F32Row ar[2] = {query_row(pbeg + stage_row(0)), query_row(pbeg + stage_row(1))};
    mainloop<VSK_METRIC_EUCLIDEAN>(acc, ar, br, dim, sm);
  } else {
    F32Row ar = query_row(pbeg + stage_row(0));
    if (stage_row(0) >= BM_) ar.ok = false;
    mainloop_m<VSK_METRIC_EUCLIDEAN, BM_>(acc, ar, br, dim, sm);
  }

#pragma unroll
  for (int i = 0; i < QM; ++i) {
    const int64_t p = pbeg + (BM_ == 128 ? tile_row(i) : mrow<BM_>(i));
    if (p >= pend) continue;
    const int item = a.order[p];
    const int pos = item / a.slots;
    const bool remainder = (item - pos * a.slots) == a.slots - 1;
    const float thr = a.cand.thr[pos];
    const uint64_t qm = a.q_masks ? a.q_masks[a.q_subset ? a.q_subset[pos] : pos] : ~0ull;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t r = r0 + tile_col(j);
      if (r >= whi || (remainder && r < a.remainder_lo)) continue;
      const float v = acc[i][j];
      if (v <= thr && (!a.row_masks || (a.row_masks[lbeg + r] & qm) != 0ull)) {
        const int slot = atomicAdd(&a.cand.count[pos], 1);
        if (slot < kCandCap) a.cand.keys[(int64_t)pos * kCandCap + slot] = make_key(v, (uint32_t)a.list_rows[lbeg + r]);
      }
    }
  }
}

// Grouping key of every (query, slot) item: stage * nlist + list, or the null key.  stage_of_rank[p] is the
// stage of probe rank p; the remainder slot (rows of the nearest list beyond the pilot window) joins stage 1
// when that list is longer than the pilot window.  per_rank: every rank is its own stage, no remainder item
// (the re-run of overflowed queries).
__global__ void ivf_pair_keys_kernel(const int64_t* __restrict__ probes, int64_t npos, int nprobe, int nlist,
                                     const int64_t* __restrict__ list_off, int per_rank, int pilot_rows,
                                     const int32_t* __restrict__ stage_of_rank, int null_key,
                                     const int32_t* __restrict__ q_subset, int32_t* __restrict__ keys) {
  const int slots = nprobe + 1;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= npos * slots) return;
  const int64_t pos = i / slots;
  const int p = (int)(i - pos * slots);
  const int64_t q = q_subset ? q_subset[pos] : pos;
  int key = null_key;
  if (p < nprobe) {
    const int64_t l = probes[q * nprobe + p];
    if (l >= 0) key = (per_rank ? p : stage_of_rank[p]) * nlist + (int)l;
  } else if (!per_rank) {
    const int64_t l = probes[q * nprobe];
    if (l >= 0 && list_off[l + 1] - list_off[l] > pilot_rows) key = 1 * nlist + (int)l;
  }
  keys[i] = key;
}

// CTAs per list for one launch: ceil(pairs/128) * ceil(window rows/128)
__global__ void ivf_item_count_kernel(const int64_t* pair_off, int stage, int nlist, const int64_t* list_off,
                                      int64_t win_lo, int64_t win_hi, int bm, int64_t* counts) {
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= nlist) return;
  const int64_t pc = pair_off[(int64_t)stage * nlist + l + 1] - pair_off[(int64_t)stage * nlist + l];
  const int64_t len = list_off[l + 1] - list_off[l];
  const int64_t rows = min(win_hi, len) - min(win_lo, len);
  counts[l] = ((pc + bm - 1) / bm) * ((rows + BN - 1) / BN);
}

__global__ void scan_i64_kernel(const int64_t* totals, int32_t n, int64_t* offsets) {
  __shared__ int64_t carry;
  __shared__ int64_t buf[1024];
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 1024) {
    const int i = base + threadIdx.x;
    const int64_t v = i < n ? totals[i] : 0;
    buf[threadIdx.x] = v;
    __syncthreads();
    for (int o = 1; o < 1024; o <<= 1) {
      const int64_t t = threadIdx.x >= o ? buf[threadIdx.x - o] : 0;
      __syncthreads();
      buf[threadIdx.x] += t;
      __syncthreads();
    }
    if (i < n) offsets[i] = carry + buf[threadIdx.x] - v;
    __syncthreads();
    if (threadIdx.x == 0) carry += buf[1023];
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[n] = carry;
}

__global__ void gather_rows_kernel(const float* __restrict__ src, const int32_t* __restrict__ order, int64_t n,
                                   int dim, float* __restrict__ dst) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const float* s = src + (int64_t)order[row] * dim;
  float* d = dst + row * dim;
  for (int i = threadIdx.x & 31; i < dim; i += 32) d[i] = __ldg(s + i);
}

// One launch of the list scan for `stage` and a row window, followed by a compaction.
int32_t ivf_pass(Ctx* ctx, Index* ix, IvfScanArgs a, int64_t npos, int32_t keep) {
  void *cnt, *off;
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_CNT, (size_t)(ix->nlist + 1) * 8, &cnt));
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_OFF, (size_t)(ix->nlist + 1) * 8, &off));
  ivf_item_count_kernel<<<(unsigned)ceil_div(ix->nlist, 256), 256, 0, ctx->stream>>>(
      a.pair_off, a.stage, ix->nlist, ix->list_offsets, a.win_lo, a.win_hi, a.bm, (int64_t*)cnt);
  scan_i64_kernel<<<1, 1024, 0, ctx->stream>>>((const int64_t*)cnt, ix->nlist, (int64_t*)off);
  ctx->stats.kernel_launches += 2;
  int64_t total = 0;
  VSK_CUDA(ctx, cudaMemcpyAsync(&total, (int64_t*)off + ix->nlist, 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (total > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many list tiles in one launch");
  if (total > 0) {
    a.item_off = (const int64_t*)off;
    prof_begin(ctx);
    if (a.bm == 32) ivf_scan_kernel<32><<<(unsigned)total, THREADS, 0, ctx->stream>>>(a);
    else if (a.bm == 64) ivf_scan_kernel<64><<<(unsigned)total, THREADS, 0, ctx->stream>>>(a);
    else ivf_scan_kernel<128><<<(unsigned)total, THREADS, 0, ctx->stream>>>(a);
    prof_end(ctx);
    ctx->stats.kernel_launches++;
    VSK_CUDA(ctx, cudaGetLastError());
  }
  SelectArgs sel{};
  sel.cand = a.cand;
  sel.nq = npos;
  sel.dense_count = -1;
  sel.keep = keep;
  return launch_select(ctx, sel);
}

int32_t ivf_search_positions(Ctx* ctx, Index* ix, const float* q, int64_t npos, const int32_t* sub_dev,
                             const int64_t* probes, int32_t nprobe, int32_t k, const uint64_t* qmasks, float* out_dist,
                             int64_t* out_ids, bool safe) {
  const int slots = nprobe + 1;
  // ---- stage plan -------------------------------------------------------------------------------------
  // Stage 0 (the pilot) scans a window of each query's nearest list and sets the first thresholds.  Later
  // stages take probe ranks in order; how many ranks a stage may take follows the same rule as the flat
  // schedule (schedule_chunk): the rows a stage adds, relative to the rows already seen, bound the keys it
  // can append to a list.  Rows per rank are estimated by the mean list length.
  const double mean_len = std::max(1.0, (double)ix->n / (double)ix->nlist);
  const int pilot_rows = (int)std::min<int64_t>(kCandCap, std::max<int64_t>(256, ceil_div(16 * (int64_t)k, 128) * 128));
  std::vector<int32_t> stage_of_rank((size_t)nprobe, 0);
  std::vector<int> ranks_in_stage;   // probe ranks per stage (stage 1 also holds the remainder items)
  int nstages;
  if (safe) {
    nstages = nprobe;
    for (int p = 0; p < nprobe; ++p) stage_of_rank[p] = p;
    ranks_in_stage.assign((size_t)nprobe, 1);
  } else {
    ranks_in_stage.push_back(1);
    double seen = std::min<double>(pilot_rows, mean_len);
    int p = 1, st = 1;
    bool first = true;
    while (p < nprobe || first) {
      const double chunk = (double)schedule_chunk((int64_t)seen, k, 0);
      // stage 1 also pays for the rest of the nearest list
      double budget = chunk - (first ? std::max(0.0, mean_len - pilot_rows) : 0.0);
      int take = (int)std::max(1.0, std::floor(budget / mean_len));
      take = std::min(take, nprobe - p);
      for (int i = 0; i < take; ++i) stage_of_rank[p + i] = st;
      ranks_in_stage.push_back(std::max(take, 0));
      seen += (first ? std::max(0.0, mean_len - pilot_rows) : 0.0) + take * mean_len;
      p += std::max(take, 0);
      ++st;
      first = false;
      if (take <= 0) break;
    }
    nstages = st;
  }
  const int nkeys = nstages * ix->nlist + 1;  // + the null key
  const int64_t nitems = npos * slots;
  if (nitems > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many (query, probe) pairs");
  void *keys, *order, *pair_off, *sor;
  VSK_TRY(scratch(ctx, SLOT_IVF_KEYS, (size_t)nitems * 4, &keys));
  VSK_TRY(scratch(ctx, SLOT_IVF_ORDER, (size_t)nitems * 4, &order));
  VSK_TRY(scratch(ctx, SLOT_IVF_PAIR_OFF, (size_t)(nkeys + 1) * 8, &pair_off));
  VSK_TRY(scratch(ctx, SLOT_IVF_STAGES, (size_t)nprobe * 4, &sor));
  VSK_CUDA(ctx, cudaMemcpyAsync(sor, stage_of_rank.data(), (size_t)nprobe * 4, cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // stage_of_rank is a local
  ivf_pair_keys_kernel<<<(unsigned)ceil_div(nitems, 256), 256, 0, ctx->stream>>>(
      probes, npos, nprobe, ix->nlist, ix->list_offsets, safe ? 1 : 0, pilot_rows, (const int32_t*)sor, nkeys - 1, sub_dev,
      (int32_t*)keys);
  ctx->stats.kernel_launches++;
  VSK_TRY(launch_stable_group(ctx, (const int32_t*)keys, nitems, nkeys, (int32_t*)order, (int64_t*)pair_off));

  CandLists cand;
  {
    void* p;
    VSK_TRY(scratch(ctx, SLOT_CAND_KEYS, (size_t)npos * kCandCap * sizeof(uint64_t), &p));
    cand.keys = (uint64_t*)p;
    VSK_TRY(scratch(ctx, SLOT_CAND_COUNT, (size_t)npos * 4, &p));
    cand.count = (int32_t*)p;
    VSK_TRY(scratch(ctx, SLOT_CAND_THR, (size_t)npos * 4, &p));
    cand.thr = (float*)p;
    VSK_TRY(scratch(ctx, SLOT_CAND_FLAGS, (size_t)npos * 4, &p));
    cand.flags = (int32_t*)p;
    cand.nq = npos;
  }
  VSK_TRY(launch_init_cand(ctx, cand, npos));

  IvfScanArgs a{};
  a.q = q;
  a.rows = ix->rows;
  a.dim = ix->dim;
  a.list_off = ix->list_offsets;
  a.list_rows = ix->list_rows;
  a.nlist = ix->nlist;
  a.slots = slots;
  a.order = (const int32_t*)order;
  a.pair_off = (const int64_t*)pair_off;
  a.q_subset = sub_dev;
  a.cand = cand;
  if (qmasks && ix->has_masks) {
    a.row_masks = ix->masks;
    a.q_masks = qmasks;
  }
  a.remainder_lo = pilot_rows;
  int64_t max_len = 0;
  for (int l = 0; l < ix->nlist; ++l) max_len = std::max(max_len, ix->list_offsets_h[l + 1] - ix->list_offsets_h[l]);
  const int64_t room = kCandCap - k;
  for (int s = 0; s < nstages; ++s) {
    a.stage = s;
    // "a" rows per CTA from the mean number of probing queries per list in this stage
    const double per_list = (double)npos * ranks_in_stage[(size_t)s] / (double)ix->nlist + (s == 1 && !safe ? (double)npos / ix->nlist : 0.0);
    a.bm = per_list <= 20.0 ? 32 : (per_list <= 80.0 ? 64 : 128);
    if (!safe) {
      a.win_lo = 0;
      a.win_hi = s == 0 ? pilot_rows : (1ll << 62);
      VSK_TRY(ivf_pass(ctx, ix, a, npos, k));
    } else {
      for (int64_t w = 0; w < std::max<int64_t>(max_len, 1); w += room) {
        a.win_lo = w;
        a.win_hi = w + room;
        VSK_TRY(ivf_pass(ctx, ix, a, npos, k));
      }
    }
  }
  SelectArgs fin{};
  fin.cand = cand;
  fin.nq = npos;
  fin.dense_count = -1;
  fin.keep = k;
  fin.out_dist = out_dist;
  fin.out_ids = out_ids;
  fin.k = k;
  fin.metric = VSK_METRIC_EUCLIDEAN;
  fin.id_base = ix->id_base;
  fin.q_subset = sub_dev;
  fin.final_sqrt = 1;
  VSK_TRY(launch_select(ctx, fin));
  if (!safe) {
    std::vector<int32_t> flags((size_t)npos), bad;
    VSK_CUDA(ctx, cudaMemcpyAsync(flags.data(), cand.flags, npos * 4, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int64_t i = 0; i < npos; ++i)
      if (flags[i]) bad.push_back((int32_t)i);
    if (!bad.empty() && sub_dev) {
      // list positions -> query indices of the caller's batch
      std::vector<int32_t> sub_h((size_t)npos);
      VSK_CUDA(ctx, cudaMemcpy(sub_h.data(), sub_dev, (size_t)npos * 4, cudaMemcpyDeviceToHost));
      for (auto& b : bad) b = sub_h[(size_t)b];
    }
    if (!bad.empty()) {
      void* p;
      VSK_TRY(scratch(ctx, SLOT_IVF_SUBSET, bad.size() * 4, &p));
      VSK_CUDA(ctx, cudaMemcpyAsync(p, bad.data(), bad.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
      VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      ctx->stats.fallback_queries += (int64_t)bad.size();
      VSK_TRY(ivf_search_positions(ctx, ix, q, (int64_t)bad.size(), (const int32_t*)p, probes, nprobe, k, qmasks, out_dist,
                                   out_ids, true));
    }
  }
  return VSK_OK;
}

int32_t ivf_build_dev(Ctx* ctx, const float* centroids, int32_t nlist, const float* rows, int64_t n, int32_t dim,
                      Index** out) {
  *out = nullptr;
  if (nlist <= 0 || !centroids) return fail(ctx, VSK_ERR_NOT_TRAINED, "no centroids: train the index first");
  if (n <= 0 || !rows) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "at most 2^31-1 rows");
  Index* ix = new Index();
  ix->ctx = ctx;
  ix->kind = INDEX_IVF;
  ix->metric = VSK_METRIC_EUCLIDEAN;
  ix->dim = dim;
  ix->n = n;
  ix->capacity = n;
  ix->nlist = nlist;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&ix->centroids, (size_t)nlist * dim * 4)) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&ix->assign, (size_t)n * 4)) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&ix->list_rows, (size_t)n * 4)) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&ix->list_offsets, (size_t)(nlist + 1) * 8)) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&ix->rows, (size_t)n * dim * 4)) != VSK_OK) {
    vsk_index_destroy(reinterpret_cast<vsk_index*>(ix));
    return st;
  }
  auto body = [&]() -> int32_t {
    VSK_CUDA(ctx, cudaMemcpyAsync(ix->centroids, centroids, (size_t)nlist * dim * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_TRY(assign_rows(ctx, rows, n, dim, ix->centroids, nlist, ix->assign, nullptr));
    VSK_TRY(launch_stable_group(ctx, ix->assign, n, nlist, ix->list_rows, ix->list_offsets));
    gather_rows_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(rows, ix->list_rows, n, dim, ix->rows);
    ctx->stats.kernel_launches++;
    ix->list_offsets_h.resize((size_t)nlist + 1);
    VSK_CUDA(ctx, cudaMemcpyAsync(ix->list_offsets_h.data(), ix->list_offsets, (size_t)(nlist + 1) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return VSK_OK;
  };
  st = body();
  if (st != VSK_OK) {
    vsk_index_destroy(reinterpret_cast<vsk_index*>(ix));
    return st;
  }
  *out = ix;
  return VSK_OK;
}

// ---- row masks and incremental insert --------------------------------------------------------------------
// masks in the caller's (insertion) order -> storage order: stored row s holds original row list_rows[s]
__global__ void ivf_permute_masks_kernel(const uint64_t* __restrict__ masks, const int32_t* __restrict__ list_rows,
                                         int64_t n, uint64_t* __restrict__ out) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s < n) out[s] = masks[list_rows[s]];
}

int32_t ivf_set_masks_dev(Index* ix, const uint64_t* masks) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_IVF) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an IVF index");
  if (!masks) return fail(ctx, VSK_ERR_INVALID_INPUT, "null masks");
  if (!ix->masks) VSK_TRY(dev_alloc(ctx, (void**)&ix->masks, (size_t)ix->capacity * sizeof(uint64_t)));
  ivf_permute_masks_kernel<<<(unsigned)ceil_div(ix->n, 256), 256, 0, ctx->stream>>>(masks, ix->list_rows, ix->n, ix->masks);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ix->has_masks = true;
  return VSK_OK;
}

// Appending rows to a built index (IVFIndex.insert, Indexes/IVFIndex.swift:80-122: nearest centroid, append to that
// list).  Only the NEW rows are assigned.  The stored arrays are list-major and contiguous, so the rows already stored
// move up by the number of new rows filed under earlier lists - one pass at copy speed, no distance is recomputed -
// and each list's new rows follow its old ones in arrival order, as appending does.
//   stored row s of list l            -> s + new_off[l]
//   p-th new row (grouped by list) l  -> old_off[l + 1] + p
__global__ void ivf_move_old_kernel(const float* __restrict__ rows, const int32_t* __restrict__ list_rows,
                                    const int32_t* __restrict__ assign, const uint64_t* __restrict__ masks, int64_t n,
                                    int dim, const int64_t* __restrict__ new_off, float* __restrict__ rows_out,
                                    int32_t* __restrict__ list_rows_out, uint64_t* __restrict__ masks_out) {
  const int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= n) return;
  const int lane = threadIdx.x & 31;
  const int32_t orig = list_rows[s];
  const int64_t dst = s + new_off[assign[orig]];
  const float* src = rows + s * dim;
  float* out = rows_out + dst * dim;
  for (int i = lane; i < dim; i += 32) out[i] = __ldg(src + i);
  if (lane == 0) {
    list_rows_out[dst] = orig;
    if (masks_out) masks_out[dst] = masks[s];
  }
}

__global__ void ivf_place_new_kernel(const float* __restrict__ rows, const int32_t* __restrict__ order,
                                     const int32_t* __restrict__ assign_new, const uint64_t* __restrict__ masks,
                                     int64_t m, int dim, const int64_t* __restrict__ old_off, int64_t n_old,
                                     float* __restrict__ rows_out, int32_t* __restrict__ list_rows_out,
                                     uint64_t* __restrict__ masks_out) {
  const int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= m) return;
  const int lane = threadIdx.x & 31;
  const int32_t r = order[p];                    // p-th new row in (list, arrival) order
  const int64_t dst = old_off[assign_new[r] + 1] + p;
  const float* src = rows + (int64_t)r * dim;
  float* out = rows_out + dst * dim;
  for (int i = lane; i < dim; i += 32) out[i] = __ldg(src + i);
  if (lane == 0) {
    list_rows_out[dst] = (int32_t)(n_old + r);
    if (masks_out) masks_out[dst] = masks ? masks[r] : 0ull;
  }
}

__global__ void ivf_add_offsets_kernel(const int64_t* __restrict__ a, const int64_t* __restrict__ b, int n, int64_t* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = a[i] + b[i];
}

int32_t ivf_add_dev(Index* ix, const float* rows, int64_t m, const uint64_t* masks) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_IVF) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an IVF index");
  if (m <= 0 || !rows) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows to add");
  if (ix->n + m > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "an index holds at most 2^31-1 rows");
  if ((masks != nullptr) != ix->has_masks && ix->n > 0)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "either every row of the index carries a mask or none does");
  const int64_t n_old = ix->n, n_new = n_old + m;
  const int dim = ix->dim, nlist = ix->nlist;
  // the new rows' lists, grouped (stable: arrival order inside a list)
  int32_t *assign_out = nullptr, *list_rows_out = nullptr, *order = nullptr;
  int64_t *new_off = nullptr, *off_out = nullptr;
  float* rows_out = nullptr;
  uint64_t* masks_out = nullptr;
  auto body = [&]() -> int32_t {
    VSK_TRY(dev_alloc(ctx, (void**)&assign_out, (size_t)n_new * 4));
    VSK_TRY(dev_alloc(ctx, (void**)&list_rows_out, (size_t)n_new * 4));
    VSK_TRY(dev_alloc(ctx, (void**)&order, (size_t)m * 4));
    VSK_TRY(dev_alloc(ctx, (void**)&new_off, (size_t)(nlist + 1) * 8));
    VSK_TRY(dev_alloc(ctx, (void**)&off_out, (size_t)(nlist + 1) * 8));
    VSK_TRY(dev_alloc(ctx, (void**)&rows_out, (size_t)n_new * dim * 4));
    if (ix->has_masks || masks) VSK_TRY(dev_alloc(ctx, (void**)&masks_out, (size_t)n_new * 8));
    VSK_CUDA(ctx, cudaMemcpyAsync(assign_out, ix->assign, (size_t)n_old * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    int32_t* assign_new = assign_out + n_old;
    VSK_TRY(assign_rows(ctx, rows, m, dim, ix->centroids, nlist, assign_new, nullptr));
    VSK_TRY(launch_stable_group(ctx, assign_new, m, nlist, order, new_off));
    ivf_move_old_kernel<<<(unsigned)ceil_div(n_old, 8), 256, 0, ctx->stream>>>(ix->rows, ix->list_rows, ix->assign, ix->masks, n_old, dim,
                                                                              new_off, rows_out, list_rows_out, masks_out);
    ivf_place_new_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, ctx->stream>>>(rows, order, assign_new, masks, m, dim, ix->list_offsets,
                                                                           n_old, rows_out, list_rows_out, masks_out);
    ivf_add_offsets_kernel<<<(unsigned)ceil_div(nlist + 1, 256), 256, 0, ctx->stream>>>(ix->list_offsets, new_off, nlist + 1, off_out);
    ctx->stats.kernel_launches += 3;
    VSK_CUDA(ctx, cudaGetLastError());
    std::vector<int64_t> off_h((size_t)nlist + 1);
    VSK_CUDA(ctx, cudaMemcpyAsync(off_h.data(), off_out, (size_t)(nlist + 1) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (off_h.back() != n_new) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "list offsets do not add up after the insert");
    ix->list_offsets_h.swap(off_h);
    return VSK_OK;
  };
  const int32_t st = body();
  dev_free(order);
  dev_free(new_off);
  if (st != VSK_OK) {
    dev_free(assign_out); dev_free(list_rows_out); dev_free(off_out); dev_free(rows_out); dev_free(masks_out);
    return st;
  }
  dev_free(ix->assign); dev_free(ix->list_rows); dev_free(ix->list_offsets); dev_free(ix->rows); dev_free(ix->masks);
  ix->assign = assign_out;
  ix->list_rows = list_rows_out;
  ix->list_offsets = off_out;
  ix->rows = rows_out;
  ix->masks = masks_out;
  ix->has_masks = masks_out != nullptr;
  ix->n = ix->capacity = n_new;
  tensor_invalidate(ix);   // the fp16 operand copy is remade at the next tensor-path search
  return VSK_OK;
}

// ---- a few queries: each streams its own probed lists ------------------------------------------------------
// IVFIndex.search is a one-query call (IVFIndex.swift:124-202).  For a handful of queries the list-major tiles
// above pad every (list, query) pair to 32 query rows; here every query gets the row numbers of its probed
// lists as a slice of one row list and the streaming scan reads each of those rows once (for one query over
// 32 of 4 096 lists of a 10 M x 128 index: 40 MB).  Keys carry stored-row numbers; the original row ids are put in
// when the final order is made.

// Entry (query, probe) -> positions [dst, dst + len) of the row list hold stored rows lbeg .. lbeg + len.
__global__ void ivf_expand_lists_kernel(const int64_t* __restrict__ triples, int32_t* __restrict__ rows) {
  const int64_t dst = triples[3 * blockIdx.x], lbeg = triples[3 * blockIdx.x + 1], len = triples[3 * blockIdx.x + 2];
  for (int64_t t = threadIdx.x; t < len; t += blockDim.x) rows[dst + t] = (int32_t)(lbeg + t);
}

// every list, in index order, as each query's probe list
__global__ void ivf_probe_all_kernel(int64_t* __restrict__ probes, int64_t nq, int nprobe) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nq * nprobe) probes[i] = i % nprobe;
}

constexpr int64_t kIvfFewMaxEntries = 32ll << 20;   // row-list entries (128 MB) the few-query path may use

// *handled = false (nothing done) when the batch does not fit this path.
int32_t ivf_search_few(Ctx* ctx, Index* ix, const float* q, int64_t nq, const int64_t* probes, int32_t nprobe,
                       int32_t k, const uint64_t* qmasks, float* out_dist, int64_t* out_ids, bool* handled) {
  *handled = false;
  ExactScanArgs a{};
  a.metric = VSK_METRIC_EUCLIDEAN;
  a.mode = SCAN_DENSE;
  a.q = q;
  a.x = ix->rows;
  a.dim = ix->dim;
  a.nq = nq;
  if (qmasks && ix->has_masks) {   // masks are kept in storage order, like the rows the slices list
    a.row_masks = ix->masks;
    a.q_masks = qmasks;
  }
  std::vector<int64_t> ph((size_t)nq * nprobe);
  VSK_CUDA(ctx, cudaMemcpyAsync(ph.data(), probes, ph.size() * 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::vector<int64_t> triples, seg_begin((size_t)nq);
  std::vector<int32_t> seg_count((size_t)nq);
  triples.reserve(ph.size() * 3);
  int64_t total = 0, longest = 0;
  for (int64_t i = 0; i < nq; ++i) {
    seg_begin[(size_t)i] = total;
    int64_t cnt = 0;
    for (int p = 0; p < nprobe; ++p) {
      const int64_t l = ph[(size_t)(i * nprobe + p)];
      if (l < 0 || l >= ix->nlist) continue;
      const int64_t lbeg = ix->list_offsets_h[(size_t)l], len = ix->list_offsets_h[(size_t)l + 1] - lbeg;
      if (len <= 0) continue;
      triples.push_back(total + cnt);
      triples.push_back(lbeg);
      triples.push_back(len);
      cnt += len;
    }
    if (cnt > 0x7fffffffLL) return VSK_OK;
    seg_count[(size_t)i] = (int32_t)cnt;
    total += cnt;
    longest = std::max(longest, cnt);
  }
  if (total > kIvfFewMaxEntries || total == 0) return VSK_OK;   // too many rows, or nothing to scan: the general path
  void *drows, *dtri, *dbeg, *dcnt;
  VSK_TRY(scratch(ctx, SLOT_IVF_ORDER, (size_t)std::max<int64_t>(total, 1) * 4, &drows));
  VSK_TRY(scratch(ctx, SLOT_IVF_PAIR_OFF, std::max<size_t>(triples.size(), 3) * 8, &dtri));
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_OFF, (size_t)nq * 8, &dbeg));
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_CNT, (size_t)nq * 4, &dcnt));
  a.x_rows = (const int32_t*)drows;
  a.seg_begin = (const int64_t*)dbeg;
  a.seg_count = (const int32_t*)dcnt;
  if (!stream_scan_applies(ctx, a)) return VSK_OK;
  *handled = true;
  if (!triples.empty())
    VSK_CUDA(ctx, cudaMemcpyAsync(dtri, triples.data(), triples.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(dbeg, seg_begin.data(), (size_t)nq * 8, cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(dcnt, seg_count.data(), (size_t)nq * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (!triples.empty()) {
    ivf_expand_lists_kernel<<<(unsigned)(triples.size() / 3), 256, 0, ctx->stream>>>((const int64_t*)dtri, (int32_t*)drows);
    ctx->stats.kernel_launches++;
    VSK_CUDA(ctx, cudaGetLastError());
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // the host vectors are locals
  // the keys carry stored-row numbers; the final ordering swaps in the rows' insertion indices, so that equal
  // distances come out by id as every other search path orders them
  a.final_id_remap = ix->list_rows;
  VSK_TRY(fp32_topk(ctx, a, longest, nq, nullptr, k, ix->id_base, out_dist, out_ids, 0));
  return VSK_OK;
}

int32_t ivf_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                       float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_IVF) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an IVF index");
  if (qmasks && !ix->has_masks) return fail(ctx, VSK_ERR_INVALID_INPUT, "query masks given but the index has no row masks");
  if (nq <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no queries");
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (nprobe <= 0) return fail(ctx, VSK_ERR_INVALID_INPUT, "nprobe must be positive");
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  nprobe = std::min(nprobe, ix->nlist);
  // The probe selection is a top-nprobe over the centroids and shares the candidate lists' limit on k.  Probing
  // every list (the reference's `.exact` strategy, IVFIndex.swift:551-560) needs no selection at all.
  const bool probe_all = nprobe == ix->nlist && nprobe > kCandCap / 2;
  if (nprobe > kCandCap / 2 && !probe_all)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "nprobe must be at most %d, or equal to the number of lists (%d)", kCandCap / 2,
                ix->nlist);
  ctx->stats.searches++;
  ctx->stats.queries += nq;
  constexpr int64_t kBatch = 16384;
  for (int64_t b = 0; b < nq; b += kBatch) {
    const int64_t bn = std::min(kBatch, nq - b);
    const float* qb = q + b * ix->dim;
    const uint64_t* mb = qmasks ? qmasks + b : nullptr;
    // coarse quantiser: the nprobe nearest centroids, ascending (IVFIndex.findNearestCentroids, :529-540)
    void *pd, *pi;
    VSK_TRY(scratch(ctx, SLOT_IVF_PROBE_D, (size_t)bn * nprobe * 4, &pd));
    VSK_TRY(scratch(ctx, SLOT_IVF_PROBE_I, (size_t)bn * nprobe * 8, &pi));
    const bool tensor = ctx->search_path == VSK_PATH_TENSOR_RERANK && ivf_tensor_applicable(ix, bn, nprobe, k);
    if (probe_all) {
      ivf_probe_all_kernel<<<(unsigned)ceil_div(bn * (int64_t)nprobe, 256), 256, 0, ctx->stream>>>((int64_t*)pi, bn, nprobe);
      ctx->stats.kernel_launches++;
      VSK_CUDA(ctx, cudaGetLastError());
    } else if (tensor && ix->nlist >= 1024 && nprobe <= 1024) {
      // the centroids are a flat euclidean index of their own: exact top-nprobe on the tensor path
      if (!ix->coarse) {
        Index* co = new Index();
        co->ctx = ctx;
        co->kind = INDEX_FLAT_F32;
        co->metric = VSK_METRIC_EUCLIDEAN;
        co->dim = ix->dim;
        co->n = co->capacity = ix->nlist;
        co->rows = ix->centroids;
        int32_t cst = dev_alloc(ctx, (void**)&co->row_norm, (size_t)ix->nlist * sizeof(float));
        if (cst == VSK_OK) cst = launch_row_norms(ctx, co->rows, co->n, co->dim, 1, co->row_norm);
        if (cst != VSK_OK) {   // the shadow index exists only once it is complete
          dev_free(co->row_norm);
          delete co;
          return cst;
        }
        ix->coarse = co;
      }
      VSK_TRY(tensor_search(ix->coarse, qb, bn, nprobe, nullptr, nullptr, (float*)pd, (int64_t*)pi));
    } else {
      ExactScanArgs c{};
      c.metric = VSK_METRIC_EUCLIDEAN;
      c.q = qb;
      c.x = ix->centroids;
      c.dim = ix->dim;
      VSK_TRY(fp32_topk(ctx, c, ix->nlist, bn, nullptr, nprobe, 0, (float*)pd, (int64_t*)pi, 0));
    }
    if (tensor) {
      // coarse scan of the probed lists on the tensor cores + exact rerank; what it cannot certify is re-run below
      std::vector<int32_t> redo;
      VSK_TRY(ivf_tensor_search(ix, qb, bn, (const int64_t*)pi, nprobe, k, mb, out_dist + b * k, out_ids + b * k, &redo));
      if (!redo.empty()) {
        void* p;
        VSK_TRY(scratch(ctx, SLOT_MISC4, redo.size() * 4, &p));
        VSK_CUDA(ctx, cudaMemcpyAsync(p, redo.data(), redo.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        ctx->stats.fallback_queries += (int64_t)redo.size();
        VSK_TRY(ivf_search_positions(ctx, ix, qb, (int64_t)redo.size(), (const int32_t*)p, (const int64_t*)pi, nprobe, k, mb,
                                     out_dist + b * k, out_ids + b * k, false));
      }
      continue;
    }
    if (bn <= kStreamScanMaxSegQueries) {
      bool few = false;
      VSK_TRY(ivf_search_few(ctx, ix, qb, bn, (const int64_t*)pi, nprobe, k, mb, out_dist + b * k, out_ids + b * k, &few));
      if (few) continue;
    }
    VSK_TRY(ivf_search_positions(ctx, ix, qb, bn, nullptr, (const int64_t*)pi, nprobe, k, mb, out_dist + b * k,
                                 out_ids + b * k, false));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace

// the IVF search for callers inside the library (the sharded search, comm.cu); the device is already selected
int32_t ivf_search_dev_entry(Index* ix, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                             float* out_dist, int64_t* out_ids) {
  return ivf_search_dev(ix, q, nq, k, nprobe, qmasks, out_dist, out_ids);
}
}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_ivf_build_dev(vsk_ctx* c, const float* centroids, int32_t nlist, const float* rows, int64_t n, int32_t dim,
                          vsk_index** out) {
  VSK_TRACE("vsk_ivf_build_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  return ivf_build_dev(ctx, centroids, nlist, rows, n, dim, reinterpret_cast<Index**>(out));
}

int32_t vsk_ivf_build(vsk_ctx* c, const float* centroids, int32_t nlist, const float* rows, int64_t n, int32_t dim,
                      vsk_index** out) {
  VSK_TRACE("vsk_ivf_build");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  *out = nullptr;
  if (nlist <= 0 || !centroids) return fail(ctx, VSK_ERR_NOT_TRAINED, "no centroids: train the index first");
  if (n <= 0 || !rows) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  float *dc = nullptr, *dx = nullptr;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&dc, (size_t)nlist * dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dx, (size_t)n * dim * 4)) == VSK_OK) {
    cudaMemcpyAsync(dc, centroids, (size_t)nlist * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    cudaMemcpyAsync(dx, rows, (size_t)n * dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    ctx->stats.h2d_bytes += ((int64_t)nlist + n) * dim * 4;
    st = ivf_build_dev(ctx, dc, nlist, dx, n, dim, reinterpret_cast<Index**>(out));
  }
  dev_free(dc);
  dev_free(dx);
  return st;
}

int32_t vsk_ivf_assignments(vsk_index* i, int32_t* assign) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix || !assign) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (ix->kind != INDEX_IVF) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an IVF index");
  VSK_CUDA(ctx, cudaMemcpy(assign, ix->assign, (size_t)ix->n * 4, cudaMemcpyDeviceToHost));
  return VSK_OK;
}

int32_t vsk_ivf_centroids(vsk_index* i, float* centroids) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix || !centroids) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (ix->kind != INDEX_IVF) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an IVF index");
  VSK_CUDA(ctx, cudaMemcpy(centroids, ix->centroids, (size_t)ix->nlist * ix->dim * 4, cudaMemcpyDeviceToHost));
  return VSK_OK;
}

int32_t vsk_ivf_search_filtered_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe,
                                    const uint64_t* qmasks, float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search_filtered_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  return ivf_search_dev(ix, q, nq, k, nprobe, qmasks, out_dist, out_ids);
}

int32_t vsk_ivf_search_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe, float* out_dist,
                           int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search_dev");
  return vsk_ivf_search_filtered_dev(i, q, nq, k, nprobe, nullptr, out_dist, out_ids);
}

int32_t vsk_ivf_set_masks_dev(vsk_index* i, const uint64_t* masks) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  return ivf_set_masks_dev(ix, masks);
}

int32_t vsk_ivf_set_masks(vsk_index* i, const uint64_t* masks) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (!masks) return fail(ctx, VSK_ERR_INVALID_INPUT, "null masks");
  uint64_t* dm = nullptr;
  VSK_TRY(dev_alloc(ctx, (void**)&dm, (size_t)ix->n * 8));
  cudaMemcpyAsync(dm, masks, (size_t)ix->n * 8, cudaMemcpyHostToDevice, ctx->stream);
  ctx->stats.h2d_bytes += ix->n * 8;
  const int32_t st = ivf_set_masks_dev(ix, dm);
  dev_free(dm);
  return st;
}

int32_t vsk_ivf_add_dev(vsk_index* i, const float* rows, int64_t n, const uint64_t* masks) {
  VSK_TRACE("vsk_ivf_add_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  return ivf_add_dev(ix, rows, n, masks);
}

int32_t vsk_ivf_add(vsk_index* i, const float* rows, int64_t n, const uint64_t* masks) {
  VSK_TRACE("vsk_ivf_add");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (n <= 0 || !rows) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows to add");
  float* dx = nullptr;
  uint64_t* dm = nullptr;
  int32_t st = dev_alloc(ctx, (void**)&dx, (size_t)n * ix->dim * 4);
  if (st == VSK_OK && masks) st = dev_alloc(ctx, (void**)&dm, (size_t)n * 8);
  if (st == VSK_OK) {
    cudaMemcpyAsync(dx, rows, (size_t)n * ix->dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (masks) cudaMemcpyAsync(dm, masks, (size_t)n * 8, cudaMemcpyHostToDevice, ctx->stream);
    ctx->stats.h2d_bytes += n * ix->dim * 4 + (masks ? n * 8 : 0);
    st = ivf_add_dev(ix, dx, n, dm);
  }
  dev_free(dx);
  dev_free(dm);
  return st;
}

int32_t vsk_ivf_search(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe, float* out_dist,
                       int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search");
  return vsk_ivf_search_filtered(i, q, nq, k, nprobe, nullptr, out_dist, out_ids);
}

int32_t vsk_ivf_search_filtered(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                                float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search_filtered");
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
    ctx->stats.h2d_bytes += nq * 8;
  }
  VSK_TRY(ivf_search_dev(ix, (const float*)dq, nq, k, nprobe, (const uint64_t*)dm, (float*)dd, (int64_t*)di));
  VSK_CUDA(ctx, cudaMemcpyAsync(out_dist, dd, (size_t)nq * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(out_ids, di, (size_t)nq * k * 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.h2d_bytes += nq * ix->dim * 4;
  ctx->stats.d2h_bytes += nq * k * 12;
  return VSK_OK;
}

}  // extern "C"
