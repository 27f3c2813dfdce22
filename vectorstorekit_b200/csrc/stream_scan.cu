// fp32 scan for a batch of at most eight queries: bound by HBM, not by arithmetic.
//
// The 128 x 128 (or 32 x 128) tile of exact_scan.cu pads a batch to at least 32 query rows, so a
// single query pays for 32: with one query over 5 M x 256 rows the tile spends 2 ms on padded lanes
// where the rows themselves cross HBM in 0.8 ms.  Here the queries sit in shared memory, every warp
// streams two rows at a time with 16-byte loads (each row read from HBM exactly once, coalesced),
// each lane accumulates its slice of every (row, query) pair with the reference's direct formulas
// (DistanceShaders.metal:75-82, 121-134, 171-175, 211-217), a halving exchange leaves each pair's
// total on one lane, and that lane applies the candidate filter of the search schedule.  Rows that
// no query of the batch may see (metadata masks) are not read at all.
//
// This is the path of VectorStore.search (one query), of small filtered or Manhattan batches, and
// of the few queries a tensor-path search re-runs when their certificate fails.  With per-query row
// lists (ExactScanArgs::seg_begin) it is also the IVF search of a few queries: one grid row per query,
// each over the rows of its own probed lists.  vsk_tuning.stream_scan = 0 switches it off.  A lane sums its
// own dimensions first and the lanes are added afterwards, so a value can differ from the tile's
// (dimension-order) sum in the last bits.
#include "common.cuh"
#include "tile_core.cuh"

namespace vsk {
namespace {

constexpr int SS_THREADS = 256;
// Rows per warp step (template parameter): a staged query value is used for all of them.

// v[0..V) per lane -> the total over the warp of v[j] on the lanes with (lane >> (5 - log2 V)) == j, in v[0].
// Each stage halves the values a lane still carries: a lane keeps the half its lane bit selects and hands the
// other half to its partner, so V values cost V - 1 + (5 - log2 V) shuffles instead of 5 V.
template <int V>
__device__ __forceinline__ void warp_reduce_scatter(float (&v)[V], int lane) {
  int off = 16;
#pragma unroll
  for (int c = V; c > 1; c >>= 1) {
    const int h = c >> 1;
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < h; ++j) {
      const float keep = upper ? v[j + h] : v[j];
      const float send = upper ? v[j] : v[j + h];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
    off >>= 1;
  }
  for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

template <int V> struct Log2 { static constexpr int value = 1 + Log2<V / 2>::value; };
template <> struct Log2<1> { static constexpr int value = 0; };

// SEG: every query scans its own slice of the row list (NQ = 1; blockIdx.y is the query's position).
template <int METRIC, int MODE, int NQ, bool VEC, bool SEG, int SS_ROWS>
__global__ void __launch_bounds__(SS_THREADS, NQ > 4 ? 3 : 4) stream_scan_kernel(ExactScanArgs a) {
  static_assert(!SEG || NQ == 1, "per-query row lists are scanned one query per grid row");
  const int qb = SEG ? (int)blockIdx.y : 0;            // first query position of this CTA
  const int nq_here = SEG ? 1 : (int)a.nq;             // queries of this CTA
  // slices belong to queries, not to list positions (a re-run of some queries keeps their slices)
  const int qseg = SEG ? (a.q_subset ? a.q_subset[qb] : qb) : 0;
  const int32_t* x_rows = SEG ? a.x_rows + a.seg_begin[qseg] : a.x_rows;
  // positions at or beyond the slice's length hold no row (a dense chunk still owns their slots)
  const int64_t live_end = SEG ? min(a.row_end, (int64_t)a.seg_count[qseg]) : a.row_end;
  extern __shared__ __align__(16) float sq[];   // [NQ][dim]; rows of queries beyond nq are zero
  __shared__ float s_thr[NQ], s_qn[NQ];
  __shared__ uint64_t s_qm[NQ];
  __shared__ uint64_t s_any;
  const int dim = a.dim;
  const int lane = threadIdx.x & 31;
  for (int idx = threadIdx.x; idx < NQ * dim; idx += SS_THREADS) {
    const int i = idx / dim, k = idx - i * dim;
    float v = 0.f;
    if (i < nq_here) {
      const int64_t qi = a.q_subset ? (int64_t)a.q_subset[qb + i] : qb + i;
      v = a.q[qi * dim + k];
    }
    sq[idx] = v;
  }
  if (threadIdx.x < NQ) {
    const int i = threadIdx.x;
    const bool mok = i < nq_here;
    const int64_t qi = mok ? (a.q_subset ? (int64_t)a.q_subset[qb + i] : qb + i) : 0;
    s_thr[i] = (MODE == SCAN_THRESHOLD && mok) ? a.cand.thr[qb + i] : 0.f;
    s_qn[i] = (METRIC == VSK_METRIC_COSINE && mok) ? a.qnorm[qi] : 0.f;
    s_qm[i] = mok ? (a.q_masks ? a.q_masks[qi] : ~0ull) : 0ull;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint64_t any = 0;
    for (int i = 0; i < NQ; ++i) any |= s_qm[i];
    s_any = any;
  }
  __syncthreads();
  const uint64_t any_mask = s_any;

  constexpr int V = SS_ROWS * NQ;
  constexpr int OWNER_SHIFT = 5 - Log2<V>::value;
  const int warps = SS_THREADS >> 5;
  const int64_t step = (int64_t)gridDim.x * warps * SS_ROWS;
  for (int64_t n0 = a.row_begin + ((int64_t)blockIdx.x * warps + (threadIdx.x >> 5)) * SS_ROWS; n0 < a.row_end;
       n0 += step) {
    bool ok[SS_ROWS], live[SS_ROWS];
    uint32_t rid[SS_ROWS];
    uint64_t rmask[SS_ROWS];
#pragma unroll
    for (int r = 0; r < SS_ROWS; ++r) {
      const int64_t n = n0 + r;
      ok[r] = n < a.row_end;
      const bool has = n < live_end;
      rid[r] = has ? (x_rows ? (uint32_t)x_rows[n] : (uint32_t)n) : 0u;
      rmask[r] = (a.row_masks && has) ? a.row_masks[rid[r]] : ~0ull;
      live[r] = has && (rmask[r] & any_mask) != 0;     // a row no query may see is not read
    }
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    if (VEC) {
      const int nv = dim >> 2;
      const float4* p[SS_ROWS];
#pragma unroll
      for (int r = 0; r < SS_ROWS; ++r) p[r] = reinterpret_cast<const float4*>(a.x + (int64_t)rid[r] * dim);
      const float4* sq4 = reinterpret_cast<const float4*>(sq);
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = lane; c < nv; c += 64) {
        // four 16-byte loads in flight per lane before the first is used
        const int c2 = c + 32;
        const bool two = c2 < nv;
        float4 x[SS_ROWS][2];
#pragma unroll
        for (int r = 0; r < SS_ROWS; ++r) {
          x[r][0] = live[r] ? __ldg(p[r] + c) : zero;
          x[r][1] = (live[r] && two) ? __ldg(p[r] + c2) : zero;
        }
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
          const float4 q = sq4[i * nv + c];
#pragma unroll
          for (int r = 0; r < SS_ROWS; ++r) {
            tile::accum<METRIC>(acc[r * NQ + i], q.x, x[r][0].x);
            tile::accum<METRIC>(acc[r * NQ + i], q.y, x[r][0].y);
            tile::accum<METRIC>(acc[r * NQ + i], q.z, x[r][0].z);
            tile::accum<METRIC>(acc[r * NQ + i], q.w, x[r][0].w);
          }
        }
        if (two) {
#pragma unroll
          for (int i = 0; i < NQ; ++i) {
            const float4 q = sq4[i * nv + c2];
#pragma unroll
            for (int r = 0; r < SS_ROWS; ++r) {
              tile::accum<METRIC>(acc[r * NQ + i], q.x, x[r][1].x);
              tile::accum<METRIC>(acc[r * NQ + i], q.y, x[r][1].y);
              tile::accum<METRIC>(acc[r * NQ + i], q.z, x[r][1].z);
              tile::accum<METRIC>(acc[r * NQ + i], q.w, x[r][1].w);
            }
          }
        }
      }
    } else {
      for (int k = lane; k < dim; k += 32) {
        float x[SS_ROWS];
#pragma unroll
        for (int r = 0; r < SS_ROWS; ++r) x[r] = live[r] ? __ldg(a.x + (int64_t)rid[r] * dim + k) : 0.f;
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
          const float q = sq[i * dim + k];
#pragma unroll
          for (int r = 0; r < SS_ROWS; ++r) tile::accum<METRIC>(acc[r * NQ + i], q, x[r]);
        }
      }
    }
    warp_reduce_scatter<V>(acc, lane);
    // the lane that owns pair j = lane >> OWNER_SHIFT finishes it
    if ((lane & ((1 << OWNER_SHIFT) - 1)) != 0) continue;
    const int j = lane >> OWNER_SHIFT;
    const int r = j / NQ, i = j - r * NQ;
    // (r is a run-time value here: pick the row's fields without indexing the register arrays)
    bool okr = ok[0], liver = live[0];
    uint32_t ridr = rid[0];
    uint64_t rmaskr = rmask[0];
#pragma unroll
    for (int t = 1; t < SS_ROWS; ++t)
      if (r == t) { okr = ok[t]; liver = live[t]; ridr = rid[t]; rmaskr = rmask[t]; }
    if (!okr || i >= nq_here) continue;
    float v = acc[0];
    if (METRIC == VSK_METRIC_COSINE) v = 1.0f - v / (s_qn[i] * (liver ? a.xnorm[ridr] : 0.f) + 1e-8f);
    else if (METRIC == VSK_METRIC_DOT_PRODUCT) v = -v;
    const bool elig = liver && (rmaskr & s_qm[i]) != 0;
    if (MODE == SCAN_DENSE) {
      a.cand.keys[(int64_t)(qb + i) * kCandCap + (n0 + r - a.row_begin)] = elig ? make_key(v, ridr) : kEmptyKey;
    } else {
      if (elig && v <= s_thr[i]) {
        const int pos = atomicAdd(&a.cand.count[qb + i], 1);
        if (pos < kCandCap) a.cand.keys[(int64_t)(qb + i) * kCandCap + pos] = make_key(v, ridr);
      }
    }
  }
}

template <int METRIC, int MODE, int NQ, int ROWS>
int32_t launch_rows(Ctx* ctx, const ExactScanArgs& a, bool vec) {
  const int64_t rows = a.row_end - a.row_begin;
  const int warps = SS_THREADS / 32;
  const int64_t want = ceil_div(rows, (int64_t)warps * ROWS);
  const int nseg = a.seg_begin ? (int)a.nq : 1;   // per-query row lists: grid (CTAs over the chunk's positions, queries)
  const int64_t cap = std::max<int64_t>(1, (int64_t)ctx->prop.multiProcessorCount * (NQ > 4 ? 3 : 4) / nseg);
  dim3 grid((unsigned)std::max<int64_t>(1, std::min(want, cap)), (unsigned)nseg);
  const size_t smem = (size_t)NQ * a.dim * sizeof(float);
  prof_begin(ctx);
  if constexpr (NQ == 1) {
    if (a.seg_begin) {
      if (vec) stream_scan_kernel<METRIC, MODE, 1, true, true, ROWS><<<grid, SS_THREADS, smem, ctx->stream>>>(a);
      else stream_scan_kernel<METRIC, MODE, 1, false, true, ROWS><<<grid, SS_THREADS, smem, ctx->stream>>>(a);
    }
  }
  if (!a.seg_begin) {
    if (vec) stream_scan_kernel<METRIC, MODE, NQ, true, false, ROWS><<<grid, SS_THREADS, smem, ctx->stream>>>(a);
    else stream_scan_kernel<METRIC, MODE, NQ, false, false, ROWS><<<grid, SS_THREADS, smem, ctx->stream>>>(a);
  }
  prof_end(ctx);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

template <int METRIC, int MODE, int NQ>
int32_t launch_nq(Ctx* ctx, const ExactScanArgs& a, bool vec) {
  // four rows per step were measured for one and two queries over rows of at most 1 KB: slower than two (one query
  // over 5 M x 256: 0.47 against 0.43 ms), so every launch takes two
  return launch_rows<METRIC, MODE, NQ, 2>(ctx, a, vec);
}

template <int METRIC, int MODE>
int32_t launch_mode(Ctx* ctx, const ExactScanArgs& a, bool vec) {
  if (a.seg_begin) return launch_nq<METRIC, MODE, 1>(ctx, a, vec);   // one query per grid row
  if (a.nq <= 1) return launch_nq<METRIC, MODE, 1>(ctx, a, vec);
  if (a.nq <= 2) return launch_nq<METRIC, MODE, 2>(ctx, a, vec);
  if (a.nq <= 4) return launch_nq<METRIC, MODE, 4>(ctx, a, vec);
  return launch_nq<METRIC, MODE, 8>(ctx, a, vec);
}

template <int METRIC>
int32_t launch_stream_metric(Ctx* ctx, const ExactScanArgs& a, bool vec) {
  if (a.mode == SCAN_DENSE) return launch_mode<METRIC, SCAN_DENSE>(ctx, a, vec);
  return launch_mode<METRIC, SCAN_THRESHOLD>(ctx, a, vec);
}

}  // namespace

bool stream_scan_applies(const Ctx* ctx, const ExactScanArgs& a) {
  if (!ctx->tuning.stream_scan) return false;
  if (a.x_codes != nullptr || a.x == nullptr) return false;                 // fp32 rows only
  if (a.mode != SCAN_DENSE && a.mode != SCAN_THRESHOLD) return false;       // candidate modes only
  // the queries stay in shared memory: the staged rows (1, 2, 4 or 8 of them) plus the kernel's few static words
  // must fit the 48 KB a launch gets without opting in to more
  constexpr size_t kSmemBudget = 48 * 1024 - 512;
  if (a.seg_begin) {
    return a.x_rows != nullptr && a.seg_count != nullptr && a.nq >= 1 && a.nq <= kStreamScanMaxSegQueries &&
           (size_t)a.dim * sizeof(float) <= kSmemBudget;
  }
  if (a.nq < 1 || a.nq > kStreamScanMaxQueries) return false;
  const size_t staged = a.nq <= 1 ? 1 : (a.nq <= 2 ? 2 : (a.nq <= 4 ? 4 : 8));
  return staged * a.dim * sizeof(float) <= kSmemBudget;
}

int32_t launch_stream_scan(Ctx* ctx, const ExactScanArgs& a) {
  if (a.row_end <= a.row_begin) return VSK_OK;
  const bool vec = (a.dim % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
  switch (a.metric) {
    case VSK_METRIC_EUCLIDEAN: return launch_stream_metric<VSK_METRIC_EUCLIDEAN>(ctx, a, vec);
    case VSK_METRIC_COSINE: return launch_stream_metric<VSK_METRIC_COSINE>(ctx, a, vec);
    case VSK_METRIC_DOT_PRODUCT: return launch_stream_metric<VSK_METRIC_DOT_PRODUCT>(ctx, a, vec);
    case VSK_METRIC_MANHATTAN: return launch_stream_metric<VSK_METRIC_MANHATTAN>(ctx, a, vec);
    default: return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", a.metric);
  }
}

}  // namespace vsk
