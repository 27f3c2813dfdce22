// fp32 query x row scan on CUDA cores with the reference's direct formulas
//   euclidean  sum (q-x)^2   (rooted when written out)      DistanceShaders.metal:75-82
//   cosine     1 - q.x/(|q||x| + 1e-8)                        DistanceShaders.metal:121-134
//   dotProduct -(q.x)                                         DistanceShaders.metal:211-217
//   manhattan  sum |q-x|                                      DistanceShaders.metal:171-175
// fused with the per-query candidate filter, so the query x row matrix is never written
// to HBM unless the caller asks for it (SCAN_MATRIX, the reference's topK == nil call).
//
// One CTA computes a 128-query x 128-row tile: 256 threads, 8x8 register micro-tile each,
// operands staged k-major in shared memory in slices of 16 dimensions, double buffered.
// Manhattan and the direct Euclidean form have no tensor-core formulation (abs / square of a
// difference), so this kernel is bound by FP32 issue, not by HBM: each operand element is read
// from HBM/L2 once per tile and reused 128 times.
#include <type_traits>

#include "common.cuh"
#include "tile_core.cuh"

namespace vsk {
namespace {

using namespace tile;

// BM_ = 128 (the default tile) or 32 / 64 query rows per CTA: the narrow tiles keep the padding small when a
// launch has few queries (a group of queries that share a filter mask).
template <int METRIC, int MODE, bool B_INT8, int BM_>
__global__ void __launch_bounds__(THREADS, 2) exact_scan_kernel(ExactScanArgs a) {
  constexpr int QM = BM_ / 16;
  __shared__ __align__(16) typename std::conditional<BM_ == 128, Smem, SmemM<(BM_ == 128 ? 64 : BM_)>>::type sm;
  // 1-D grid over (row tile, query tile): no 65535 limit on either extent
  const int64_t tiles_x = (a.row_end - a.row_begin + BN - 1) / BN;
  const int64_t m0 = ((int64_t)blockIdx.x / tiles_x) * BM_;
  const int64_t n0 = a.row_begin + ((int64_t)blockIdx.x % tiles_x) * BN;
  const int dim = a.dim;

  auto query_row = [&](int64_t m, bool in_tile) {
    F32Row r;
    r.ok = in_tile && m < a.nq;
    const int64_t qi = r.ok ? (a.q_subset ? (int64_t)a.q_subset[m] : m) : 0;
    r.base = a.q + qi * dim;
    r.vec = (dim % 4 == 0) && aligned16(a.q);
    return r;
  };
  typename std::conditional<B_INT8, I8Row, F32Row>::type br[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int64_t n = n0 + stage_row(h);
    br[h].ok = n < a.row_end;
    // x_rows: the scan walks a list of row numbers instead of a contiguous range
    const int64_t row = br[h].ok ? (a.x_rows ? (int64_t)a.x_rows[n] : n) : 0;
    if constexpr (B_INT8) {
      br[h].base = a.x_codes + row * dim;
      br[h].scale = a.sq_scale;
      br[h].offset = a.sq_offset;
      br[h].vec = (dim % 4 == 0) && aligned4(a.x_codes);
    } else {
      br[h].base = a.x + row * dim;
      br[h].vec = (dim % 4 == 0) && aligned16(a.x);
    }
  }

  float acc[QM][8];
  if constexpr (BM_ == 128) {
    F32Row ar[2] = {query_row(m0 + stage_row(0), true), query_row(m0 + stage_row(1), true)};
    mainloop<METRIC>(acc, ar, br, dim, sm);
  } else {
    F32Row ar = query_row(m0 + stage_row(0), stage_row(0) < BM_);
    mainloop_m<METRIC, BM_>(acc, ar, br, dim, sm);
  }

  // ---- epilogue: distance value, filter, candidate append --------------------------------
  int64_t ncol[8];
  uint32_t rid[8];     // row id stored in a key
  float xn[8];
  uint64_t rmask[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    ncol[j] = n0 + tile_col(j);
    const bool ok = ncol[j] < a.row_end;
    rid[j] = ok ? (a.x_rows ? (uint32_t)a.x_rows[ncol[j]] : (uint32_t)ncol[j]) : 0u;
    xn[j] = (METRIC == VSK_METRIC_COSINE && ok) ? a.xnorm[rid[j]] : 0.f;
    rmask[j] = (a.row_masks && ok) ? a.row_masks[rid[j]] : ~0ull;
  }
#pragma unroll
  for (int i = 0; i < QM; ++i) {
    const int64_t m = m0 + (BM_ == 128 ? tile_row(i) : mrow<BM_>(i));
    const bool mok = m < a.nq;
    const int64_t qi = mok ? (a.q_subset ? (int64_t)a.q_subset[m] : m) : 0;
    const float qn = (METRIC == VSK_METRIC_COSINE && mok) ? a.qnorm[qi] : 0.f;
    const uint64_t qm = (a.q_masks && mok) ? a.q_masks[qi] : ~0ull;
    const float thr = (MODE == SCAN_THRESHOLD && mok) ? a.cand.thr[m] : 0.f;
    uint64_t best = kEmptyKey;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool ok = mok && ncol[j] < a.row_end;
      float v;
      if (METRIC == VSK_METRIC_COSINE) v = 1.0f - acc[i][j] / (qn * xn[j] + 1e-8f);
      else if (METRIC == VSK_METRIC_DOT_PRODUCT) v = -acc[i][j];
      else v = acc[i][j];
      const bool elig = (rmask[j] & qm) != 0;
      if (MODE == SCAN_MATRIX) {
        if (METRIC == VSK_METRIC_EUCLIDEAN) v = sqrtf(v);
        if (ok) a.out[m * a.ld_out + (ncol[j] - a.row_begin)] = v;
      } else if (MODE == SCAN_DENSE) {
        if (ok)
          a.cand.keys[m * kCandCap + (ncol[j] - a.row_begin)] = elig ? make_key(v, rid[j]) : kEmptyKey;
      } else if (MODE == SCAN_THRESHOLD) {
        if (ok && elig && v <= thr) {
          const int pos = atomicAdd(&a.cand.count[m], 1);
          if (pos < kCandCap) a.cand.keys[m * kCandCap + pos] = make_key(v, rid[j]);
        }
      } else {  // SCAN_ARGMIN: smallest (value, column) key of the row
        if (ok) best = min(best, make_key(v, rid[j]));
      }
    }
    if (MODE == SCAN_ARGMIN) {
      // the 16 lanes that share this block row hold the other columns
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
      if ((threadIdx.x & 15) == 0 && mok && best != kEmptyKey) atomicMin(a.best + m, (unsigned long long)best);
    }
  }
}

template <int METRIC>
int32_t launch_metric(Ctx* ctx, const ExactScanArgs& a) {
  const int64_t rows = a.row_end - a.row_begin;
  if (rows <= 0 || a.nq <= 0) return VSK_OK;
  const bool i8 = a.x_codes != nullptr;
  // narrow query tiles (fp32 rows, candidate modes only) when they waste clearly fewer padded query rows
  int bm = 128;
  if (!i8 && (a.mode == SCAN_DENSE || a.mode == SCAN_THRESHOLD) && a.bm_hint > 0) bm = a.bm_hint;
  const int64_t tiles = ceil_div(rows, BN) * ceil_div(a.nq, bm);
  if (tiles > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many tiles in one launch");
  dim3 grid((unsigned)tiles);
  prof_begin(ctx);
#define VSK_LAUNCH(MODE_)                                                                             \
  if (i8) exact_scan_kernel<METRIC, MODE_, true, 128><<<grid, THREADS, 0, ctx->stream>>>(a);          \
  else exact_scan_kernel<METRIC, MODE_, false, 128><<<grid, THREADS, 0, ctx->stream>>>(a)
#define VSK_LAUNCH_M(MODE_)                                                                           \
  if (bm == 32) exact_scan_kernel<METRIC, MODE_, false, 32><<<grid, THREADS, 0, ctx->stream>>>(a);    \
  else if (bm == 64) exact_scan_kernel<METRIC, MODE_, false, 64><<<grid, THREADS, 0, ctx->stream>>>(a); \
  else { VSK_LAUNCH(MODE_); }
  switch (a.mode) {
    case SCAN_DENSE: VSK_LAUNCH_M(SCAN_DENSE); break;
    case SCAN_THRESHOLD: VSK_LAUNCH_M(SCAN_THRESHOLD); break;
    case SCAN_ARGMIN: VSK_LAUNCH(SCAN_ARGMIN); break;
    default: VSK_LAUNCH(SCAN_MATRIX); break;
  }
#undef VSK_LAUNCH_M
#undef VSK_LAUNCH
  prof_end(ctx);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

// |x| or |x|^2 per row: one warp per row, lanes stride the dimensions.
__global__ void row_norm_kernel(const float* __restrict__ x, int64_t n, int dim, int squared,
                                float* __restrict__ out) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float* p = x + row * dim;
  float s = 0.f;
  for (int i = lane; i < dim; i += 32) {
    float v = __ldg(p + i);
    s = fmaf(v, v, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[row] = squared ? s : sqrtf(s);
}

}  // namespace

int32_t launch_exact_scan(Ctx* ctx, const ExactScanArgs& a) {
  if (stream_scan_applies(ctx, a)) return launch_stream_scan(ctx, a);   // a few queries: HBM-bound streaming kernel
  if (a.seg_begin) return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "per-query row lists need the streaming scan");
  switch (a.metric) {
    case VSK_METRIC_EUCLIDEAN: return launch_metric<VSK_METRIC_EUCLIDEAN>(ctx, a);
    case VSK_METRIC_COSINE: return launch_metric<VSK_METRIC_COSINE>(ctx, a);
    case VSK_METRIC_DOT_PRODUCT: return launch_metric<VSK_METRIC_DOT_PRODUCT>(ctx, a);
    case VSK_METRIC_MANHATTAN: return launch_metric<VSK_METRIC_MANHATTAN>(ctx, a);
    default: return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", a.metric);
  }
}

int32_t launch_row_norms(Ctx* ctx, const float* x, int64_t n, int32_t dim, int squared, float* out) {
  if (n <= 0) return VSK_OK;
  const int warps = 8;
  static bool carveout_done = false;
  if (!carveout_done) {
    prefer_shared_carveout(row_norm_kernel);
    carveout_done = true;
  }
  row_norm_kernel<<<(unsigned)ceil_div(n, warps), warps * 32, 0, ctx->stream>>>(x, n, dim, squared, out);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

}  // namespace vsk
