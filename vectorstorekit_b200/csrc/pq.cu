// Product quantisation: codebook training, encode / decode, distance tables and the asymmetric-distance (ADC)
// scan with fused top-k, after ProductQuantizer (Quantization/ProductQuantizer.swift) and its shaders
// (Shaders/QuantizationShaders.metal:113-204).
//
//   codebooks  [m][ksub][ds], ds = dim / m                        (ProductQuantizerCodebook.swift:8-11)
//   code       per segment the nearest codeword by squared L2 accumulated in dimension order, strict '<'
//              (Codebook.encode :12-30): one byte per segment
//   table      t[s][c] = squared L2 between the query's segment s and codeword c       (:205-233)
//   distance   sqrt(sum over s, in order, of t[s][code[s]])       (ProductQuantizerTypes.swift:14-20)
//
// Every sum is formed with separately rounded multiplies and adds in the reference's order, so codes and
// distances equal the CPU restatement bit for bit.  The scan is byte work: per (row, query) m table look-ups in
// shared memory and m adds.  A CTA keeps the tables of TQ queries in shared memory, interleaved by query
// ([segment][code][query]) so that one 16-byte shared-memory load serves four queries, streams blocks of 256
// rows (each thread reads its row's codes from global memory, four segments per 32-bit load) and appends keys to
// the candidate lists of the search schedule (dense first chunk, thresholded later chunks).
#include <math_constants.h>

#include <algorithm>
#include <vector>

#include "common.cuh"

namespace vsk {

int32_t kmeans_dev(Ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k, int32_t max_iters, float tolerance,
                   const float* init, float* centroids, int32_t* assign, float* inertia, int32_t* iters_run);

namespace {

constexpr int PQ_THREADS = 512;
constexpr size_t PQ_SMEM_LIMIT = 200 * 1024;

__device__ __forceinline__ float sqdiff_accum(float acc, float a, float b) {
  const float diff = __fsub_rn(a, b);
  return __fadd_rn(acc, __fmul_rn(diff, diff));
}

// tables[q][s][c]; one block per (query, segment), one thread per codeword
__global__ void __launch_bounds__(256) pq_tables_kernel(const float* __restrict__ q, int dim, int m, int ksub, int ds,
                                                        const float* __restrict__ cb, float* __restrict__ tables) {
  const int64_t a = blockIdx.x / m;
  const int s = (int)(blockIdx.x % m);
  const float* seg = q + a * dim + (int64_t)s * ds;
  for (int c = threadIdx.x; c < ksub; c += blockDim.x) {
    const float* cw = cb + ((int64_t)s * ksub + c) * ds;
    float sum = 0.f;
    for (int i = 0; i < ds; ++i) sum = sqdiff_accum(sum, __ldg(seg + i), __ldg(cw + i));
    tables[(a * m + s) * ksub + c] = sum;
  }
}

// One thread per (row, segment); the segment's codebook sits in shared memory (read as a broadcast), the row's
// segment in registers when its length is one of the usual ones.
template <int DS>
__global__ void __launch_bounds__(PQ_THREADS) pq_encode_kernel(const float* __restrict__ x, int64_t n, int dim, int m,
                                                              int ksub, int ds_rt, const float* __restrict__ cb,
                                                              uint8_t* __restrict__ codes) {
  extern __shared__ float cbs[];
  const int ds = DS > 0 ? DS : ds_rt;
  const int s = blockIdx.y;
  for (int i = threadIdx.x; i < ksub * ds; i += blockDim.x) cbs[i] = cb[(int64_t)s * ksub * ds + i];
  __syncthreads();
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const float* seg = x + r * dim + (int64_t)s * ds;
  float best = CUDART_INF_F;
  int bc = 0;
  if (DS > 0) {
    float v[DS > 0 ? DS : 1];
#pragma unroll
    for (int i = 0; i < DS; ++i) v[i] = __ldg(seg + i);
    for (int c = 0; c < ksub; ++c) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < DS; ++i) d = sqdiff_accum(d, v[i], cbs[c * DS + i]);
      if (d < best) { best = d; bc = c; }
    }
  } else {
    for (int c = 0; c < ksub; ++c) {
      float d = 0.f;
      for (int i = 0; i < ds; ++i) d = sqdiff_accum(d, __ldg(seg + i), cbs[c * ds + i]);
      if (d < best) { best = d; bc = c; }
    }
  }
  codes[r * m + s] = (uint8_t)bc;
}

__global__ void pq_decode_kernel(const uint8_t* __restrict__ codes, int64_t n, int dim, int m, int ksub, int ds,
                                 const float* __restrict__ cb, float* __restrict__ x) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * dim) return;
  const int64_t r = i / dim;
  const int j = (int)(i % dim);
  const int s = j / ds;
  x[i] = cb[((int64_t)s * ksub + codes[r * m + s]) * ds + (j - s * ds)];
}

__global__ void pq_gather_segment_kernel(const float* __restrict__ x, int64_t n, int dim, int s, int ds,
                                         float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * ds) return;
  out[i] = x[(i / ds) * dim + (int64_t)s * ds + (i % ds)];
}

struct PqScanArgs {
  const float* tables;     // [nq_all][m][ksub]
  const uint8_t* codes;    // [n][m]
  int32_t m, ksub;
  int64_t nq;              // list positions
  const int32_t* q_subset; // or null: position -> query whose table to use
  int64_t row_begin, row_end;
  int32_t rows_per_cta;    // rows one CTA walks (a multiple of PQ_THREADS)
  CandLists cand;
};

// grid.x = query tiles * row parts.  Shared memory holds the tables of the tile's TQ queries; a thread walks rows
// and reads its row's codes straight from global memory, four segments per 32-bit load when the row length
// allows (the 512 rows of a CTA's step are one contiguous block of m * 512 bytes).
template <int TQ, int MODE>
__global__ void __launch_bounds__(PQ_THREADS) pq_scan_kernel(PqScanArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* tab = reinterpret_cast<float*>(smem_raw);   // m * ksub * TQ floats (layout below)
  const int64_t parts = (a.row_end - a.row_begin + a.rows_per_cta - 1) / a.rows_per_cta;
  const int64_t qt = blockIdx.x / parts;
  const int64_t part = blockIdx.x % parts;
  const int64_t p0 = qt * TQ;
  const int entries = a.m * a.ksub;
  // tables of the tile; a missing query of the last tile reads as +inf (never appended)
  for (int t = 0; t < TQ; ++t) {
    const int64_t pos = p0 + t;
    const bool ok = pos < a.nq;
    const int64_t qi = ok ? (a.q_subset ? (int64_t)a.q_subset[pos] : pos) : 0;
    const float* src = a.tables + qi * entries;
    // TQ >= 4: [segment][group of 4 queries][code][4], so that the 32 lanes of one 16-byte load (one group, 32
    // different codes) spread over all banks; a [segment][code][query] layout would put them on 8 of the 32
    for (int e = threadIdx.x; e < entries; e += PQ_THREADS) {
      const float v = ok ? __ldg(src + e) : CUDART_INF_F;
      if (TQ % 4 == 0) {
        const int sseg = e / a.ksub, c = e - sseg * a.ksub;
        tab[(((size_t)sseg * (TQ / 4) + (t >> 2)) * a.ksub + c) * 4 + (t & 3)] = v;
      } else {
        tab[(size_t)e * TQ + t] = v;
      }
    }
  }
  float thr[TQ];
#pragma unroll
  for (int t = 0; t < TQ; ++t) thr[t] = (MODE == SCAN_THRESHOLD && p0 + t < a.nq) ? a.cand.thr[p0 + t] : -CUDART_INF_F;
  __syncthreads();
  const int64_t r_begin = a.row_begin + part * a.rows_per_cta;
  const int64_t r_end = min(a.row_end, r_begin + a.rows_per_cta);
  const bool words = (a.m & 3) == 0 && (reinterpret_cast<uintptr_t>(a.codes) & 3) == 0;
  const size_t group_stride = (size_t)a.ksub * 4;   // floats between the groups of 4 queries of one segment
  for (int64_t row = r_begin + threadIdx.x; row < r_end; row += PQ_THREADS) {
    float acc[TQ];
#pragma unroll
    for (int t = 0; t < TQ; ++t) acc[t] = 0.f;
    // adds one segment's table entries, in segment order (the reference's order of the sum)
    auto add_segment = [&](int s, int c) {
      if (TQ % 4 == 0) {
        const float* e = tab + ((size_t)s * (TQ / 4) * a.ksub + c) * 4;
#pragma unroll
        for (int t = 0; t < TQ; t += 4) {
          const float4 v = *reinterpret_cast<const float4*>(e + (size_t)(t >> 2) * group_stride);
          acc[t] = __fadd_rn(acc[t], v.x);
          acc[t + 1] = __fadd_rn(acc[t + 1], v.y);
          acc[t + 2] = __fadd_rn(acc[t + 2], v.z);
          acc[t + 3] = __fadd_rn(acc[t + 3], v.w);
        }
      } else {
        const float* e = tab + ((size_t)s * a.ksub + c) * TQ;
#pragma unroll
        for (int t = 0; t < TQ; ++t) acc[t] = __fadd_rn(acc[t], e[t]);
      }
    };
    if (words) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(a.codes + row * a.m);
      for (int s4 = 0; s4 < (a.m >> 2); ++s4) {
        const uint32_t w = __ldg(src + s4);
#pragma unroll
        for (int b = 0; b < 4; ++b) add_segment(s4 * 4 + b, (int)((w >> (8 * b)) & 0xffu));
      }
    } else {
      const uint8_t* src = a.codes + row * a.m;
      for (int s = 0; s < a.m; ++s) add_segment(s, (int)__ldg(src + s));
    }
#pragma unroll
    for (int t = 0; t < TQ; ++t) {
      const int64_t pos = p0 + t;
      if (pos >= a.nq) break;
      const float v = __fsqrt_rn(acc[t]);
      if (MODE == SCAN_DENSE) {
        a.cand.keys[pos * kCandCap + (row - a.row_begin)] = make_key(v, (uint32_t)row);
      } else if (v < thr[t]) {
        // strict: rows arrive in ascending order, so a later row that only ties the current k-th value has a
        // larger row number than every kept key and cannot displace one (quantised distances tie in bulk)
        const int slot = atomicAdd(&a.cand.count[pos], 1);
        if (slot < kCandCap) a.cand.keys[pos * kCandCap + slot] = make_key(v, (uint32_t)row);
      }
    }
  }
}

template <int TQ>
int32_t launch_scan_tq(Ctx* ctx, const PqScanArgs& a, int mode, size_t smem, unsigned grid) {
  auto kern = mode == SCAN_DENSE ? pq_scan_kernel<TQ, SCAN_DENSE> : pq_scan_kernel<TQ, SCAN_THRESHOLD>;
  VSK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  prof_begin(ctx);
  kern<<<grid, PQ_THREADS, smem, ctx->stream>>>(a);
  prof_end(ctx);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

// Queries per CTA: as many tables as fit next to the block of codes, a power of two, at most 16.
int pick_tq(int m, int ksub, int64_t nq) {
  const size_t per_query = (size_t)m * ksub * sizeof(float);
  int tq = 16;
  while (tq > 1 && (tq * per_query > PQ_SMEM_LIMIT || tq / 2 >= nq)) tq >>= 1;
  return tq;
}

int32_t launch_pq_scan(Ctx* ctx, PqScanArgs a, int mode) {
  const int64_t rows = a.row_end - a.row_begin;
  if (rows <= 0 || a.nq <= 0) return VSK_OK;
  const int tq = pick_tq(a.m, a.ksub, a.nq);
  const size_t smem = (size_t)tq * a.m * a.ksub * sizeof(float);
  if (smem > PQ_SMEM_LIMIT)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "one query's distance table (%d x %d floats) does not fit in shared memory", a.m, a.ksub);
  const int64_t qtiles = ceil_div(a.nq, tq);
  // enough row parts to fill the GPU a few times over, each at least 4 096 rows so the table load is amortised
  const int64_t want_ctas = (int64_t)ctx->prop.multiProcessorCount * 4;
  int64_t parts = std::max<int64_t>(1, std::min(ceil_div(want_ctas, qtiles), ceil_div(rows, 4096)));
  a.rows_per_cta = (int32_t)(ceil_div(ceil_div(rows, parts), PQ_THREADS) * PQ_THREADS);
  parts = ceil_div(rows, a.rows_per_cta);
  const int64_t grid = qtiles * parts;
  if (grid > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many tiles in one launch");
  switch (tq) {
    case 16: return launch_scan_tq<16>(ctx, a, mode, smem, (unsigned)grid);
    case 8: return launch_scan_tq<8>(ctx, a, mode, smem, (unsigned)grid);
    case 4: return launch_scan_tq<4>(ctx, a, mode, smem, (unsigned)grid);
    case 2: return launch_scan_tq<2>(ctx, a, mode, smem, (unsigned)grid);
    default: return launch_scan_tq<1>(ctx, a, mode, smem, (unsigned)grid);
  }
}

int32_t check_shape(Ctx* ctx, int32_t dim, int32_t m, int32_t ksub) {
  // ProductQuantizationConfig.validate (Config/Quantization/ProductQuantizationConfig.swift:42-49); a code is one
  // byte (QuantizedVector.codes is [UInt8]), so at most 256 codewords per segment
  if (dim <= 0 || m <= 0 || dim % m != 0)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "invalid segmentation: %d dimensions into %d segments", dim, m);
  if (ksub < 2 || ksub > 256) return fail(ctx, VSK_ERR_INVALID_INPUT, "codebook size %d is outside [2, 256]", ksub);
  return VSK_OK;
}

int32_t encode_dev(Ctx* ctx, const float* cb, int32_t dim, int32_t m, int32_t ksub, const float* x, int64_t n,
                   uint8_t* codes) {
  const int ds = dim / m;
  const size_t smem = (size_t)ksub * ds * sizeof(float);
  if (smem > PQ_SMEM_LIMIT) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "a segment's codebook (%d x %d floats) does not fit in shared memory", ksub, ds);
  const dim3 grid((unsigned)ceil_div(n, PQ_THREADS), (unsigned)m);
#define VSK_PQ_ENC(DS_)                                                                                          \
  do {                                                                                                           \
    VSK_CUDA(ctx, cudaFuncSetAttribute(pq_encode_kernel<DS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    pq_encode_kernel<DS_><<<grid, PQ_THREADS, smem, ctx->stream>>>(x, n, dim, m, ksub, ds, cb, codes);            \
  } while (0)
  switch (ds) {
    case 1: VSK_PQ_ENC(1); break;
    case 2: VSK_PQ_ENC(2); break;
    case 4: VSK_PQ_ENC(4); break;
    case 8: VSK_PQ_ENC(8); break;
    case 16: VSK_PQ_ENC(16); break;
    case 32: VSK_PQ_ENC(32); break;
    default: VSK_PQ_ENC(0); break;
  }
#undef VSK_PQ_ENC
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

int32_t tables_dev(Ctx* ctx, const float* cb, int32_t dim, int32_t m, int32_t ksub, const float* q, int64_t nq,
                   float* tables) {
  if (nq * m > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many (query, segment) pairs");
  pq_tables_kernel<<<(unsigned)(nq * m), 256, 0, ctx->stream>>>(q, dim, m, ksub, dim / m, cb, tables);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

// Temporary device copies of host arrays for the blocking host-pointer entry points.
struct Tmp {
  std::vector<void*> bufs;
  ~Tmp() { for (void* p : bufs) dev_free(p); }
  int32_t get(Ctx* ctx, size_t bytes, void** out) {
    VSK_TRY(dev_alloc(ctx, out, std::max<size_t>(bytes, 16)));
    bufs.push_back(*out);
    return VSK_OK;
  }
  int32_t up(Ctx* ctx, const void* host, size_t bytes, void** out) {
    VSK_TRY(get(ctx, bytes, out));
    VSK_CUDA(ctx, cudaMemcpyAsync(*out, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    ctx->stats.h2d_bytes += (int64_t)bytes;
    return VSK_OK;
  }
};

int32_t train_dev(Ctx* ctx, const float* x, int64_t n, int32_t dim, int32_t m, int32_t ksub, int32_t iters,
                  const float* init, float* cb) {
  VSK_TRY(check_shape(ctx, dim, m, ksub));
  // ProductQuantizer.train (:34-41) asks for codebookSize * segments vectors
  if (n < (int64_t)ksub * m)
    return fail(ctx, VSK_ERR_INSUFFICIENT_TRAINING_DATA, "provided %lld, required %lld", (long long)n, (long long)ksub * m);
  if (!x || !cb) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  const int ds = dim / m;
  Tmp tmp;
  void *seg, *asg, *first;
  VSK_TRY(tmp.get(ctx, (size_t)n * ds * 4, &seg));
  VSK_TRY(tmp.get(ctx, (size_t)n * 4, &asg));
  VSK_TRY(tmp.get(ctx, (size_t)ksub * ds * 4, &first));
  for (int s = 0; s < m; ++s) {
    pq_gather_segment_kernel<<<(unsigned)ceil_div(n * ds, 256), 256, 0, ctx->stream>>>(x, n, dim, s, ds, (float*)seg);
    ctx->stats.kernel_launches++;
    const float* init_s = init ? init + (int64_t)s * ksub * ds : (const float*)first;
    if (!init)   // default initial codewords: the segment of the first ksub rows
      VSK_CUDA(ctx, cudaMemcpyAsync(first, seg, (size_t)ksub * ds * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    float inertia = 0.f;
    int32_t run = 0;
    VSK_TRY(kmeans_dev(ctx, (const float*)seg, n, ds, ksub, iters, -1.0f, init_s, cb + (int64_t)s * ksub * ds,
                       (int32_t*)asg, &inertia, &run));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace

int32_t pq_reserve(Index* ix, int64_t need) {
  Ctx* ctx = ix->ctx;
  if (need <= ix->capacity) return VSK_OK;
  const int64_t cap = std::max<int64_t>(need, ix->capacity + ix->capacity / 2);
  uint8_t* codes = nullptr;
  VSK_TRY(dev_alloc(ctx, (void**)&codes, (size_t)cap * ix->pq_m));
  if (ix->n > 0) {
    VSK_CUDA(ctx, cudaMemcpyAsync(codes, ix->pq_codes, (size_t)ix->n * ix->pq_m, cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  dev_free(ix->pq_codes);
  ix->pq_codes = codes;
  ix->capacity = cap;
  return VSK_OK;
}

// A code must name a codeword of its segment's codebook before a scan indexes a table with it.
__global__ void pq_check_codes_kernel(const uint8_t* __restrict__ codes, int64_t total, int ksub, int32_t* bad) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total && codes[i] >= ksub) *bad = 1;
}

static int32_t pq_check_codes(Index* ix, int64_t first, int64_t n) {
  Ctx* ctx = ix->ctx;
  if (ix->pq_ksub >= 256) return VSK_OK;   // every byte is a valid code
  int32_t* flag = nullptr;
  VSK_TRY(dev_alloc(ctx, (void**)&flag, 4));
  cudaMemsetAsync(flag, 0, 4, ctx->stream);
  const int64_t total = n * ix->pq_m;
  pq_check_codes_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, ctx->stream>>>(ix->pq_codes + first * ix->pq_m, total, ix->pq_ksub, flag);
  ctx->stats.kernel_launches++;
  int32_t h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, flag, 4, cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  dev_free(flag);
  if (e != cudaSuccess) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "%s", cudaGetErrorString(e));
  if (h) return fail(ctx, VSK_ERR_INVALID_INPUT, "a code is outside the codebook (size %d)", ix->pq_ksub);
  return VSK_OK;
}

// Codes were written straight into the reserved storage (an index image being loaded).
int32_t pq_adopt_rows(Index* ix, int64_t n) {
  if (n > ix->capacity) return fail(ix->ctx, VSK_ERR_INVALID_BUFFER_SIZE, "more rows than reserved");
  VSK_TRY(pq_check_codes(ix, 0, n));
  ix->n = n;
  return VSK_OK;
}

int32_t pq_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  ctx->stats.searches++;
  ctx->stats.queries += nq;
  const int m = ix->pq_m, ksub = ix->pq_ksub;
  constexpr int64_t kBatch = 16384;
  for (int64_t b = 0; b < nq; b += kBatch) {
    const int64_t bn = std::min(kBatch, nq - b);
    void* tables;
    VSK_TRY(scratch(ctx, SLOT_PQ_TABLES, (size_t)bn * m * ksub * sizeof(float), &tables));
    VSK_TRY(tables_dev(ctx, ix->pq_codebooks, ix->dim, m, ksub, q + b * ix->dim, bn, (float*)tables));
    const ScanBinder bind = [=](const CandLists& cand, int64_t pn, const int32_t* sub) -> ScanFn {
      PqScanArgs a{};
      a.tables = (const float*)tables;
      a.codes = ix->pq_codes;
      a.m = m;
      a.ksub = ksub;
      a.nq = pn;
      a.q_subset = sub;
      a.cand = cand;
      return [ctx, a](int mode, int64_t rb, int64_t re) mutable {
        a.row_begin = rb;
        a.row_end = re;
        return launch_pq_scan(ctx, a, mode);
      };
    };
    VSK_TRY(scan_topk(ctx, bind, ix->n, bn, nullptr, k, ix->id_base, 0, out_dist + b * k, out_ids + b * k, 0));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_pq_train(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t segments, int32_t codebook_size,
                     int32_t iterations, const float* init_codebooks, float* codebooks) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (n <= 0 || !rows || !codebooks) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no training rows");
  Tmp tmp;
  void *dx, *dinit = nullptr, *dcb;
  const size_t cb_bytes = (size_t)codebook_size * dim * 4;   // m * ksub * ds floats
  VSK_TRY(tmp.up(ctx, rows, (size_t)n * dim * 4, &dx));
  if (init_codebooks) VSK_TRY(tmp.up(ctx, init_codebooks, cb_bytes, &dinit));
  VSK_TRY(tmp.get(ctx, cb_bytes, &dcb));
  VSK_TRY(train_dev(ctx, (const float*)dx, n, dim, segments, codebook_size, iterations, (const float*)dinit, (float*)dcb));
  VSK_CUDA(ctx, cudaMemcpy(codebooks, dcb, cb_bytes, cudaMemcpyDeviceToHost));
  ctx->stats.d2h_bytes += (int64_t)cb_bytes;
  return VSK_OK;
}

int32_t vsk_pq_train_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t segments, int32_t codebook_size,
                         int32_t iterations, const float* init_codebooks, float* codebooks) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  return train_dev(ctx, rows, n, dim, segments, codebook_size, iterations, init_codebooks, codebooks);
}

int32_t vsk_pq_encode_dev(vsk_ctx* c, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                          const float* rows, int64_t n, uint8_t* codes) {
  VSK_TRACE("vsk_pq_encode_dev");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (!codebooks || !rows || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  VSK_TRY(encode_dev(ctx, codebooks, dim, segments, codebook_size, rows, n, codes));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_pq_encode(vsk_ctx* c, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                      const float* rows, int64_t n, uint8_t* codes) {
  VSK_TRACE("vsk_pq_encode");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (!codebooks || !rows || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  Tmp tmp;
  void *dcb, *dx, *dc;
  VSK_TRY(tmp.up(ctx, codebooks, (size_t)codebook_size * dim * 4, &dcb));
  VSK_TRY(tmp.up(ctx, rows, (size_t)n * dim * 4, &dx));
  VSK_TRY(tmp.get(ctx, (size_t)n * segments, &dc));
  VSK_TRY(encode_dev(ctx, (const float*)dcb, dim, segments, codebook_size, (const float*)dx, n, (uint8_t*)dc));
  VSK_CUDA(ctx, cudaMemcpyAsync(codes, dc, (size_t)n * segments, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.d2h_bytes += n * segments;
  return VSK_OK;
}

int32_t vsk_pq_decode(vsk_ctx* c, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                      const uint8_t* codes, int64_t n, float* rows) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no codes");
  if (!codebooks || !rows || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  // a code must name a codeword: checked on the host before anything indexes the codebook with it
  for (int64_t i = 0; i < n * segments; ++i)
    if (codes[i] >= codebook_size) return fail(ctx, VSK_ERR_INVALID_INPUT, "code %d at %lld is outside the codebook", (int)codes[i], (long long)i);
  Tmp tmp;
  void *dcb, *dc, *dx;
  VSK_TRY(tmp.up(ctx, codebooks, (size_t)codebook_size * dim * 4, &dcb));
  VSK_TRY(tmp.up(ctx, codes, (size_t)n * segments, &dc));
  VSK_TRY(tmp.get(ctx, (size_t)n * dim * 4, &dx));
  pq_decode_kernel<<<(unsigned)ceil_div(n * dim, 256), 256, 0, ctx->stream>>>((const uint8_t*)dc, n, dim, segments, codebook_size,
                                                                             dim / segments, (const float*)dcb, (float*)dx);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaMemcpyAsync(rows, dx, (size_t)n * dim * 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.d2h_bytes += n * dim * 4;
  return VSK_OK;
}

int32_t vsk_pq_distance_tables(vsk_ctx* c, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                               const float* queries, int64_t nq, float* tables) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (nq <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no queries");
  if (!codebooks || !queries || !tables) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  Tmp tmp;
  void *dcb, *dq, *dt;
  const size_t tb = (size_t)nq * segments * codebook_size * 4;
  VSK_TRY(tmp.up(ctx, codebooks, (size_t)codebook_size * dim * 4, &dcb));
  VSK_TRY(tmp.up(ctx, queries, (size_t)nq * dim * 4, &dq));
  VSK_TRY(tmp.get(ctx, tb, &dt));
  VSK_TRY(tables_dev(ctx, (const float*)dcb, dim, segments, codebook_size, (const float*)dq, nq, (float*)dt));
  VSK_CUDA(ctx, cudaMemcpyAsync(tables, dt, tb, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.d2h_bytes += (int64_t)tb;
  return VSK_OK;
}

int32_t vsk_pq_index_create(vsk_ctx* c, int32_t dim, int32_t segments, int32_t codebook_size, const float* codebooks,
                            vsk_index** out) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  *out = nullptr;
  VSK_TRY(check_shape(ctx, dim, segments, codebook_size));
  if (!codebooks) return fail(ctx, VSK_ERR_NOT_TRAINED, "no codebooks: train the quantiser first");
  if ((size_t)segments * codebook_size * sizeof(float) > PQ_SMEM_LIMIT)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "one query's distance table (%d x %d floats) does not fit in shared memory", segments, codebook_size);
  Index* ix = new Index();
  ix->ctx = ctx;
  ix->kind = INDEX_PQ;
  ix->metric = VSK_METRIC_EUCLIDEAN;
  ix->dim = dim;
  ix->pq_m = segments;
  ix->pq_ksub = codebook_size;
  const size_t cb_bytes = (size_t)codebook_size * dim * 4;
  int32_t st = dev_alloc(ctx, (void**)&ix->pq_codebooks, cb_bytes);
  // on the context's stream, which the kernels that read the codebooks run on (it does not wait for the legacy stream)
  if (st == VSK_OK && (cudaMemcpyAsync(ix->pq_codebooks, codebooks, cb_bytes, cudaMemcpyDefault, ctx->stream) != cudaSuccess ||
                       cudaStreamSynchronize(ctx->stream) != cudaSuccess))
    st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "copy of the codebooks failed");
  if (st != VSK_OK) {
    vsk_index_destroy(reinterpret_cast<vsk_index*>(ix));
    return st;
  }
  *out = reinterpret_cast<vsk_index*>(ix);
  return VSK_OK;
}

static int32_t pq_add(vsk_index* i, const uint8_t* codes, int64_t n, bool on_device) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (ix->kind != INDEX_PQ) return fail(ctx, VSK_ERR_INVALID_INPUT, "not a product-quantised index");
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows to add");
  if (!codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null codes");
  if (ix->n + n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "an index holds at most 2^31-1 rows");
  VSK_TRY(pq_reserve(ix, ix->n + n));
  VSK_CUDA(ctx, cudaMemcpyAsync(ix->pq_codes + ix->n * ix->pq_m, codes, (size_t)n * ix->pq_m,
                                on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
  if (!on_device) ctx->stats.h2d_bytes += n * ix->pq_m;
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  VSK_TRY(pq_check_codes(ix, ix->n, n));   // rejected rows are not counted in
  ix->n += n;
  return VSK_OK;
}

int32_t vsk_pq_index_add(vsk_index* i, const uint8_t* codes, int64_t n) { return pq_add(i, codes, n, false); }
int32_t vsk_pq_index_add_dev(vsk_index* i, const uint8_t* codes, int64_t n) { return pq_add(i, codes, n, true); }

}  // extern "C"
