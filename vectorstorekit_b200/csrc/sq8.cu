// Scalar int8 quantiser and the scan over its codes.
// Replaces ScalarQuantizer.quantizeBatch / dequantize for `.int8`
// (Quantization/ScalarQuantizer.swift:129-164,251-270,389-451,568-580):
//   parameters  scale = 255/(max-min), offset = -min*scale - 128            (:428-431)
//   encode      code = truncate_toward_zero(x*scale + offset)               (:258-267, vsmsa + vfix8)
//   decode      x^ = (code - offset)/scale                                  (:576-578)
// Every operation is rounded separately (no fused multiply-add), so codes and decoded values are
// bit-identical to a plain fp32 evaluation of those formulas.
// The reference has no search over codes; the scan here is the chosen metric between the fp32
// query and the dequantised row, computed by the fp32 tile with rows dequantised while staging.
#include <math_constants.h>

#include "common.cuh"
#include "tensor_scan.cuh"

namespace vsk {
namespace {

// per-dimension min/max: thread = dimension (coalesced), block = a slab of rows
__global__ void minmax_kernel(const float* __restrict__ x, int64_t n, int dim, int64_t rows_per_block,
                              unsigned* __restrict__ omin, unsigned* __restrict__ omax) {
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_block, r1 = min(n, r0 + rows_per_block);
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  float mn = CUDART_INF_F, mx = -CUDART_INF_F;
  for (int64_t r = r0; r < r1; ++r) {
    const float v = __ldg(x + r * dim + d);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  atomicMin(omin + d, float_to_ordered(mn));
  atomicMax(omax + d, float_to_ordered(mx));
}
__global__ void minmax_init_kernel(unsigned* omin, unsigned* omax, int dim) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d < dim) {
    omin[d] = float_to_ordered(CUDART_INF_F);
    omax[d] = float_to_ordered(-CUDART_INF_F);
  }
}
__global__ void minmax_decode_kernel(const unsigned* omin, const unsigned* omax, int dim, float* minv, float* maxv) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d < dim) {
    minv[d] = ordered_to_float(omin[d]);
    maxv[d] = ordered_to_float(omax[d]);
  }
}

// single block: optional reduction over dimensions (global mode), then the parameter formulas
__global__ void sq8_params_kernel(const float* minv, const float* maxv, int dim, int global_mode, float* scale,
                                  float* offset) {
  __shared__ float smin[256], smax[256];
  float mn = CUDART_INF_F, mx = -CUDART_INF_F;
  if (global_mode) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
      mn = fminf(mn, minv[d]);
      mx = fmaxf(mx, maxv[d]);
    }
    smin[threadIdx.x] = mn;
    smax[threadIdx.x] = mx;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if (threadIdx.x < o) {
        smin[threadIdx.x] = fminf(smin[threadIdx.x], smin[threadIdx.x + o]);
        smax[threadIdx.x] = fmaxf(smax[threadIdx.x], smax[threadIdx.x + o]);
      }
      __syncthreads();
    }
  }
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float lo = global_mode ? smin[0] : minv[d];
    const float hi = global_mode ? smax[0] : maxv[d];
    const float range = __fsub_rn(hi, lo);
    const float s = __fdiv_rn(255.0f, range);
    scale[d] = s;
    offset[d] = __fsub_rn(__fmul_rn(-lo, s), 128.0f);
  }
}

__global__ void sq8_encode_kernel(const float* __restrict__ x, int64_t total, int dim, const float* __restrict__ scale,
                                  const float* __restrict__ offset, int8_t* __restrict__ codes) {
  // 4 elements per thread when the row length allows aligned 16-byte loads
  const int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= total) return;
  // (a caller's view may start at any 4-byte offset: the wide path also needs both pointers aligned)
  const bool wide = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(codes) & 3) == 0;
  if (wide && i4 + 3 < total) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(x + i4));
    const int d = (int)(i4 % dim);
    const float in[4] = {v.x, v.y, v.z, v.w};
    char4 c;
    int8_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float t = __fadd_rn(__fmul_rn(in[j], __ldg(scale + d + j)), __ldg(offset + d + j));
      int q = __float2int_rz(t);
      q = max(-128, min(127, q));
      o[j] = (int8_t)q;
    }
    c.x = o[0]; c.y = o[1]; c.z = o[2]; c.w = o[3];
    *reinterpret_cast<char4*>(codes + i4) = c;
  } else {
    for (int64_t i = i4; i < min(total, i4 + 4); ++i) {
      const int d = (int)(i % dim);
      const float t = __fadd_rn(__fmul_rn(__ldg(x + i), __ldg(scale + d)), __ldg(offset + d));
      int q = __float2int_rz(t);
      codes[i] = (int8_t)max(-128, min(127, q));
    }
  }
}

__global__ void sq8_decode_kernel(const int8_t* __restrict__ codes, int64_t total, int dim,
                                  const float* __restrict__ scale, const float* __restrict__ offset,
                                  float* __restrict__ x) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int d = (int)(i % dim);
  x[i] = __fdiv_rn(__fsub_rn((float)codes[i], __ldg(offset + d)), __ldg(scale + d));
}

// |x^| of dequantised rows (cosine): one warp per row
__global__ void sq8_row_norm_kernel(const int8_t* __restrict__ codes, int64_t n, int dim,
                                    const float* __restrict__ scale, const float* __restrict__ offset,
                                    float* __restrict__ out) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = __fdiv_rn(__fsub_rn((float)codes[row * dim + i], __ldg(offset + i)), __ldg(scale + i));
    s = fmaf(v, v, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[row] = sqrtf(s);
}

int32_t check_ctx(vsk_ctx* c, Ctx** ctx) {
  *ctx = reinterpret_cast<Ctx*>(c);
  if (!*ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice((*ctx)->device);
  return VSK_OK;
}

}  // namespace

int32_t sq8_reserve(Index* ix, int64_t need) {
  Ctx* ctx = ix->ctx;
  if (need <= ix->capacity) return VSK_OK;
  const int64_t cap = std::max<int64_t>(need, ix->capacity + ix->capacity / 2);
  int8_t* codes = nullptr;
  float* norm = nullptr;
  VSK_TRY(dev_alloc(ctx, (void**)&codes, (size_t)cap * ix->dim));
  VSK_TRY(dev_alloc(ctx, (void**)&norm, (size_t)cap * 4));
  if (ix->n > 0) {
    VSK_CUDA(ctx, cudaMemcpyAsync(codes, ix->codes, (size_t)ix->n * ix->dim, cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(norm, ix->row_norm, (size_t)ix->n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  }
  dev_free(ix->codes);
  dev_free(ix->row_norm);
  ix->codes = codes;
  ix->row_norm = norm;
  ix->capacity = cap;
  return VSK_OK;
}

// Codes were written straight into the reserved storage (an index image being loaded): compute what an add
// computes and count them in.
int32_t sq8_adopt_rows(Index* ix, int64_t n) {
  Ctx* ctx = ix->ctx;
  if (n > ix->capacity) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "more rows than reserved");
  if (ix->metric == VSK_METRIC_COSINE) {
    sq8_row_norm_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(ix->codes, n, ix->dim, ix->sq_scale,
                                                                           ix->sq_offset, ix->row_norm);
    ctx->stats.kernel_launches++;
  }
  ix->n = n;
  tensor_invalidate(ix);
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

namespace {

int32_t sq8_add(Index* ix, const int8_t* codes, int64_t n, bool on_device) {
  Ctx* ctx = ix->ctx;
  if (ix->kind != INDEX_FLAT_I8) return fail(ctx, VSK_ERR_INVALID_INPUT, "not an int8 index");
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows to add");
  if (!codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null codes");
  if (ix->n + n > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "an index holds at most 2^31-1 rows");
  VSK_TRY(sq8_reserve(ix, ix->n + n));
  VSK_CUDA(ctx, cudaMemcpyAsync(ix->codes + ix->n * ix->dim, codes, (size_t)n * ix->dim,
                                on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
  if (!on_device) ctx->stats.h2d_bytes += n * ix->dim;
  if (ix->metric == VSK_METRIC_COSINE) {
    sq8_row_norm_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(ix->codes + ix->n * ix->dim, n, ix->dim,
                                                                           ix->sq_scale, ix->sq_offset, ix->row_norm + ix->n);
    ctx->stats.kernel_launches++;
  }
  ix->n += n;
  tensor_invalidate(ix);
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace

int32_t sq8_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  ctx->stats.searches++;
  ctx->stats.queries += nq;
  constexpr int64_t kBatch = 16384;
  const bool tensor = ctx->search_path == VSK_PATH_TENSOR_RERANK &&
                      (ix->metric == VSK_METRIC_DOT_PRODUCT || ix->metric == VSK_METRIC_EUCLIDEAN);
  for (int64_t b = 0; b < nq; b += kBatch) {
    const int64_t bn = std::min(kBatch, nq - b);
    if (tensor) {
      VSK_TRY(tensor_search(ix, q + b * ix->dim, bn, k, nullptr, nullptr, out_dist + b * k, out_ids + b * k));
      continue;
    }
    ExactScanArgs a{};
    a.metric = ix->metric;
    a.q = q + b * ix->dim;
    a.x_codes = ix->codes;
    a.sq_scale = ix->sq_scale;
    a.sq_offset = ix->sq_offset;
    a.dim = ix->dim;
    a.xnorm = ix->row_norm;
    if (ix->metric == VSK_METRIC_COSINE) {
      void* p;
      VSK_TRY(scratch(ctx, SLOT_QNORM, bn * 4, &p));
      VSK_TRY(launch_row_norms(ctx, a.q, bn, ix->dim, 0, (float*)p));
      a.qnorm = (float*)p;
    }
    VSK_TRY(fp32_topk(ctx, a, ix->n, bn, nullptr, k, ix->id_base, out_dist + b * k, out_ids + b * k, 0));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_sq8_minmax_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, float* minv, float* maxv) {
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !minv || !maxv) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  void* p;
  VSK_TRY(scratch(ctx, SLOT_SQ_A, (size_t)dim * 8, &p));
  unsigned* omin = (unsigned*)p;
  unsigned* omax = omin + dim;
  const unsigned bx = (unsigned)ceil_div(dim, 128);
  minmax_init_kernel<<<bx, 128, 0, ctx->stream>>>(omin, omax, dim);
  const int64_t rpb = std::max<int64_t>(64, ceil_div(n, 4096));
  dim3 grid(bx, (unsigned)ceil_div(n, rpb));
  minmax_kernel<<<grid, 128, 0, ctx->stream>>>(rows, n, dim, rpb, omin, omax);
  minmax_decode_kernel<<<bx, 128, 0, ctx->stream>>>(omin, omax, dim, minv, maxv);
  ctx->stats.kernel_launches += 3;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_sq8_params_dev(vsk_ctx* c, const float* minv, const float* maxv, int32_t dim, int32_t mode, float* scale,
                           float* offset) {
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (mode != VSK_SQ8_GLOBAL && mode != VSK_SQ8_PER_DIM) return fail(ctx, VSK_ERR_INVALID_INPUT, "unknown mode");
  if (!minv || !maxv || !scale || !offset) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  sq8_params_kernel<<<1, 256, 0, ctx->stream>>>(minv, maxv, dim, mode == VSK_SQ8_GLOBAL, scale, offset);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

int32_t vsk_sq8_encode_dev(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, const float* scale,
                           const float* offset, int8_t* codes) {
  VSK_TRACE("vsk_sq8_encode_dev");
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !scale || !offset || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  const int64_t total = n * dim;
  sq8_encode_kernel<<<(unsigned)ceil_div(ceil_div(total, 4), 256), 256, 0, ctx->stream>>>(rows, total, dim, scale, offset, codes);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VSK_OK;
}

static int32_t sq8_host_call(Ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t mode, float* scale,
                             float* offset, bool train, int8_t* codes_out, const int8_t* codes_in, float* rows_out) {
  // one helper for the three host-pointer entry points: stage in, run the device call, stage out.  The copies in go
  // through the context's stream, like the kernels that read them: that stream does not wait for the legacy default
  // stream, and a plain cudaMemcpy from pageable memory may return before its last bytes have landed.
  float *dx = nullptr, *dscale = nullptr, *doffset = nullptr, *dmm = nullptr;
  int8_t* dcodes = nullptr;
  int32_t st = VSK_OK;
  const size_t elems = (size_t)n * dim;
  vsk_ctx* c = reinterpret_cast<vsk_ctx*>(ctx);
  if ((st = dev_alloc(ctx, (void**)&dx, elems * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dscale, (size_t)dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&doffset, (size_t)dim * 4)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dmm, (size_t)dim * 8)) == VSK_OK &&
      (st = dev_alloc(ctx, (void**)&dcodes, elems)) == VSK_OK) {
    if (train) {
      cudaMemcpyAsync(dx, rows, elems * 4, cudaMemcpyHostToDevice, ctx->stream);
      st = vsk_sq8_minmax_dev(c, dx, n, dim, dmm, dmm + dim);
      if (st == VSK_OK) st = vsk_sq8_params_dev(c, dmm, dmm + dim, dim, mode, dscale, doffset);
      if (st == VSK_OK) {
        cudaMemcpy(scale, dscale, (size_t)dim * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(offset, doffset, (size_t)dim * 4, cudaMemcpyDeviceToHost);
      }
    } else {
      cudaMemcpyAsync(dscale, scale, (size_t)dim * 4, cudaMemcpyHostToDevice, ctx->stream);
      cudaMemcpyAsync(doffset, offset, (size_t)dim * 4, cudaMemcpyHostToDevice, ctx->stream);
      if (codes_out) {
        cudaMemcpyAsync(dx, rows, elems * 4, cudaMemcpyHostToDevice, ctx->stream);
        st = vsk_sq8_encode_dev(c, dx, n, dim, dscale, doffset, dcodes);
        if (st == VSK_OK) cudaMemcpy(codes_out, dcodes, elems, cudaMemcpyDeviceToHost);
      } else {
        cudaMemcpyAsync(dcodes, codes_in, elems, cudaMemcpyHostToDevice, ctx->stream);
        sq8_decode_kernel<<<(unsigned)ceil_div((int64_t)elems, 256), 256, 0, ctx->stream>>>(dcodes, (int64_t)elems, dim, dscale, doffset, dx);
        ctx->stats.kernel_launches++;
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "decode failed: %s", cudaGetErrorString(e));
        else cudaMemcpy(rows_out, dx, elems * 4, cudaMemcpyDeviceToHost);
      }
    }
    cudaError_t e = cudaGetLastError();
    if (st == VSK_OK && e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "%s", cudaGetErrorString(e));
  }
  dev_free(dx); dev_free(dscale); dev_free(doffset); dev_free(dmm); dev_free(dcodes);
  return st;
}

int32_t vsk_sq8_train(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, int32_t mode, float* scale, float* offset) {
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !scale || !offset) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  return sq8_host_call(ctx, rows, n, dim, mode, scale, offset, true, nullptr, nullptr, nullptr);
}

int32_t vsk_sq8_encode(vsk_ctx* c, const float* rows, int64_t n, int32_t dim, const float* scale, const float* offset,
                       int8_t* codes) {
  VSK_TRACE("vsk_sq8_encode");
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !scale || !offset || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  return sq8_host_call(ctx, rows, n, dim, 0, const_cast<float*>(scale), const_cast<float*>(offset), false, codes, nullptr, nullptr);
}

int32_t vsk_sq8_decode(vsk_ctx* c, const int8_t* codes, int64_t n, int32_t dim, const float* scale, const float* offset,
                       float* rows) {
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no rows");
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!rows || !scale || !offset || !codes) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  return sq8_host_call(ctx, nullptr, n, dim, 0, const_cast<float*>(scale), const_cast<float*>(offset), false, nullptr, codes, rows);
}

int32_t vsk_sq8_index_create(vsk_ctx* c, int32_t metric, int32_t dim, const float* scale, const float* offset,
                             vsk_index** out) {
  Ctx* ctx;
  VSK_TRY(check_ctx(c, &ctx));
  if (!out) return VSK_ERR_INVALID_INPUT;
  *out = nullptr;
  if (metric < VSK_METRIC_EUCLIDEAN || metric > VSK_METRIC_MANHATTAN)
    return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "metric %d is not supported", metric);
  if (dim <= 0) return fail(ctx, VSK_ERR_DIMENSION_MISMATCH, "dimension must be positive");
  if (!scale || !offset) return fail(ctx, VSK_ERR_INVALID_INPUT, "null scale/offset");
  Index* ix = new Index();
  ix->ctx = ctx;
  ix->kind = INDEX_FLAT_I8;
  ix->metric = metric;
  ix->dim = dim;
  int32_t st;
  if ((st = dev_alloc(ctx, (void**)&ix->sq_scale, (size_t)dim * 4)) != VSK_OK ||
      (st = dev_alloc(ctx, (void**)&ix->sq_offset, (size_t)dim * 4)) != VSK_OK) {
    vsk_index_destroy(reinterpret_cast<vsk_index*>(ix));
    return st;
  }
  // scale/offset are host arrays (a few hundred floats the host computed or received)
  cudaMemcpyAsync(ix->sq_scale, scale, (size_t)dim * 4, cudaMemcpyDefault, ctx->stream);
  cudaMemcpyAsync(ix->sq_offset, offset, (size_t)dim * 4, cudaMemcpyDefault, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  *out = reinterpret_cast<vsk_index*>(ix);
  return VSK_OK;
}

int32_t vsk_sq8_index_add(vsk_index* i, const int8_t* codes, int64_t n) {
  VSK_TRACE("vsk_sq8_index_add");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  return sq8_add(ix, codes, n, false);
}

int32_t vsk_sq8_index_add_dev(vsk_index* i, const int8_t* codes, int64_t n) {
  VSK_TRACE("vsk_sq8_index_add_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  return sq8_add(ix, codes, n, true);
}

}  // extern "C"
