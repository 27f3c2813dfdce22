// Measured ceilings for the scans that are bound by neither HBM nor the tensor cores.
//
//   VSK_PEAK_FP32_ISSUE   FP32-pipe instructions per second (lane-instructions: one per thread and instruction): the
//                         bound of the Manhattan scan, whose inner step is a subtract and an add-with-|.| per
//                         (pair, dimension).  Kernel: long chains of independent FADD / FFMA per thread.
//   VSK_PEAK_SMEM_GATHER  4-byte words per second fetched from shared memory at RANDOM addresses (bank conflicts
//                         included): the bound of the product-quantised scan, one table word per (query, row, segment).
//   VSK_PEAK_TMEM_READ    bytes per second read out of tensor memory into registers (tcgen05.ld): the bound of a
//                         contraction with a short inner dimension, whose every accumulator is looked at once
//                         (k-means assignment and the inverted-list scan at d = 128: 4 bytes per (row, centroid) pair).
//
// Both run for a few milliseconds on the context's stream, are timed with CUDA events there, and report the best of
// five runs.  The reference has no such measurement; its nearest relative is the thread-configuration benchmark
// (Acceleration/Metal/MetalThreadConfigurationOptimizer.swift:430-440).
#include <algorithm>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace vsk {
namespace {

constexpr int kFpChains = 8;

__global__ void __launch_bounds__(256) fp32_issue_kernel(float* out, int iters, float seed) {
  float a[kFpChains];
#pragma unroll
  for (int i = 0; i < kFpChains; ++i) a[i] = seed + (float)(threadIdx.x + i);
  const float b = 1.0000001f, c = 1e-7f;
#pragma unroll 4
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < kFpChains; ++i) {
      a[i] = fmaf(a[i], b, c);          // FFMA
      a[i] = fabsf(a[i] - c) + b;       // FADD with |.| on its operand, FADD
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kFpChains; ++i) s += a[i];
  if (s == 123.456f) out[0] = s;   // keeps the chains alive
}

constexpr int kGatherWords = 8192;   // 32 KB table

__global__ void __launch_bounds__(256) smem_gather_kernel(float* out, int iters) {
  __shared__ float table[kGatherWords];
  for (int i = threadIdx.x; i < kGatherWords; i += blockDim.x) table[i] = (float)i * 1e-3f;
  __syncthreads();
  // four independent index streams per thread (a multiplicative generator each), four loads in flight
  uint32_t x0 = 2654435761u * (threadIdx.x + 1 + blockIdx.x * 977u), x1 = x0 * 40503u + 1u, x2 = x1 * 40503u + 7u,
           x3 = x2 * 40503u + 13u;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int it = 0; it < iters; ++it) {
    s0 += table[(x0 >> 12) & (kGatherWords - 1)];
    s1 += table[(x1 >> 12) & (kGatherWords - 1)];
    s2 += table[(x2 >> 12) & (kGatherWords - 1)];
    s3 += table[(x3 >> 12) & (kGatherWords - 1)];
    x0 = x0 * 1664525u + 1013904223u;
    x1 = x1 * 1664525u + 1013904223u;
    x2 = x2 * 1664525u + 1013904223u;
    x3 = x3 * 1664525u + 1013904223u;
  }
  const float s = s0 + s1 + s2 + s3;
  if (s == 123.456f) out[0] = s;
}

// Tensor-memory read-out: 16 warps (the epilogue of the short-contraction kernels: four lane quarters x four column
// parts of 64) read two 32-column groups per step with tcgen05.ld, over and over, from an allocation nobody wrote.
// Counts bytes delivered to registers.  No MMA, no barrier, no copy: the kernel allocates, reads, frees.
__global__ void __launch_bounds__(512, 1) tmem_read_kernel(float* out, int iters) {
  __shared__ uint32_t s_base;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(&s_base)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t base = s_base;
  const uint32_t trow = base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * 64);
  float acc = 0.f;
  for (int it = 0; it < iters; ++it) {
    float v0[32], v1[32];
    const uint32_t col = (uint32_t)((it & 1) * 256);   // alternate between the two 256-column accumulators
    tc::tc_ld32_issue(trow + col, v0);
    tc::tc_ld32_issue(trow + col + 32u, v1);
    tc::tc_ld_wait();
    acc += v0[0] + v0[31] + v1[0] + v1[31];            // fixed registers (a computed index would spill the arrays)
  }
  if (acc == 123.456f) out[0] = acc;
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc::tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(512) : "memory");
  }
}

}  // namespace
}  // namespace vsk

using namespace vsk;

extern "C" int32_t vsk_measure_peak(vsk_ctx* c, int32_t what, double* per_second) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !per_second) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (what != VSK_PEAK_FP32_ISSUE && what != VSK_PEAK_SMEM_GATHER && what != VSK_PEAK_TMEM_READ)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "unknown peak %d", what);
  void* p;
  VSK_TRY(scratch(ctx, SLOT_MISC6, 256, &p));
  cudaEvent_t e0, e1;
  VSK_CUDA(ctx, cudaEventCreate(&e0));
  VSK_CUDA(ctx, cudaEventCreate(&e1));
  const int sms = ctx->prop.multiProcessorCount;
  // eight 256-thread CTAs per SM (every warp slot filled); the tensor-memory read: one 512-thread CTA per SM, which
  // holds all of the SM's tensor memory
  const unsigned grid = what == VSK_PEAK_TMEM_READ ? (unsigned)sms : (unsigned)sms * 8u;
  const int iters = 16384;   // 1.2e11 FP32 instructions / 2e10 gathered words / 3e11 bytes: a few milliseconds each
  double best = 0.0;
  for (int run = 0; run < 7; ++run) {
    cudaEventRecord(e0, ctx->stream);
    if (what == VSK_PEAK_FP32_ISSUE) fp32_issue_kernel<<<grid, 256, 0, ctx->stream>>>((float*)p, iters, 1.0f);
    else if (what == VSK_PEAK_SMEM_GATHER) smem_gather_kernel<<<grid, 256, 0, ctx->stream>>>((float*)p, iters);
    else tmem_read_kernel<<<grid, 512, 0, ctx->stream>>>((float*)p, iters);
    cudaEventRecord(e1, ctx->stream);
    ctx->stats.kernel_launches++;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (run < 2 || ms <= 0.f) continue;   // warm-up
    const double ops = what == VSK_PEAK_FP32_ISSUE    ? (double)grid * 256.0 * iters * kFpChains * 3.0
                       : what == VSK_PEAK_SMEM_GATHER ? (double)grid * 256.0 * iters * 4.0
                                                      : (double)grid * 512.0 * iters * 64.0 * 4.0;   // bytes
    best = std::max(best, ops / (ms * 1e-3));
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  VSK_CUDA(ctx, cudaGetLastError());
  *per_second = best;
  return VSK_OK;
}
