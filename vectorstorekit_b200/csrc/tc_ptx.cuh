// tcgen05 / TMA / mbarrier building blocks shared by the contraction kernels (inline PTX for sm_100a).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vsk {
namespace tc {

constexpr int TM = 128;        // queries per tile (UMMA M)
constexpr int TN = 256;        // rows per tile (UMMA N)
constexpr int TK = 64;         // fp16 elements per k-block (128 bytes: one swizzle atom)
constexpr int A_BYTES = TM * TK * 2;   // 16 KB: 128 query rows x 64 fp16
constexpr int B_BYTES = TN * TK * 2;   // 32 KB: 256 database rows x 64 fp16
constexpr uint32_t WAIT_LIMIT = 1u << 23;
constexpr int TMEM_COLS = 512;

// ---- PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// True in exactly one lane of a converged warp.  A warp that runs its loop converged and issues through the elected
// lane keeps descriptors, coordinates and barrier addresses warp-uniform (the tensor and copy instructions take their
// operands from uniform registers; inside an `if (lane == 0)` region every operand is moved there per instruction).
__device__ __forceinline__ bool elect_one() {
  uint32_t is_leader;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(is_leader));
  return is_leader != 0;
}
// One look at the barrier, never suspended: true when the phase with this parity has completed.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag and the error word) when the limit runs out
// or another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* err, int code,
                                          uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) {
      if ((it & 63) == 0 && *abort_flag) return false;
      __nanosleep(64);
    }
  }
  *abort_flag = 1;
  atomicCAS(err, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; M = 128, N = 256, K = 16, fp16 x fp16 -> fp32
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait: several loads can be in flight before one tc_ld_wait.
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, float (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
        "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
        "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
        "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// largest of 32 values by a tree (depth 5) instead of a chain of 31 dependent operations
__device__ __forceinline__ float max32(const float (&v)[32]) {
  float m[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) m[i] = fmaxf(v[2 * i], v[2 * i + 1]);
#pragma unroll
  for (int w = 8; w > 0; w >>= 1)
#pragma unroll
    for (int i = 0; i < w; ++i) m[i] = fmaxf(m[i], m[i + w]);
  return m[0];
}

// max of three in one instruction (sm_100 has a three-input max; NaN operands are passed over as in fmaxf)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// largest of v[O .. O+7]: four instructions, depth three
template <int O>
__device__ __forceinline__ float max8(const float (&v)[32]) {
  return max3(v[O + 6], v[O + 7], fmaxf(max3(v[O], v[O + 1], v[O + 2]), max3(v[O + 3], v[O + 4], v[O + 5])));
}

// bit j of the result: v[O + j] >= bar, j = 0..7
template <int O>
__device__ __forceinline__ uint32_t ge_bits8(const float (&v)[32], float bar) {
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) bits |= (v[O + j] >= bar) ? (1u << j) : 0u;
  return bits;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 fp16), 128-byte
// swizzled, rows packed: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                      // leading-dimension byte offset (unused with swizzle): 1
  d |= (uint64_t)(1024 >> 4) << 32;            // stride between 8-row groups: 1024 bytes
  d |= (uint64_t)1 << 46;                      // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                      // 128-byte swizzle
  return d;
}

// The same for a tile of ONE K16 step: rows of 32 bytes (16 fp16), 32-byte swizzled, 8-row groups 256 bytes apart
// (what a TMA box of 16 columns with CU_TENSOR_MAP_SWIZZLE_32B writes).
constexpr int A_NARROW_BYTES = TM * 32;   // 4 KB
constexpr int B_NARROW_BYTES = TN * 32;   // 8 KB
__device__ __forceinline__ uint64_t make_desc_narrow(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(256 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)6 << 61;                      // 32-byte swizzle
  return d;
}

// The descriptors above split into the word that changes with the address and the constant word, and barrier
// operations that take a shared-memory address as a 32-bit number: an issuer loop that keeps its state in 32-bit
// registers spends fewer instructions between the last MMA of one tile and the first of the next.
// (A CTA's shared memory ends below 256 KB, so an address in 16-byte units stays below 2^14: offsets inside the CTA's
// buffers may be added to the low word without a carry into the field above it.)
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3fffu) | (1u << 16); }
constexpr uint32_t kDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescHiNarrow = (uint32_t)(256 >> 4) | (1u << 14) | (6u << 29);
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }
__device__ __forceinline__ bool mbar_test_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void tc_commit_a(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

}  // namespace tc
}  // namespace vsk
