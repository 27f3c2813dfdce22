// Device side of the CHECKED build (-DVSK_CHECKED): the range test every instrumented global access calls.
//
// The build runs a pass over each module's PTX (vectorstorekit_b200/ptx_check.py) that routes the address of every
// global or generic load, store, atomic and reduction through vsk_chk_access below.  The function and the pointer to
// the range table are `static`: every module carries its own copy (the library is built without relocatable device
// code), and every module registers a setter with the host side (checked.cu) so that vsk_open can hand all of them
// the same table.
#pragma once
#ifdef VSK_CHECKED
#include <cuda_runtime.h>
#include <stdint.h>

namespace vsk {
namespace chk {

constexpr int kMaxRanges = 2048;
constexpr int kTables = 4;

struct Range {
  unsigned long long lo, hi;   // [lo, hi)
};

// Lives in device memory, one per GPU.  The host rewrites table (version + 1) % kTables and then publishes `version`;
// a kernel in flight keeps reading the table it started with.
struct State {
  int version;
  int count[kTables];
  unsigned long long faults;        // accesses refused so far
  unsigned long long first_addr;    // the first of them
  unsigned long long first_info;    // its size in bytes | write << 8 | misaligned << 9
  unsigned long long sink[64];      // where refused accesses go instead (a 256-byte-aligned window inside it)
  Range ranges[kTables][kMaxRanges];
};

static __device__ State* d_state = nullptr;

// Host side (checked.cu).
void register_module(void (*setter)(State*));
static void set_state(State* s) { cudaMemcpyToSymbol(d_state, &s, sizeof(s)); }
namespace {
struct ModuleRegistration {
  ModuleRegistration() { register_module(&set_state); }
};
static ModuleRegistration module_registration;
}  // namespace

// Returns `addr` when [addr, addr + bytes) lies inside a known range (or is not a global address); otherwise records
// the violation and returns the sink's address.  info = bytes | write << 8.
static __device__ __noinline__ unsigned long long vsk_chk_access(unsigned long long addr, unsigned info) {
  if (!__isGlobal(reinterpret_cast<const void*>(addr))) return addr;   // shared / local windows: bounded by hardware
  State* s = d_state;
  if (s == nullptr) return addr;                                       // no table yet (a launch before vsk_open)
  const unsigned bytes = info & 0xffu;
  const bool misaligned = (addr & (unsigned long long)(bytes - 1u)) != 0ull;   // every access size is a power of two
  const int t = *reinterpret_cast<volatile int*>(&s->version) & (kTables - 1);
  const Range* r = s->ranges[t];
  int lo = 0, hi = s->count[t];   // first range with r.lo > addr
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (r[mid].lo <= addr) lo = mid + 1; else hi = mid;
  }
  const bool inside = lo > 0 && addr + bytes <= r[lo - 1].hi;
  // the state itself (the sink included) is always a legal target
  const unsigned long long sb = reinterpret_cast<unsigned long long>(s);
  const bool own = addr >= sb && addr + bytes <= sb + sizeof(State);
  if ((inside || own) && !misaligned) return addr;
  if (atomicAdd(&s->faults, 1ull) == 0ull) {
    s->first_addr = addr;
    s->first_info = (unsigned long long)info | (misaligned ? 0x200ull : 0ull);
  }
  return (reinterpret_cast<unsigned long long>(&s->sink[0]) + 255ull) & ~255ull;
}

// Keeps the function in modules whose own code never calls it before the PTX pass adds the calls.
static __global__ void keepalive_kernel(unsigned long long* p, unsigned info) {
  *p = vsk_chk_access(reinterpret_cast<unsigned long long>(p), info);
}

}  // namespace chk
}  // namespace vsk
#endif  // VSK_CHECKED
