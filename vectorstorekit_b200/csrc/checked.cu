// Host side of the CHECKED build: the table of device address ranges the instrumented kernels may touch.
//
// In a normal build this file only provides the exported entry points as "not a checked build" answers and the
// allocation hooks as no-ops.  With -DVSK_CHECKED (python -m vectorstorekit_b200.build --checked) every global access
// of every kernel is routed through vsk_chk_access (checked.cuh, added to the PTX by ptx_check.py), which looks the
// address up in the table kept here:
//   * every device allocation of the library, with the size the call asked for (dev_alloc, scratch),
//   * device buffers the caller announces with vsk_checked_register (the `_dev` entry points take caller memory; the
//     Python mirror announces every tensor it passes),
//   * the library's own static device arrays.
// A refused access goes to a sink instead of its address and is counted; vsk_checked_faults reads the count and the
// first offender.  Nothing traps and no invalid address is ever touched, so the context stays usable.
// The reference's counterpart is Metal's shader validation layer and its API validation, which a Swift host turns on
// per process; compute-sanitizer would be CUDA's, where it is available.
#include <algorithm>
#include <map>
#include <mutex>
#include <vector>

#include "common.cuh"

#ifdef VSK_CHECKED
namespace vsk {
namespace chk {
namespace {

struct DeviceTable {
  State* dev = nullptr;
  int version = 0;
  std::map<unsigned long long, unsigned long long> ranges;   // lo -> hi, disjoint
};

std::mutex& mu() {
  static std::mutex m;
  return m;
}
std::vector<void (*)(State*)>& setters() {
  static std::vector<void (*)(State*)> v;
  return v;
}
std::map<int, DeviceTable>& tables() {
  static std::map<int, DeviceTable> t;
  return t;
}

// Writes the next table slot and publishes it.  Synchronous copies: the caller is about to launch work that needs it.
void upload(DeviceTable& t) {
  if (!t.dev) return;
  std::vector<Range> flat;
  flat.reserve(t.ranges.size());
  for (auto& kv : t.ranges) flat.push_back(Range{kv.first, kv.second});
  if ((int)flat.size() > kMaxRanges) {
    static bool told = false;
    if (!told) fprintf(stderr, "vsk (checked): more than %d ranges, the largest addresses are not covered\n", kMaxRanges);
    told = true;
    flat.resize(kMaxRanges);
  }
  const int next = (t.version + 1) & (kTables - 1);
  const int n = (int)flat.size();
  if (n) cudaMemcpy(&t.dev->ranges[next][0], flat.data(), sizeof(Range) * (size_t)n, cudaMemcpyHostToDevice);
  cudaMemcpy(&t.dev->count[next], &n, sizeof(int), cudaMemcpyHostToDevice);
  cudaMemcpy(&t.dev->version, &next, sizeof(int), cudaMemcpyHostToDevice);
  t.version = next;
}

DeviceTable* current() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return nullptr;
  return &tables()[d];
}

}  // namespace

void register_module(void (*setter)(State*)) { setters().push_back(setter); }

}  // namespace chk

// Called by vsk_open with the device selected.
int32_t chk_open(Ctx* ctx) {
  std::lock_guard<std::mutex> lk(chk::mu());
  chk::DeviceTable* t = chk::current();
  if (!t) return VSK_OK;
  if (!t->dev) {
    VSK_CUDA(ctx, cudaMalloc((void**)&t->dev, sizeof(chk::State)));
    VSK_CUDA(ctx, cudaMemset(t->dev, 0, sizeof(chk::State)));
    for (auto set : chk::setters()) set(t->dev);
    VSK_CUDA(ctx, cudaGetLastError());
    chk::upload(*t);
  }
  return VSK_OK;
}

static void chk_add_to(chk::DeviceTable* t, const void* p, size_t bytes) {
  const unsigned long long lo = (unsigned long long)(uintptr_t)p, hi = lo + bytes;
  // Ranges that overlap the new one are leftovers of buffers the caller's allocator has since reused (live buffers
  // do not overlap).  A leftover that contains the new range whole may equally be a live buffer of which this is a
  // slice: it stays.  Others lose the part that overlaps - not more: the rest may still cover a live buffer that
  // was announced while it lay inside the leftover.
  auto it = t->ranges.upper_bound(lo);
  if (it != t->ranges.begin()) {
    auto prev = std::prev(it);
    if (prev->first <= lo && prev->second >= hi) return;   // already covered
    if (prev->second > lo) it = prev;
  }
  std::vector<std::pair<unsigned long long, unsigned long long>> keep;
  while (it != t->ranges.end() && it->first < hi) {
    if (it->first < lo) keep.emplace_back(it->first, lo);
    if (it->second > hi) keep.emplace_back(hi, it->second);
    it = t->ranges.erase(it);
  }
  for (auto& r : keep) t->ranges[r.first] = r.second;
  t->ranges[lo] = hi;
  chk::upload(*t);
}

void chk_add(const void* p, size_t bytes) {
  if (!p || !bytes) return;
  std::lock_guard<std::mutex> lk(chk::mu());
  chk::DeviceTable* t = chk::current();
  if (t) chk_add_to(t, p, bytes);
}

void chk_remove(const void* p) {
  if (!p) return;
  std::lock_guard<std::mutex> lk(chk::mu());
  chk::DeviceTable* t = chk::current();
  if (!t) return;
  if (t->ranges.erase((unsigned long long)(uintptr_t)p)) chk::upload(*t);
}

namespace {
// Reads one word just past a buffer's announced end: an instrumented build refuses the access (it reads the sink).
__global__ void selftest_kernel(const int* buf, int words, int* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = buf[words];
}
}  // namespace

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_checked_build(void) { return 1; }

int32_t vsk_checked_register(const void* p, int64_t bytes) {
  if (!p || bytes <= 0) return VSK_ERR_INVALID_INPUT;
  // the buffer's own GPU, whichever device the calling thread has selected
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    cudaGetLastError();
    return VSK_ERR_INVALID_INPUT;
  }
  std::lock_guard<std::mutex> lk(chk::mu());
  chk_add_to(&chk::tables()[attr.device], p, (size_t)bytes);
  return VSK_OK;
}

int32_t vsk_checked_unregister(const void* p) {
  chk_remove(p);
  return VSK_OK;
}

int32_t vsk_checked_faults(vsk_ctx* c, uint64_t* out3) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out3) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream_main));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream_aux));
  std::lock_guard<std::mutex> lk(chk::mu());
  chk::DeviceTable* t = chk::current();
  out3[0] = out3[1] = out3[2] = 0;
  if (!t || !t->dev) return VSK_OK;
  unsigned long long h[3];
  VSK_CUDA(ctx, cudaMemcpy(h, &t->dev->faults, sizeof(h), cudaMemcpyDeviceToHost));
  out3[0] = h[0]; out3[1] = h[1]; out3[2] = h[2];
  VSK_CUDA(ctx, cudaMemset(&t->dev->faults, 0, sizeof(h)));
  return VSK_OK;
}

// A positive control that touches no invalid memory: a 4 KB allocation of which only the first 1 KB is announced;
// the kernel reads the word at byte 1024.  Instrumented, the read is refused (one fault recorded, value from the sink);
// the memory behind the announced end is the library's own either way.
int32_t vsk_checked_selftest(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  void* buf = nullptr;
  VSK_CUDA(ctx, cudaMalloc(&buf, 4096));
  VSK_CUDA(ctx, cudaMemsetAsync(buf, 0, 4096, ctx->stream));
  chk_add(buf, 1024);
  int* out = reinterpret_cast<int*>(buf) + 8;   // inside the announced part
  selftest_kernel<<<1, 32, 0, ctx->stream>>>(reinterpret_cast<const int*>(buf), 256, out);
  const cudaError_t e = cudaStreamSynchronize(ctx->stream);
  chk_remove(buf);
  cudaFree(buf);
  if (e != cudaSuccess) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "self-test kernel failed: %s", cudaGetErrorString(e));
  return VSK_OK;
}

}  // extern "C"

#else  // ---------------------------------------------------------------- normal build

namespace vsk {
int32_t chk_open(Ctx*) { return VSK_OK; }
void chk_add(const void*, size_t) {}
void chk_remove(const void*) {}
}  // namespace vsk

extern "C" {
int32_t vsk_checked_build(void) { return 0; }
int32_t vsk_checked_register(const void*, int64_t) { return VSK_OK; }
int32_t vsk_checked_unregister(const void*) { return VSK_OK; }
int32_t vsk_checked_faults(vsk_ctx* c, uint64_t* out3) {
  if (!c || !out3) return VSK_ERR_INVALID_INPUT;
  out3[0] = out3[1] = out3[2] = 0;
  return VSK_OK;
}
int32_t vsk_checked_selftest(vsk_ctx* c) {
  vsk::Ctx* ctx = reinterpret_cast<vsk::Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  return vsk::fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "not a checked build");
}
}  // extern "C"

#endif
