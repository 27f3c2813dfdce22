// Shared declarations of the similarity-search library: context, index, candidate-list
// workspace and the launch functions each .cu file exports to the C ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <cstdio>

#include <functional>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>   // header-only; ranges cost nothing unless a profiler is attached

#include "../../include/vsk_cuda.h"
#include "checked.cuh"   // empty unless VSK_CHECKED

namespace vsk {

// ------------------------------------------------------------------------------------------
// Error plumbing: every CUDA call is checked; a failure records text on the context and
// returns a status, never throws.
// ------------------------------------------------------------------------------------------
struct Ctx;
int32_t fail(Ctx* ctx, int32_t status, const char* fmt, ...);

// NVTX range over a scope: entry points and the phases of a search show up by name on a profiler's timeline (the
// reference marks the same spans with os_signpost, Acceleration/Metal/MetalPerformanceProfiler.swift:10-43).
struct TraceRange {
  explicit TraceRange(const char* name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
  TraceRange(const TraceRange&) = delete;
  TraceRange& operator=(const TraceRange&) = delete;
};
#define VSK_TRACE_CAT2(a, b) a##b
#define VSK_TRACE_CAT(a, b) VSK_TRACE_CAT2(a, b)
#define VSK_TRACE(name) ::vsk::TraceRange VSK_TRACE_CAT(vsk_trace_range_, __LINE__)(name)

#define VSK_CUDA(ctx, expr)                                                                   \
  do {                                                                                        \
    cudaError_t e__ = (expr);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return vsk::fail((ctx),                                                                 \
                       e__ == cudaErrorMemoryAllocation ? VSK_ERR_OUT_OF_MEMORY               \
                                                        : VSK_ERR_EXECUTION_FAILED,           \
                       "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__,     \
                       __LINE__);                                                             \
  } while (0)

#define VSK_TRY(expr)                  \
  do {                                 \
    int32_t s__ = (expr);              \
    if (s__ != VSK_OK) return s__;     \
  } while (0)

// ------------------------------------------------------------------------------------------
// Orderable keys: a (distance, row) pair packed so that unsigned 64-bit order is
// (distance ascending, row ascending).  The all-ones key marks an empty slot.
// ------------------------------------------------------------------------------------------
__host__ __device__ inline uint32_t float_to_ordered(float f) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
#endif
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__host__ __device__ inline float ordered_to_float(uint32_t o) {
  uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
__host__ __device__ inline uint64_t make_key(float v, uint32_t id) {
  return ((uint64_t)float_to_ordered(v) << 32) | id;
}
constexpr uint64_t kEmptyKey = ~0ull;

// ------------------------------------------------------------------------------------------
// Candidate lists: per query a fixed-capacity list of (value, row) keys in HBM.
// Scan kernels append every row whose value is <= the query's current threshold;
// compaction keeps the best `keep` and tightens the threshold.
// ------------------------------------------------------------------------------------------
constexpr int kCandCap = 4096;  // keys per query

struct CandLists {
  uint64_t* keys = nullptr;   // [nq][kCandCap]
  int32_t* count = nullptr;   // [nq] appended so far (may exceed cap: overflow)
  float* thr = nullptr;       // [nq] rows with value <= thr are appended
  int32_t* flags = nullptr;   // [nq] bit0: list overflowed; bit1: certificate failed
  int64_t nq = 0;
};

enum ScanMode : int { SCAN_DENSE = 0, SCAN_THRESHOLD = 1, SCAN_MATRIX = 2, SCAN_ARGMIN = 3 };

struct Index;
// What the second half of a search needs from the first (device pointers into the context's scratch, valid until
// the next call on the context).
struct ShardPending {
  bool active = false;
  bool tensor = false;        // false: the index kind or search path has no split form; `finish` runs the whole search
  bool need_cert = false;     // the certifying compaction was left to the second half
  Index* ix = nullptr;
  const float* q = nullptr;
  const float* qnorm = nullptr;
  const uint64_t* qmasks = nullptr;
  int64_t nq = 0;
  int32_t k = 0, keep = 0, max_count = 0;
  CandLists cand;
  const float* eps = nullptr;
  int32_t* err = nullptr;
  unsigned long long* rr_total = nullptr;
  // second half issued, results not yet looked at by the host
  bool issued = false;
  float* out_dist = nullptr;
  int64_t* out_ids = nullptr;
};

struct Comm;   // NCCL communicator of a row-sharded search (comm.cu)
struct Worker; // thread and queue behind the *_async entry points (async.cu)

// Pinned host memory that grows on demand (results the host reads back right after a stream drains).
struct PinnedBuf {
  void* p = nullptr;
  size_t bytes = 0;
};

// A context issues work on one of two LANES.  Lane 0 is the context's stream (`stream_main`, the one vsk_stream
// returns).  A large tensor-path batch is split in two halves; the second half is issued on lane 1 (`stream_aux`),
// so that one half's compactions, re-scoring and exchanges run under the other half's contraction.  `stream` and
// `lane` say where launches and scratch requests go right now (LaneGuard switches them); each lane has its own
// scratch slots and its own pending half-search, so the halves never share a work buffer.
struct Ctx {
  int device = 0;
  cudaStream_t stream = nullptr;        // where launches go now: stream_main, or stream_aux while lane 1 is issued
  cudaStream_t stream_main = nullptr;
  cudaStream_t stream_aux = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  int lane = 0;
  cudaDeviceProp prop{};
  std::string err;
  int32_t search_path = VSK_PATH_TENSOR_RERANK;
  vsk_tuning tuning{};
  vsk_stats stats{};
  // optional timing of the dominant (scan) kernels with CUDA events on `stream`
  bool profile = false;
  std::vector<cudaEvent_t> prof_events;  // begin/end pairs
  size_t prof_used = 0;
  // grow-only device scratch, one buffer per (lane, slot) (see Slot)
  void* scratch[2 * 64] = {};
  size_t scratch_bytes[2 * 64] = {};
  ShardPending pending[2];
  PinnedBuf host_flags[2];   // per lane: the flag words a finished half-search hands to the host
  Comm* comm = nullptr;
  Worker* worker = nullptr;
  // optional event log (vsk_timeline): one event after each marked launch, on the stream it went to
  bool timeline = false;
  struct Mark { const char* name; int lane; cudaEvent_t ev; };
  std::vector<Mark> marks;
  size_t marks_used = 0;
  cudaEvent_t tl_origin = nullptr;
};
// A CUDA runtime error that is not sticky stays in the thread's "last error" slot until somebody reads it; a launch
// check that reads the slot would then blame its own kernel for a failure of an earlier, unrelated call.  Entry points
// drain the slot first and say once on stderr what they found.
inline void drain_stale_error(const char* where) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    static int told = 0;
    if (told++ < 4) fprintf(stderr, "vsk: stale CUDA error before %s: %s\n", where, cudaGetErrorString(e));
  }
}

// Records "the work issued so far on the current lane, up to `name`, is done" when the event log is on.
void tl_mark(Ctx* ctx, const char* name);

// Small kernels (selection, re-scoring, operand preparation, key packing) ask for the largest shared-memory
// carve-out, the configuration the contraction kernel runs under: an SM does not switch its L1 / shared-memory split
// while it holds a CTA, so a kernel that preferred another split could not join the contraction's CTAs on an SM and
// the two lanes of a context would take turns instead of overlapping.
template <typename K>
inline void prefer_shared_carveout(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaGetLastError();
}

// Issues on lane `lane` until it goes out of scope.
struct LaneGuard {
  Ctx* c;
  LaneGuard(Ctx* ctx, int lane) : c(ctx) {
    c->lane = lane;
    c->stream = lane ? c->stream_aux : c->stream_main;
  }
  ~LaneGuard() {
    c->lane = 0;
    c->stream = c->stream_main;
  }
};
// lane 1 starts after everything issued on lane 0 so far; lane 0 continues after everything issued on lane 1
int32_t lanes_fork(Ctx* ctx);
int32_t lanes_join(Ctx* ctx);
int32_t pinned_reserve(Ctx* ctx, PinnedBuf* b, size_t bytes);

enum Slot : int {
  SLOT_Q = 0, SLOT_OUT_D, SLOT_OUT_I, SLOT_QMASK, SLOT_CAND_KEYS, SLOT_CAND_COUNT, SLOT_CAND_THR,
  SLOT_CAND_FLAGS, SLOT_QNORM, SLOT_SUBSET, SLOT_Q16, SLOT_QAUX, SLOT_X_TMP, SLOT_MISC0, SLOT_MISC1,
  SLOT_MISC2, SLOT_MISC3, SLOT_MISC4, SLOT_MISC5, SLOT_MISC6,
  SLOT_IVF_PROBE_D, SLOT_IVF_PROBE_I, SLOT_IVF_KEYS, SLOT_IVF_ORDER, SLOT_IVF_PAIR_OFF, SLOT_IVF_ITEM_CNT,
  SLOT_IVF_ITEM_OFF, SLOT_IVF_SUBSET, SLOT_IVF_STAGES, SLOT_KM_NSEG, SLOT_KM_SEGOFF, SLOT_KM_PARTIAL, SLOT_FILTER_PERM, SLOT_FILTER_ROWS, SLOT_FILTER_COUNT, SLOT_SQ_A, SLOT_SQ_B, SLOT_TC_A, SLOT_TC_B, SLOT_TC_C, SLOT_TC_D,
  SLOT_PQ_TABLES, SLOT_SH_D, SLOT_SH_I, SLOT_SH_SEND, SLOT_SH_RECV, SLOT_SH_BOUND, SLOT_SH_MERGED, SLOT_SH_ALL,
  SLOT_COUNT
};
static_assert(SLOT_COUNT <= 64, "grow Ctx::scratch");
// Event pair around a scan-kernel launch when profiling is on (api.cu).
void prof_begin(Ctx* ctx);
void prof_end(Ctx* ctx);
// After the stream has drained: adds the recorded intervals to stats.scan_kernel_ms.
void prof_collect(Ctx* ctx);

// Device pointer of at least `bytes` for the slot; contents are not preserved across growth.
int32_t scratch(Ctx* ctx, int slot, size_t bytes, void** out);

enum IndexKind : int { INDEX_FLAT_F32 = 0, INDEX_FLAT_I8 = 1, INDEX_IVF = 2, INDEX_PQ = 3 };

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
};

// One block of rows added to a flat index.  Blocks are concatenated logically.
struct Index {
  Ctx* ctx = nullptr;
  int kind = INDEX_FLAT_F32;
  int32_t metric = 0;
  int32_t dim = 0;
  int64_t n = 0;
  int64_t capacity = 0;
  int64_t id_base = 0;
  float* rows = nullptr;       // [capacity][dim] fp32
  float* row_norm = nullptr;   // [capacity] |x| (cosine), |x|^2 (euclidean)
  uint64_t* masks = nullptr;   // [capacity]; meaningful when has_masks
  bool has_masks = false;
  // fp16 operand copy for the tensor path (built lazily, invalidated by add)
  __half* rows16 = nullptr;    // [n16_rows][dim16]
  int32_t dim16 = 0;
  int64_t n16 = 0;             // rows converted
  float* row_aux = nullptr;    // [n] per-row epilogue term (|x*s|^2 in operand units for L2)
  float scale16 = 1.0f;        // power-of-two operand scale s_x
  float max_xnorm16 = 0.f;     // max |x'| over rows
  float max_xerr16 = 0.f;      // max |x*s - x'| over rows
  float min_xnorm_nz = 0.f;    // min nonzero |x|
  float max_xnorm = 0.f;       // max |x|
  bool fold16 = false;         // euclidean: the per-row term |x|^2 rides in sixteen operand columns behind the data (tensor_scan.cu)
  int32_t fold_exp = 0;        // ... scaled by 2^fold_exp
  float fold_bmax = 0.f;       // ... max |x|^2 / 2
  // int8
  int8_t* codes = nullptr;     // [capacity][dim]
  float* sq_scale = nullptr;   // [dim]
  float* sq_offset = nullptr;  // [dim]
  // ivf
  int32_t nlist = 0;
  float* centroids = nullptr;      // [nlist][dim]
  int64_t* list_offsets = nullptr; // [nlist+1] device
  std::vector<int64_t> list_offsets_h;
  int32_t* list_rows = nullptr;    // [n] original row of each stored row
  int32_t* assign = nullptr;       // [n] row -> list (original order)
  Index* coarse = nullptr;         // the centroids as a flat euclidean index (made at the first tensor-path search;
                                   // shares `centroids`, owns only its derived buffers)
  // product quantisation
  int32_t pq_m = 0, pq_ksub = 0;   // segments, codewords per segment
  float* pq_codebooks = nullptr;   // [pq_m][pq_ksub][dim / pq_m]
  uint8_t* pq_codes = nullptr;     // [capacity][pq_m]
};

// ---- exact_scan.cu -----------------------------------------------------------------------
struct ExactScanArgs {
  int32_t metric;
  int mode;                 // ScanMode
  const float* q;           // [nq][dim]
  const float* x;           // [n][dim] fp32 rows, or
  const int8_t* x_codes;    // [n][dim] int8 codes with per-dimension sq_scale / sq_offset
  const float* sq_scale;
  const float* sq_offset;
  int32_t dim;
  int64_t nq;
  int64_t row_begin, row_end;   // rows of this launch
  const float* qnorm;       // [nq] |q| (cosine)
  const float* xnorm;       // [n] |x| (cosine)
  const uint64_t* row_masks;  // or null
  const uint64_t* q_masks;    // or null
  const int32_t* q_subset;  // or null: indices of the queries to run (nq = subset size)
  const int32_t* x_rows;    // or null: the rows to scan, as a list of row numbers (row_begin/row_end index the list)
  int32_t bm_hint;          // 0, or 32 / 64: query rows per CTA for launches with few queries
  CandLists cand;           // SCAN_DENSE / SCAN_THRESHOLD
  float* out;               // SCAN_MATRIX: [nq][ld_out]
  int64_t ld_out;
  unsigned long long* best; // SCAN_ARGMIN: [nq] smallest (value, row) key, pre-set to all ones
  // Per-query row lists (streaming scan only; the probed lists of an IVF search for a few queries): query i
  // (q_subset[m] for list position m) scans entries [seg_begin[i], seg_begin[i] + seg_count[i]) of x_rows, and
  // row_begin / row_end index positions inside each query's own slice.  Null otherwise.
  const int64_t* seg_begin;
  const int32_t* seg_count;
  // fp32_topk only (or null): the scan's row numbers are positions in some stored order and final_id_remap[row] is
  // the row's id; the final ordering then breaks equal values by id, and the ids (plus id_base) are what is returned.
  const int32_t* final_id_remap;
};
int32_t launch_exact_scan(Ctx* ctx, const ExactScanArgs& a);
// ---- stream_scan.cu ------------------------------------------------------------------------
// The same scan for a batch of at most kStreamScanMaxQueries queries over fp32 rows, candidate modes only: queries
// in shared memory, every row streamed from HBM once.  launch_exact_scan hands such launches over.
constexpr int kStreamScanMaxQueries = 8;
constexpr int kStreamScanMaxSegQueries = 16;   // with per-query row lists (one grid row per query): beyond this the
                                               // list-major tiles, which read a list once for all its queries, win
bool stream_scan_applies(const Ctx* ctx, const ExactScanArgs& a);
int32_t launch_stream_scan(Ctx* ctx, const ExactScanArgs& a);
int32_t launch_row_norms(Ctx* ctx, const float* x, int64_t n, int32_t dim, int squared, float* out);

// ---- group.cu ----------------------------------------------------------------------------
// Stable grouping of n items by key in [0, nkeys): order[] lists item indices key by key, ascending
// item index inside a key; offsets[nkeys+1] (int64) bounds each key's run.  Deterministic.
int32_t launch_stable_group(Ctx* ctx, const int32_t* keys, int64_t n, int32_t nkeys, int32_t* order,
                            int64_t* offsets);

// ---- kmeans.cu ---------------------------------------------------------------------------
int32_t assign_rows(Ctx* ctx, const float* rows, int64_t n, int32_t dim, const float* centroids, int32_t k,
                    int32_t* assign, float* dist);

// offsets[0..n] = exclusive scan of totals[0..n) (single block; group.cu)
int32_t launch_scan_i64(Ctx* ctx, const int64_t* totals, int32_t n, int64_t* offsets);

// ---- select.cu ---------------------------------------------------------------------------
struct SelectArgs {
  CandLists cand;
  int64_t nq;
  int32_t dense_count;      // >=0: list holds exactly this many slots (dense chunk); <0: use count[]
  int32_t keep;             // keep the best `keep`
  // final output (null while compacting)
  float* out_dist;          // [nq][k]
  int64_t* out_ids;
  int32_t k;
  int32_t metric;           // output transform of the stored value
  int64_t id_base;
  const int32_t* q_subset;  // or null; lists are indexed by position, outputs by q_subset[pos]
  int final_sqrt;           // 1: stored value is a squared L2 distance
  const float* cert_eps;    // non-null: last compaction of a coarse scan (see select.cu); uses k
  int32_t max_count;        // > 0: no list of this launch is expected to hold more keys (picks the kernel width)
  // Row-sharded search (the two halves of a shard's search, see tensor_scan.cuh):
  float* bound_out;         // non-null: measure only.  Writes the bound_rank-th smallest value of the list plus
  int32_t bound_rank;       //   bound_eps[q] (+inf when the list is shorter) and leaves the list as it is.
  const float* bound_eps;
  const float* ext_bound;   // with cert_eps: per query, a value (same units, error bound included) that at least k
                            //   rows over all shards do not exceed; rows above ext_bound + eps cannot matter
  const int32_t* id_remap;  // final output only (or null): a key's row field is replaced by id_remap[row] before the
                            //   list is ordered, so equal values are ordered by that id
};
int32_t launch_select(Ctx* ctx, const SelectArgs& a);
int32_t launch_merge_topk(Ctx* ctx, const float* dist, const int64_t* ids, int32_t g, int64_t nq,
                          int32_t k, float* out_dist, int64_t* out_ids);
int32_t launch_init_cand(Ctx* ctx, const CandLists& c, int64_t nq);
// Packed (distance, global row) keys for the exchange between shards (select.cu): pack [nq][k] results into
// [rows][k] keys (rows >= nq: padding is filled with missing entries), merge g lists per query, unpack.
int32_t launch_pack_keys(Ctx* ctx, const float* dist, const int64_t* ids, int64_t nq, int64_t rows, int32_t k,
                         uint64_t* keys);
int32_t launch_unpack_keys(Ctx* ctx, const uint64_t* keys, int64_t count, float* dist, int64_t* ids);
int32_t launch_merge_keys(Ctx* ctx, const uint64_t* in, int32_t g, int64_t stride_q, int64_t nq, int32_t k, uint64_t* out);

// ---- search schedule in api.cu -------------------------------------------------------------
// A scan of rows [row_begin, row_end) in ScanMode `mode` that writes keys into candidate lists, and the function
// that binds lists, batch size and query subset to such a scan.
using ScanFn = std::function<int32_t(int mode, int64_t row_begin, int64_t row_end)>;
using ScanBinder = std::function<ScanFn(const CandLists& cand, int64_t nq, const int32_t* sub_dev)>;
int32_t scan_topk(Ctx* ctx, const ScanBinder& make_scan, int64_t n, int64_t nq, const int32_t* sub_dev, int32_t k,
                  int64_t id_base, int final_sqrt, float* out_dist, int64_t* out_ids, int level,
                  const int32_t* id_remap = nullptr);
// Exact top-k of nq queries over n rows with the fp32 scan; `proto` carries metric, operands,
// norms and masks.  Outputs are device pointers [nq][k] (indexed by sub_dev[pos] when given).
int32_t fp32_topk(Ctx* ctx, const ExactScanArgs& proto, int64_t n, int64_t nq, const int32_t* sub_dev, int32_t k,
                  int64_t id_base, float* out_dist, int64_t* out_ids, int level);
// Rows of the next chunk of the search schedule (api.cu).
int64_t schedule_chunk(int64_t seen, int32_t keep, int level);
// Rows of the dense first chunk, and an upper bound (mean + 8 deviations) on the keys a list holds after a
// thresholded chunk of `chunk` rows that followed `seen` rows.
int64_t schedule_dense_rows(const Ctx* ctx, int32_t keep);
int32_t schedule_max_count(int64_t seen, int64_t chunk, int32_t keep);

// ---- pq.cu -------------------------------------------------------------------------------
int32_t pq_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, float* out_dist, int64_t* out_ids);
int32_t pq_reserve(Index* ix, int64_t need);

// ---- helpers in api.cu ---------------------------------------------------------------------
vsk_tuning default_tuning();
// comm.cu: leaves the context's communicator, if any
void comm_release(Ctx* ctx);
// Range table of the checked build (checked.cu); no-ops otherwise.
int32_t chk_open(Ctx* ctx);
void chk_add(const void* p, size_t bytes);
void chk_remove(const void* p);
void worker_release(Ctx* ctx);
int32_t dev_alloc(Ctx* ctx, void** p, size_t bytes);
void dev_free(void* p);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace vsk
