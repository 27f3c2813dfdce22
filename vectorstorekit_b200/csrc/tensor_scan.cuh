// Entry points of the tensor-core search path (tensor_scan.cu) and of the int8 scan (sq8.cu)
// used by the C ABI layer, plus the fp32 re-run the tensor path falls back on per query.
#pragma once
#include <vector>

#include "common.cuh"

namespace vsk {

// fp16 tcgen05 contraction + bounded-error filter + exact fp32 rerank over a flat fp32 index.
// q: [nq][dim] device; qnorm: |q| per query (cosine) or null; qmasks: per-query filter masks or null (the index
// must then carry row masks); outputs device [nq][k].  A large batch issued on lane 0 runs as two halves on the
// context's two lanes (tensor_lane_split).
int32_t tensor_search(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm, const uint64_t* qmasks,
                      float* out_dist, int64_t* out_ids);
// The same search in two halves, for a shard of a row-sharded search.  `begin` scans and, when bound_out is given,
// writes per query a value that this shard's ceil(k / shards) best rows do not exceed (error bound included, in the
// units of the scan's coarse values, which depend on the query only); the host takes the maximum over the shards and
// passes it to `finish`, which then re-scores only rows that can reach the overall top-k.  `finish` is
// finish_issue (enqueues everything, including the copy of the flag words to pinned host memory), a drain of the
// lane's stream, and finish_collect (reads the flags of lane `from_lane`, -1 = the current one, and re-runs flagged
// queries on the fp32 scan of the current lane).  All state is per lane: the two lanes of a context can each hold one
// search between `begin` and `finish`.
int32_t tensor_search_begin(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm, const uint64_t* qmasks,
                            int32_t shards, float* bound_out);
int32_t tensor_search_finish_issue(Index* ix, const float* ext_bound, float* out_dist, int64_t* out_ids);
int32_t tensor_search_finish_collect(Index* ix, int from_lane);
int32_t tensor_search_finish(Index* ix, const float* ext_bound, float* out_dist, int64_t* out_ids);
int64_t tensor_lane_split(const Ctx* ctx, int64_t nq);
// The coarse values of one dense chunk and the per-query error bound (vsk_coarse_values_dev).
int32_t tensor_coarse_values(Index* ix, const float* q, int64_t nq, int64_t rows, float* coarse, float* eps_out);
// The probed lists of an IVF index scanned on the tensor cores (coarse values, certificate, exact rerank).
// probes: [nq][nprobe] device, nearest list first.  Results go to out_dist / out_ids for every query; the queries
// whose result could not be certified (or whose candidate list overflowed) are returned in `flagged` for the
// caller to re-run on the fp32 list scan.
bool ivf_tensor_applicable(const Index* ix, int64_t nq, int32_t nprobe, int32_t k);
int32_t ivf_tensor_search(Index* ix, const float* q, int64_t nq, const int64_t* probes, int32_t nprobe, int32_t k,
                          const uint64_t* qmasks, float* out_dist, int64_t* out_ids, std::vector<int32_t>* flagged);
// Drops the fp16 operand copy after rows were added; makes it (once per index state).
void tensor_invalidate(Index* ix);
int32_t tensor_prepare_index(Index* ix);

// fp32 scan of the listed queries of a batch (api.cu).
int32_t fp32_search_subset(Index* ix, const float* q, const std::vector<int32_t>& subset, int32_t k,
                           const float* qnorm, const uint64_t* qmasks, float* out_dist, int64_t* out_ids);

// Nearest-centroid assignment on the tensor cores for one k-means run over fixed data rows: the fp16
// operand copy of the rows and the work buffers are made once, then every Lloyd iteration calls
// tensor_assign with the current centroids.
struct TensorAssign {
  int64_t n = 0;
  int32_t dim = 0, dim16 = 0;
  __half* rows16 = nullptr;           // [n][dim16]
  float* stats = nullptr;             // [4][n]: |x'|, |s x - x'|, |x|, eps
  uint64_t* keys = nullptr;           // [n][8] candidate centroids per row
  unsigned long long* best = nullptr; // [n]
  int32_t* count = nullptr;           // [n]
  float* thr = nullptr;               // [n]
  int32_t* bad_rows = nullptr;        // [n] rows handed to the fp32 tile
  void* small = nullptr;              // scalars and centroid-operand statistics
  bool stationary = false;            // short contraction: resident centroid block, |c|^2 / 2 folded into the operands
  float* prev_cent = nullptr;         // [prev_k][dim] the centroids of the previous call (stationary path) ...
  float* shift = nullptr;             // [prev_k] ... and how far each has moved since
  int32_t prev_k = 0;
  bool have_prev = false;
  bool bound_allowed = true;          // thresholds from the triangle inequality where a centroid has hardly moved
  alignas(64) unsigned char map_rows[128] = {};  // TMA tensor map of rows16
  alignas(64) unsigned char map_rows_narrow[128] = {};  // the same through a 16-column box (the fold columns' K16 step)
};
int32_t tensor_assign_prepare(Ctx* ctx, const float* rows, int64_t n, int32_t dim, TensorAssign* ta);
// assign_holds_previous: `assign` holds, for every row, a valid centroid index (the previous iteration's
// assignment), which gives the candidate threshold without the coarse arg-min pass.
int32_t tensor_assign(Ctx* ctx, TensorAssign* ta, const float* rows, const float* centroids, int32_t k,
                      int32_t* assign, float* dist, bool assign_holds_previous);
void tensor_assign_release(TensorAssign* ta);

// Search over an int8-coded flat index (sq8.cu).
int32_t sq8_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, float* out_dist, int64_t* out_ids);

}  // namespace vsk
