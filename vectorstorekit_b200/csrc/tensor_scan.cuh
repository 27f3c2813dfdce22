// Entry points of the tensor-core search path (tensor_scan.cu) and of the int8 scan (sq8.cu)
// used by the C ABI layer, plus the fp32 re-run the tensor path falls back on per query.
#pragma once
#include <vector>

#include "common.cuh"

namespace vsk {

// fp16 tcgen05 contraction + bounded-error filter + exact fp32 rerank over a flat fp32 index.
// q: [nq][dim] device; qnorm: |q| per query (cosine) or null; outputs device [nq][k].
int32_t tensor_search(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm,
                      float* out_dist, int64_t* out_ids);
// Drops the fp16 operand copy after rows were added.
void tensor_invalidate(Index* ix);

// fp32 scan of the listed queries of a batch (api.cu).
int32_t fp32_search_subset(Index* ix, const float* q, const std::vector<int32_t>& subset, int32_t k,
                           const float* qnorm, float* out_dist, int64_t* out_ids);

// Search over an int8-coded flat index (sq8.cu).
int32_t sq8_search_dev(Index* ix, const float* q, int64_t nq, int32_t k, float* out_dist, int64_t* out_ids);

}  // namespace vsk
