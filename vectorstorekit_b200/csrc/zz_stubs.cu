#include "common.cuh"
#include "tensor_scan.cuh"
namespace vsk {
int32_t tensor_search(Index* ix, const float*, int64_t, int32_t, const float*, float*, int64_t*) { return fail(ix->ctx, VSK_ERR_UNSUPPORTED_OPERATION, "tensor path not built"); }
void tensor_invalidate(Index*) {}
}
