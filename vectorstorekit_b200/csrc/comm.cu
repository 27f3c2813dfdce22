// Row-sharded search over the GPUs of one box, one process and one context per GPU.
//
// The reference has no multi-device search; its hosts await one call
// (MetalAccelerationEngine.batchComputeDistances, Acceleration/MetalAccelerationEngine.swift:139-204,444-449), and
// vsk_search_sharded is that one call for a database whose rows are spread over several GPUs.
//
//   scan       every rank scans its shard with the single-GPU kernels (for a flat fp32 index on the tensor path:
//              in two halves, so that the shards can agree on a bound between them)
//   bound      one all-reduce (max) of nq floats: a value that at least k rows of the whole database do not
//              exceed; a shard then re-scores only rows that can reach the overall top-k
//   exchange   the per-shard [nq][k] results travel as packed 64-bit (distance, global row) keys in ONE all-to-all:
//              rank g receives every shard's lists for its slice of the queries
//   merge      rank g merges its slice (unsigned key order = (distance, global row) order: the unsharded result)
//   gather     optional: one all-gather of the merged keys hands every rank the whole result
//
// Collectives are NCCL's, enqueued on the context's streams: data lands in local HBM before any kernel of this
// library reads it, and no kernel here touches another GPU's memory.  NCCL is loaded with dlopen when a
// communicator is first asked for, so the library itself has no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>   // types and enumerators only; every function is looked up at run time

#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "tensor_scan.cuh"

namespace vsk {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
};

// The process's NCCL, or null.  A library with this soname that the process has already loaded (a Python host that
// imported torch) is the one dlopen returns, so both use the same NCCL.
static const NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return nullptr;
  bool ok = true;
  auto sym = [&](const char* name) {
    void* p = dlsym(h, name);
    if (!p) ok = false;
    return p;
  };
  api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
  api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
  api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
  api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
  api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
  api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
  api.Send = (decltype(api.Send))sym("ncclSend");
  api.Recv = (decltype(api.Recv))sym("ncclRecv");
  api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
  api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
  if (!ok) return nullptr;
  api.handle = h;
  return &api;
}

struct Comm {
  ncclComm_t comm = nullptr;
  int nranks = 1, rank = 0;
  cudaEvent_t ev[VSK_SHARDED_PHASES + 1] = {};
  bool timed = false;                       // the events of the last call were recorded
  float phase_ms[VSK_SHARDED_PHASES] = {};
};

#define VSK_NCCL(ctx, api, expr)                                                                              \
  do {                                                                                                        \
    ncclResult_t r__ = (expr);                                                                                \
    if (r__ != ncclSuccess)                                                                                   \
      return vsk::fail((ctx), VSK_ERR_EXECUTION_FAILED, "%s failed: %s", #expr, (api)->GetErrorString(r__)); \
  } while (0)

void comm_release(Ctx* ctx) {
  Comm* cm = ctx->comm;
  if (!cm) return;
  const NcclApi* api = nccl_api();
  if (api && cm->comm) api->CommDestroy(cm->comm);
  for (auto& e : cm->ev)
    if (e) cudaEventDestroy(e);
  delete cm;
  ctx->comm = nullptr;
}

static void slice_of(int64_t nq, int nranks, int rank, int64_t* first, int64_t* count) {
  const int64_t per = ceil_div(nq, std::max(nranks, 1));
  const int64_t lo = std::min<int64_t>((int64_t)rank * per, nq);
  *first = lo;
  *count = std::min<int64_t>(per, nq - lo);
}

// Phase boundary p of a sharded call: an event on lane 0's stream when profiling is on.
static void phase_mark(Ctx* ctx, Comm* cm, int p) {
  if (cm->timed) cudaEventRecord(cm->ev[p], ctx->stream_main);
}

// all-to-all of `per * k` keys per peer: peer p gets send[p], this rank's recv[p] comes from p
static int32_t exchange_keys(Ctx* ctx, const NcclApi* api, Comm* cm, const uint64_t* send, uint64_t* recv, int64_t per,
                             int32_t k) {
  const size_t cnt = (size_t)per * k;
  VSK_NCCL(ctx, api, api->GroupStart());
  for (int p = 0; p < cm->nranks; ++p) {
    ncclResult_t r = api->Send(send + (size_t)p * cnt, cnt, ncclUint64, p, cm->comm, ctx->stream);
    if (r == ncclSuccess) r = api->Recv(recv + (size_t)p * cnt, cnt, ncclUint64, p, cm->comm, ctx->stream);
    if (r != ncclSuccess) {
      api->GroupEnd();
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "ncclSend/ncclRecv failed: %s", api->GetErrorString(r));
    }
  }
  VSK_NCCL(ctx, api, api->GroupEnd());
  tl_mark(ctx, "all_to_all");
  return VSK_OK;
}

int32_t flat_search_dev_entry(Index* ix, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, float* out_dist,
                              int64_t* out_ids);   // api.cu: vsk_search_dev without the device selection
int32_t ivf_search_dev_entry(Index* ix, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                             float* out_dist, int64_t* out_ids);   // ivf.cu

// nprobe > 0: an IVF index whose every shard holds a slice of every list (the centroids are the same on all ranks:
// vsk_kmeans_trainer_* with all-reduced sums), probed with that many lists; nprobe == 0: flat fp32 / int8.
static int32_t search_sharded_dev(Index* ix, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, int32_t layout,
                                  float* out_dist, int64_t* out_ids, int32_t nprobe = 0) {
  Ctx* ctx = ix->ctx;
  Comm* cm = ctx->comm;
  if (nq <= 0 || ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "empty queries or empty index");
  if (k <= 0 || k > kCandCap / 2) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be in [1, %d]", kCandCap / 2);
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  const bool ivf = nprobe > 0;
  if (ivf ? ix->kind != INDEX_IVF : (ix->kind != INDEX_FLAT_F32 && ix->kind != INDEX_FLAT_I8))
    return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION,
                "the sharded search covers flat fp32 and int8 indexes (vsk_search_sharded) and IVF indexes (vsk_ivf_search_sharded)");
  if (qmasks && !((ix->kind == INDEX_FLAT_F32 || ix->kind == INDEX_IVF) && ix->has_masks))
    return fail(ctx, VSK_ERR_INVALID_INPUT, "query masks given but the index has no row masks");
  auto whole_local_search = [&](float* d, int64_t* i) -> int32_t {
    return ivf ? ivf_search_dev_entry(ix, q, nq, k, nprobe, qmasks, d, i) : flat_search_dev_entry(ix, q, nq, k, qmasks, d, i);
  };
  const int what = layout & 15;
  if (what != VSK_SHARDED_SLICE && what != VSK_SHARDED_ALL) return fail(ctx, VSK_ERR_INVALID_INPUT, "unknown result layout %d", what);
  if (!cm || cm->nranks == 1) {
    // one shard: the plain search is the whole answer, and every layout is the same
    return whole_local_search(out_dist, out_ids);
  }
  const NcclApi* api = nccl_api();
  if (!api) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "NCCL is not available");
  if (ix->id_base < 0 || ix->id_base + ix->n > 0xffffffffLL)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "global rows must fit 32 bits for the sharded search (id base %lld + %lld rows)",
                (long long)ix->id_base, (long long)ix->n);
  const int G = cm->nranks;
  if ((int64_t)G * k > kCandCap) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "ranks x k must not exceed %d", kCandCap);
  const int64_t per = ceil_div(nq, G), padded = per * G;
  int64_t first, count;
  slice_of(nq, G, cm->rank, &first, &count);

  void* p;
  VSK_TRY(scratch(ctx, SLOT_SH_D, (size_t)nq * k * 4, &p));
  float* loc_d = (float*)p;
  VSK_TRY(scratch(ctx, SLOT_SH_I, (size_t)nq * k * 8, &p));
  int64_t* loc_i = (int64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_SH_SEND, (size_t)padded * k * 8, &p));
  uint64_t* send = (uint64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_SH_RECV, (size_t)padded * k * 8, &p));
  uint64_t* recv = (uint64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_SH_MERGED, (size_t)per * k * 8, &p));
  uint64_t* merged = (uint64_t*)p;
  cm->timed = ctx->profile;
  phase_mark(ctx, cm, 1);

  // ---- local search: in two halves around the bound all-reduce where the index has that form ----
  const bool split = ix->kind == INDEX_FLAT_F32 && ctx->search_path == VSK_PATH_TENSOR_RERANK &&
                     ix->metric != VSK_METRIC_MANHATTAN && nq <= 16384;
  if (split) {
    VSK_TRY(scratch(ctx, SLOT_SH_BOUND, (size_t)nq * 4, &p));
    float* bound = (float*)p;
    float* qnorm = nullptr;
    if (ix->metric == VSK_METRIC_COSINE) {
      VSK_TRY(scratch(ctx, SLOT_QNORM, (size_t)nq * sizeof(float), &p));
      qnorm = (float*)p;
      VSK_TRY(launch_row_norms(ctx, q, nq, ix->dim, 0, qnorm));
    }
    ctx->stats.searches++;
    ctx->stats.queries += nq;
    const int64_t na = tensor_lane_split(ctx, nq);
    if (na == 0) {
      VSK_TRY(tensor_search_begin(ix, q, nq, k, qnorm, qmasks, G, bound));
      phase_mark(ctx, cm, 2);
      VSK_NCCL(ctx, api, api->AllReduce(bound, bound, (size_t)nq, ncclFloat32, ncclMax, cm->comm, ctx->stream));
      tl_mark(ctx, "bound_allreduce");
      phase_mark(ctx, cm, 3);
      VSK_TRY(tensor_search_finish(ix, bound, loc_d, loc_i));
    } else {
      // Two halves on two lanes.  Both lanes use the one communicator; NCCL runs its operations in the order they
      // were enqueued (the same order on every rank), whatever stream each is on.
      VSK_TRY(tensor_prepare_index(ix));
      const int64_t nb = nq - na;
      VSK_TRY(lanes_fork(ctx));
      int32_t st = VSK_OK;
      auto on_lane = [&](int lane, auto&& fn) {
        if (st != VSK_OK) return;
        LaneGuard g(ctx, lane);
        st = fn();
      };
      auto reduce = [&](float* b, int64_t n) -> int32_t {
        VSK_NCCL(ctx, api, api->AllReduce(b, b, (size_t)n, ncclFloat32, ncclMax, cm->comm, ctx->stream));
        tl_mark(ctx, "bound_allreduce");
        return VSK_OK;
      };
      on_lane(0, [&] { return tensor_search_begin(ix, q, na, k, qnorm, qmasks, G, bound); });
      on_lane(1, [&] {
        return tensor_search_begin(ix, q + na * ix->dim, nb, k, qnorm ? qnorm + na : nullptr, qmasks ? qmasks + na : nullptr, G,
                                   bound + na);
      });
      on_lane(0, [&] { return reduce(bound, na); });
      on_lane(1, [&] { return reduce(bound + na, nb); });
      on_lane(0, [&] { return tensor_search_finish_issue(ix, bound, loc_d, loc_i); });
      on_lane(1, [&] { return tensor_search_finish_issue(ix, bound + na, loc_d + na * k, loc_i + na * k); });
      const int32_t jst = lanes_join(ctx);
      cudaStreamSynchronize(ctx->stream_main);
      if (st != VSK_OK || jst != VSK_OK) {
        cudaStreamSynchronize(ctx->stream_aux);
        ctx->pending[0] = ShardPending{};
        ctx->pending[1] = ShardPending{};
        return st != VSK_OK ? st : jst;
      }
      const int32_t sa = tensor_search_finish_collect(ix, 0);
      const int32_t sb = tensor_search_finish_collect(ix, 1);
      if (sa != VSK_OK) return sa;
      if (sb != VSK_OK) return sb;
    }
  } else {
    phase_mark(ctx, cm, 2);
    phase_mark(ctx, cm, 3);
    VSK_TRY(whole_local_search(loc_d, loc_i));
  }

  // ---- exchange and merge: this rank's slice of the queries ----
  VSK_TRY(launch_pack_keys(ctx, loc_d, loc_i, nq, padded, k, send));
  phase_mark(ctx, cm, 4);
  VSK_TRY(exchange_keys(ctx, api, cm, send, recv, per, k));
  phase_mark(ctx, cm, 5);
  VSK_TRY(launch_merge_keys(ctx, recv, G, per, per, k, merged));
  phase_mark(ctx, cm, 6);
  if (what == VSK_SHARDED_SLICE) {
    VSK_TRY(launch_unpack_keys(ctx, merged, count * k, out_dist, out_ids));
  } else {
    VSK_TRY(scratch(ctx, SLOT_SH_ALL, (size_t)padded * k * 8, &p));
    uint64_t* all = (uint64_t*)p;
    VSK_NCCL(ctx, api, api->AllGather(merged, all, (size_t)per * k, ncclUint64, cm->comm, ctx->stream));
    VSK_TRY(launch_unpack_keys(ctx, all, nq * k, out_dist, out_ids));
  }
  phase_mark(ctx, cm, 7);
  return VSK_OK;
}

static void collect_phases(Comm* cm) {
  if (!cm || !cm->timed) return;
  for (int p = 0; p < VSK_SHARDED_PHASES; ++p) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, cm->ev[p], cm->ev[p + 1]) != cudaSuccess) {
      cudaGetLastError();
      ms = 0.f;
    }
    cm->phase_ms[p] = ms;
  }
}

}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_comm_unique_id(void* id_bytes) {
  if (!id_bytes) return VSK_ERR_INVALID_INPUT;
  static_assert(sizeof(ncclUniqueId) == VSK_COMM_ID_BYTES, "ncclUniqueId is 128 bytes");
  const NcclApi* api = nccl_api();
  if (!api) return VSK_ERR_EXECUTION_FAILED;
  ncclUniqueId id;
  if (api->GetUniqueId(&id) != ncclSuccess) return VSK_ERR_EXECUTION_FAILED;
  memcpy(id_bytes, &id, sizeof(id));
  return VSK_OK;
}

int32_t vsk_comm_init(vsk_ctx* c, int32_t nranks, int32_t rank, const void* id_bytes) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  if (nranks <= 0 || rank < 0 || rank >= nranks) return fail(ctx, VSK_ERR_INVALID_INPUT, "rank %d of %d", rank, nranks);
  if (ctx->comm) return fail(ctx, VSK_ERR_INVALID_INPUT, "the context already has a communicator");
  Comm* cm = new Comm();
  cm->nranks = nranks;
  cm->rank = rank;
  for (auto& e : cm->ev)
    if (cudaEventCreate(&e) != cudaSuccess) {
      cudaGetLastError();
      for (auto& d : cm->ev)
        if (d) cudaEventDestroy(d);
      delete cm;
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "could not create timing events");
    }
  if (nranks > 1) {
    if (!id_bytes) {
      ctx->comm = cm;
      comm_release(ctx);
      return fail(ctx, VSK_ERR_INVALID_INPUT, "null communicator id");
    }
    const NcclApi* api = nccl_api();
    if (!api) {
      ctx->comm = cm;
      comm_release(ctx);
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "libnccl.so.2 could not be loaded: %s", dlerror());
    }
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    const ncclResult_t r = api->CommInitRank(&cm->comm, nranks, id, rank);
    if (r != ncclSuccess) {
      cm->comm = nullptr;
      ctx->comm = cm;
      comm_release(ctx);
      return fail(ctx, VSK_ERR_EXECUTION_FAILED, "ncclCommInitRank failed: %s", api->GetErrorString(r));
    }
  }
  ctx->comm = cm;
  return VSK_OK;
}

int32_t vsk_comm_destroy(vsk_ctx* c) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream_main);
  cudaStreamSynchronize(ctx->stream_aux);
  comm_release(ctx);
  return VSK_OK;
}

int32_t vsk_comm_info(vsk_ctx* c, int32_t* nranks, int32_t* rank) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx) return VSK_ERR_INVALID_INPUT;
  if (nranks) *nranks = ctx->comm ? ctx->comm->nranks : 1;
  if (rank) *rank = ctx->comm ? ctx->comm->rank : 0;
  return VSK_OK;
}

void vsk_sharded_slice(int64_t nq, int32_t nranks, int32_t rank, int64_t* first, int64_t* count) {
  int64_t f = 0, c = 0;
  if (nq > 0 && nranks > 0 && rank >= 0 && rank < nranks) slice_of(nq, nranks, rank, &f, &c);
  if (first) *first = f;
  if (count) *count = c;
}

static int32_t sharded_dev_entry(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, int32_t layout,
                                 float* out_dist, int64_t* out_ids, int32_t nprobe) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (ctx->comm) {
    ctx->comm->timed = ctx->profile;
    if (ctx->comm->timed) {
      cudaEventRecord(ctx->comm->ev[0], ctx->stream_main);
    }
  }
  VSK_TRY(search_sharded_dev(ix, q, nq, k, qmasks, layout, out_dist, out_ids, nprobe));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream_main));
  collect_phases(ctx->comm);
  return VSK_OK;
}

static int32_t sharded_host_entry(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, int32_t layout,
                                  float* out_dist, int64_t* out_ids, int32_t nprobe) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  Ctx* ctx = ix->ctx;
  cudaSetDevice(ctx->device);
  if (nq <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no queries");
  if (k <= 0) return fail(ctx, VSK_ERR_INVALID_INPUT, "k must be positive");
  if (!q || !out_dist || !out_ids) return fail(ctx, VSK_ERR_INVALID_INPUT, "null pointer");
  Comm* cm = ctx->comm;
  const int G = cm ? cm->nranks : 1, r = cm ? cm->rank : 0;
  const int64_t per = ceil_div(nq, G), padded = per * G;
  int64_t first, count;
  slice_of(nq, G, r, &first, &count);
  const int dim = ix->dim;
  void *dq, *dd, *di, *dm = nullptr;
  VSK_TRY(scratch(ctx, SLOT_Q, (size_t)padded * dim * 4, &dq));
  VSK_TRY(scratch(ctx, SLOT_OUT_D, (size_t)nq * k * 4, &dd));
  VSK_TRY(scratch(ctx, SLOT_OUT_I, (size_t)nq * k * 8, &di));
  if (cm) {
    cm->timed = ctx->profile;
    if (cm->timed) cudaEventRecord(cm->ev[0], ctx->stream_main);
  }
  if ((layout & VSK_SHARDED_QUERIES_SPLIT) && G > 1) {
    // every rank holds the same host queries: this rank sends its 1/G of them over PCIe, NVLink does the rest
    const NcclApi* api = nccl_api();
    if (!api) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "NCCL is not available");
    float* part = (float*)dq + (size_t)r * per * dim;
    if (count > 0)
      VSK_CUDA(ctx, cudaMemcpyAsync(part, q + (size_t)first * dim, (size_t)count * dim * 4, cudaMemcpyHostToDevice, ctx->stream));
    VSK_NCCL(ctx, api, api->AllGather(part, dq, (size_t)per * dim, ncclFloat32, cm->comm, ctx->stream));
    ctx->stats.h2d_bytes += count * dim * 4;
  } else {
    VSK_CUDA(ctx, cudaMemcpyAsync(dq, q, (size_t)nq * dim * 4, cudaMemcpyHostToDevice, ctx->stream));
    ctx->stats.h2d_bytes += nq * dim * 4;
  }
  if (qmasks) {
    VSK_TRY(scratch(ctx, SLOT_QMASK, (size_t)nq * 8, &dm));
    VSK_CUDA(ctx, cudaMemcpyAsync(dm, qmasks, (size_t)nq * 8, cudaMemcpyHostToDevice, ctx->stream));
    ctx->stats.h2d_bytes += nq * 8;
  }
  VSK_TRY(search_sharded_dev(ix, (const float*)dq, nq, k, (const uint64_t*)dm, layout, (float*)dd, (int64_t*)di, nprobe));
  const int64_t outn = ((layout & 15) == VSK_SHARDED_SLICE && G > 1) ? count : nq;
  if (outn > 0) {
    VSK_CUDA(ctx, cudaMemcpyAsync(out_dist, dd, (size_t)outn * k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(out_ids, di, (size_t)outn * k * 8, cudaMemcpyDeviceToHost, ctx->stream));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.d2h_bytes += outn * k * 12;
  collect_phases(cm);
  return VSK_OK;
}

int32_t vsk_search_sharded_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, int32_t layout,
                               float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_search_sharded_dev");
  return sharded_dev_entry(i, q, nq, k, qmasks, layout, out_dist, out_ids, 0);
}

int32_t vsk_search_sharded(vsk_index* i, const float* q, int64_t nq, int32_t k, const uint64_t* qmasks, int32_t layout,
                           float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_search_sharded");
  return sharded_host_entry(i, q, nq, k, qmasks, layout, out_dist, out_ids, 0);
}

int32_t vsk_ivf_search_sharded_dev(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                                   int32_t layout, float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search_sharded_dev");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  if (nprobe <= 0) return fail(ix->ctx, VSK_ERR_INVALID_INPUT, "nprobe must be positive");
  return sharded_dev_entry(i, q, nq, k, qmasks, layout, out_dist, out_ids, nprobe);
}

int32_t vsk_ivf_search_sharded(vsk_index* i, const float* q, int64_t nq, int32_t k, int32_t nprobe, const uint64_t* qmasks,
                               int32_t layout, float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk_ivf_search_sharded");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  if (nprobe <= 0) return fail(ix->ctx, VSK_ERR_INVALID_INPUT, "nprobe must be positive");
  return sharded_host_entry(i, q, nq, k, qmasks, layout, out_dist, out_ids, nprobe);
}

int32_t vsk_sharded_phase_ms(vsk_ctx* c, float* ms) {
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !ms) return VSK_ERR_INVALID_INPUT;
  for (int p = 0; p < VSK_SHARDED_PHASES; ++p) ms[p] = ctx->comm ? ctx->comm->phase_ms[p] : 0.f;
  return VSK_OK;
}

}  // extern "C"
