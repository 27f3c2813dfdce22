/*
 * vsk_cuda.h — C ABI of the B200 (sm_100a) similarity-search library.
 *
 * This is the boundary a VectorStoreKit host binds instead of its Metal
 * acceleration layer.  Every entry point names the reference interface it
 * replaces (paths are relative to the VectorStoreKit source tree).
 *
 * Conventions
 *   - All functions return a vsk_status (int32_t); VSK_OK == 0.  No C++ types
 *     and no exceptions cross the boundary.  vsk_last_error() gives the text
 *     of the most recent failure on a context.
 *   - Matrices are dense row-major fp32 (`rows[n*dim + i]`), the layout the
 *     reference flattens into before every dispatch
 *     (Acceleration/MetalAccelerationEngine.swift:393-405).
 *   - Host-pointer calls copy in/out during the call and never keep a host
 *     pointer.  `_dev` calls take pointers to memory of the context's GPU and
 *     run on the context's stream; they return after the stream has drained.
 *   - Row ids are dense int64 insertion indices (the host keeps the
 *     index -> VectorID(String) table, as Indexes/IVFIndex.swift:104-111 does).
 *     Missing results (fewer than k eligible rows) have id -1, distance +inf.
 *   - Results per query are ascending by distance, ties by id.
 *   - A context is used by one thread at a time (the reference serialises
 *     through an actor); distinct contexts are independent.
 *   - There is no CPU path: without a CUDA device vsk_open fails with
 *     VSK_ERR_DEVICE_NOT_AVAILABLE.
 */
#ifndef VSK_CUDA_H_
#define VSK_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  Mirrors MetalComputeError (Acceleration/Metal/MetalErrors.swift:10-39)
 * and IVFError (Indexes/IVFIndex.swift:619-637). */
typedef enum vsk_status {
  VSK_OK = 0,
  VSK_ERR_DEVICE_NOT_AVAILABLE = 1,      /* deviceNotAvailable */
  VSK_ERR_OUT_OF_MEMORY = 2,             /* deviceOutOfMemory(required, available) */
  VSK_ERR_UNSUPPORTED_OPERATION = 3,     /* unsupportedOperation: metric outside the four */
  VSK_ERR_INVALID_BUFFER_SIZE = 4,       /* invalidBufferSize */
  VSK_ERR_EXECUTION_FAILED = 5,          /* commandBufferExecutionFailed */
  VSK_ERR_TIMEOUT = 6,                   /* commandBufferTimeout: a bounded device wait ran out */
  VSK_ERR_INVALID_INPUT = 7,             /* invalidInput */
  VSK_ERR_DIMENSION_MISMATCH = 8,        /* dimensionMismatch */
  VSK_ERR_EMPTY_INPUT = 9,               /* emptyInput (MetalDistanceCompute.swift:51-53) */
  VSK_ERR_NOT_TRAINED = 10,              /* IVFError.notTrained */
  VSK_ERR_INSUFFICIENT_TRAINING_DATA = 11,/* IVFError.insufficientTrainingData */
  VSK_ERR_IMPORT_FAILED = 12,            /* ImportError.decodingFailed (Indexes/IVFIndex.swift:640-643), VectorStoreError.importError */
  VSK_ERR_EXPORT_FAILED = 13             /* VectorStoreError.exportError (Core/Errors.swift:661-680) */
} vsk_status;

/* The four cases of DistanceMetric the accelerated path supports
 * (Core/SearchTypes.swift:105-118; MetalDistanceCompute.swift:342-344 rejects the rest).
 *   euclidean   sqrt(sum (q-x)^2)            cosine      1 - q.x/(|q||x| + 1e-8)
 *   dotProduct  -(q.x)                        manhattan   sum |q-x|
 * (Acceleration/AccelerateOptimizer.swift:251-383, Shaders/DistanceShaders.metal:62-218) */
typedef enum vsk_metric {
  VSK_METRIC_EUCLIDEAN = 0,
  VSK_METRIC_COSINE = 1,
  VSK_METRIC_DOT_PRODUCT = 2,
  VSK_METRIC_MANHATTAN = 3
} vsk_metric;

typedef enum vsk_sq8_mode {
  VSK_SQ8_GLOBAL = 0,  /* one min/max over all values: ScalarQuantizer.swift:389-418 */
  VSK_SQ8_PER_DIM = 1  /* the same formulas column by column */
} vsk_sq8_mode;

/* Which kernels a flat fp32 search runs. */
typedef enum vsk_search_path {
  VSK_PATH_TENSOR_RERANK = 0, /* fp16 tcgen05 contraction + bounded-error filter + exact fp32 rerank;
                                 queries whose result cannot be certified exact are re-run on the
                                 fp32 scan.  Manhattan always uses the fp32 scan. */
  VSK_PATH_FP32_SCAN = 1      /* direct fp32 formulas on CUDA cores for every pair */
} vsk_search_path;

typedef struct vsk_ctx vsk_ctx;
typedef struct vsk_index vsk_index;

/* Capabilities of the opened device.  Stands in for the CapabilitiesType of the reference's
 * ComputeAccelerator strategies (API/Strategies/AcceleratorStrategies.swift:437-455). */
typedef struct vsk_device_info {
  int32_t device;
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  int64_t hbm_bytes;
  int64_t l2_bytes;
  int32_t max_smem_per_block;
  char name[128];
} vsk_device_info;

/* Counters since vsk_open.  Stands in for MetalAccelerationEngine.getPerformanceStatistics()
 * (Acceleration/MetalAccelerationEngine.swift:987-998). */
typedef struct vsk_stats {
  int64_t searches;            /* search calls */
  int64_t queries;             /* queries answered */
  int64_t kernel_launches;     /* kernels of this library launched */
  int64_t tensor_tiles;        /* tcgen05 output tiles computed */
  int64_t reranked_rows;       /* rows re-scored by the exact rerank */
  int64_t fallback_queries;    /* queries re-run on the fp32 scan after a failed certificate */
  int64_t h2d_bytes, d2h_bytes;
  int64_t scan_kernel_launches; /* with vsk_profile on: launches of the dominant scan kernels ... */
  double scan_kernel_ms;        /* ... and their summed device time (CUDA events on the stream) */
} vsk_stats;

/* What a handle holds (vsk_index_info_get); a loaded index image is described the same way. */
typedef enum vsk_index_kind { VSK_INDEX_FLAT_F32 = 0, VSK_INDEX_FLAT_I8 = 1, VSK_INDEX_IVF = 2, VSK_INDEX_PQ = 3 } vsk_index_kind;
typedef struct vsk_index_info {
  int32_t kind;        /* vsk_index_kind */
  int32_t metric;      /* vsk_metric */
  int32_t dimensions;
  int32_t nlist;       /* IVF lists, else 0 */
  int64_t count;       /* rows */
  int64_t id_base;
  int32_t has_masks;   /* rows carry 64-bit filter masks */
  int32_t pq_segments;       /* product-quantised index: segments, else 0 */
  int32_t pq_codebook_size;  /* ... codewords per segment */
  int32_t reserved;
} vsk_index_info;

/* Tuning of the search schedule, per context (vsk_tuning_get / vsk_tuning_set).  The defaults are what the
 * library was measured with; the fields exist for experiments and for hosts that know their workload.  Stands in
 * for the reference's AccelerationConfiguration (Acceleration/MetalAccelerationEngine.swift:1025-1049). */
typedef struct vsk_tuning {
  int32_t fold_row_term;        /* 1: euclidean contractions up to d = 256 carry |x|^2 inside the operands */
  int32_t chunk_growth;         /* 3: a chunk of the flat tensor-path scan is at most this multiple of the rows seen
                                   (batches of up to 2 048 queries, which are bound by their launches, use at least 16) */
  int32_t dense_rows;           /* 0 = automatic; rows of the first (unfiltered) chunk otherwise */
  int32_t ivf_pilot_tiles;      /* 4: 256-row tiles of the nearest list that set an IVF query's first threshold */
  int32_t stream_scan;          /* 1: batches of up to eight queries stream the rows instead of padding a tile */
  int32_t overlap_min_queries;  /* 0 = never; otherwise tensor-path batches of at least this many queries run as
                                   two halves on two streams (one half's selection, re-scoring and exchange under
                                   the other's contraction).  Off by default: on one power-capped GPU the two
                                   halves were measured to slow each other down by what the overlap gains. */
  int32_t wait_limit_log2;      /* 0 = default (23): a pipeline wait inside the contraction kernel gives up after
                                   2^this polls (tens of nanoseconds each) and the call returns VSK_ERR_TIMEOUT,
                                   the counterpart of commandBufferTimeout (Acceleration/Metal/MetalErrors.swift:30) */
  int32_t test_stall_scan;      /* testing only: 1 makes the next contraction launch leave one operand stage
                                   unfilled, so that a bounded wait runs out; resets itself to 0 */
  int32_t assign_stages;        /* measurement only: 0 = the k-means assignment kernel's operand ring holds a whole
                                   data tile per stage, as many stages as fit (fold columns as a 16-column tile where
                                   they begin a K block of their own); n > 0 = stages of one K block, at most n */
  int32_t stage_kblocks;        /* K blocks (64 operand columns) per stage of the contraction kernel's operand ring: 1 =
                                   four stages of 48 KB, 2 = two stages of 96 KB (half the hand-overs per tile) */
  int32_t reserved[6];
} vsk_tuning;

/* --- context ------------------------------------------------------------------------------
 * Replaces ComputeAccelerator.initialize()/capabilities() (Core/Protocols.swift:11-20) and the
 * process-wide MetalAccelerationEngine.shared (MetalAccelerationEngine.swift:25-30). */
int32_t vsk_open(int32_t device, vsk_ctx** out_ctx);
int32_t vsk_close(vsk_ctx* ctx);
int32_t vsk_device_info_get(vsk_ctx* ctx, vsk_device_info* out);
int32_t vsk_stats_get(vsk_ctx* ctx, vsk_stats* out);
const char* vsk_last_error(vsk_ctx* ctx);
const char* vsk_status_string(int32_t status);
/* vsk_search_path; default VSK_PATH_TENSOR_RERANK. */
int32_t vsk_set_search_path(vsk_ctx* ctx, int32_t path);
/* Time the scan kernels (tcgen05 contraction, fp32 tile scan, IVF list scan) with CUDA events on the
 * context's stream; totals appear in vsk_stats.  Stands in for MetalProfiler's per-operation timing
 * (Acceleration/Metal/MetalProfiler.swift:74-110). */
int32_t vsk_profile(vsk_ctx* ctx, int32_t enable);
/* Event log of the next calls on this context: one CUDA event after each scan, selection, re-scoring and exchange,
 * on the stream it was enqueued on.  vsk_timeline_read drains both streams, writes one line per event - "<lane>
 * <what> <milliseconds since the log was switched on or last read>" - into `text` (at most `capacity` bytes,
 * NUL-terminated), clears the log and returns the bytes written (-1 on bad arguments).  Shows how the two halves of
 * a large batch overlap.  Stands in for MetalProfiler's event log (Acceleration/Metal/MetalProfiler.swift:74-110). */
int32_t vsk_timeline(vsk_ctx* ctx, int32_t enable);
int64_t vsk_timeline_read(vsk_ctx* ctx, char* text, int64_t capacity);
/* The CUDA stream (cudaStream_t) every call on this context is enqueued on. */
void* vsk_stream(vsk_ctx* ctx);
/* Rows of the next chunk of the search schedule after `seen` rows, for candidate lists compacted to `keep` keys
 * (1 <= keep <= 2048), at re-run level 0 - 2; -1 for arguments outside that range.  Host arithmetic only (needs no
 * device): the schedule advances by this many rows, so it is positive for every valid input. */
int64_t vsk_schedule_chunk(int64_t seen, int32_t keep, int32_t level);
/* Measured ceilings of this GPU for the scans that neither HBM nor the tensor cores bound (a few milliseconds of
 * a synthetic kernel on the context's stream, best of five, CUDA events):
 *   VSK_PEAK_FP32_ISSUE   FP32 instructions per second, counted per thread (the Manhattan scan's bound)
 *   VSK_PEAK_SMEM_GATHER  4-byte shared-memory words per second at random addresses (the product-quantised scan's)
 *   VSK_PEAK_TMEM_READ    bytes per second read out of tensor memory by tcgen05.ld (the bound of contractions with a
 *                         short inner dimension: every accumulator is read once, 4 bytes per (row, centroid) pair)
 * The reference has no counterpart; its thread-configuration benchmark is the nearest relative
 * (Acceleration/Metal/MetalThreadConfigurationOptimizer.swift:430-440). */
typedef enum vsk_peak { VSK_PEAK_FP32_ISSUE = 0, VSK_PEAK_SMEM_GATHER = 1, VSK_PEAK_TMEM_READ = 2 } vsk_peak;
int32_t vsk_measure_peak(vsk_ctx* ctx, int32_t what, double* per_second);
/* The checked build variant (libvsk_cuda_checked.so, `python -m vectorstorekit_b200.build --checked`): every global
 * load, store and atomic of every kernel is range-tested against the device buffers the library allocated (with the
 * sizes the calls asked for) and the buffers the caller announced; an access outside them, or one not aligned to its
 * own size, is diverted to a sink and counted instead of being executed - no trap, the context stays usable.  It is
 * what Metal's shader validation layer is to the reference and what compute-sanitizer is to CUDA where that tool can
 * run.  In the normal library these calls exist and do nothing (vsk_checked_build returns 0).
 *   vsk_checked_register    announce a caller-owned device buffer that `_dev` entry points will be given
 *   vsk_checked_faults      out3 = {refused accesses since the last call, first refused address,
 *                           its size in bytes | write << 8 | misaligned << 9}; waits for the context's streams
 *   vsk_checked_selftest    reads one word past the announced end of a buffer of the library's own (the memory behind
 *                           it is valid): an instrumented build records exactly one refused access */
int32_t vsk_checked_build(void);
int32_t vsk_checked_register(const void* device_ptr, int64_t bytes);
int32_t vsk_checked_unregister(const void* device_ptr);
int32_t vsk_checked_faults(vsk_ctx* ctx, uint64_t* out3);
int32_t vsk_checked_selftest(vsk_ctx* ctx);

int32_t vsk_tuning_get(vsk_ctx* ctx, vsk_tuning* out);
int32_t vsk_tuning_set(vsk_ctx* ctx, const vsk_tuning* in);

/* --- stateless distances -------------------------------------------------------------------
 * Full nq x nx matrix, out[q*nx + c].  Replaces MetalAccelerationEngine.batchComputeDistances
 * with topK == nil (MetalAccelerationEngine.swift:139-204,377-478), MetalDistanceCompute
 * .batchComputeDistances (Metal/MetalDistanceCompute.swift:260-318) and, with nq == 1,
 * computeDistances (MetalAccelerationEngine.swift:76-136). */
int32_t vsk_batch_distances(vsk_ctx* ctx, int32_t metric, const float* queries, int64_t nq,
                            const float* rows, int64_t nx, int32_t dim, float* out);
int32_t vsk_batch_distances_dev(vsk_ctx* ctx, int32_t metric, const float* queries, int64_t nq,
                                const float* rows, int64_t nx, int32_t dim, float* out);

/* --- flat exact k-NN -----------------------------------------------------------------------
 * A resident database searched by many query batches.  Replaces
 * MetalAccelerationEngine.batchComputeDistances(queries:candidates:metric:topK:)
 * (MetalAccelerationEngine.swift:139-204), which re-uploads the candidates on every call and
 * sorts on the CPU (:465-471), and the flat scan of InMemoryVectorStore.search
 * (LLM/LLMVectorStore.swift:83-114).  `masks` (may be NULL) gives each row a 64-bit metadata
 * bitmask; a search with query masks keeps row r for query q iff (masks[r] & qmasks[q]) != 0,
 * applied before distances as the reference's filters are (Indexes/IVFIndex.swift:163-172). */
int32_t vsk_flat_create(vsk_ctx* ctx, int32_t metric, int32_t dim, vsk_index** out_index);
int32_t vsk_flat_add_f32(vsk_index* index, const float* rows, int64_t n, const uint64_t* masks);
int32_t vsk_flat_add_f32_dev(vsk_index* index, const float* rows, int64_t n, const uint64_t* masks);
int32_t vsk_index_destroy(vsk_index* index);
int64_t vsk_index_size(vsk_index* index);
/* Added to every returned id (row-sharded databases: the shard's first global row). */
int32_t vsk_index_set_id_base(vsk_index* index, int64_t id_base);

int32_t vsk_index_info_get(vsk_index* index, vsk_index_info* out);

/* --- index image (export / import) -----------------------------------------------------------
 * Replaces VectorIndex.export(format: .binary) -> Data / import(data:format:) (Core/Protocols.swift:157-160;
 * Indexes/IVFIndex.swift:297-326) and the store envelope of VectorStore.combineExport
 * (API/VectorStore.swift:707-727): "VSTR", version bytes 1,0,0,0, u64 metadata length, JSON metadata, index data.
 * Unlike the reference's IVF export (centroids only, IVFIndex.swift:612-616) the image carries the rows, the
 * inverted lists, masks and quantiser parameters, so a loaded index answers searches identically.  Each data
 * section carries a 64-bit checksum computed on the GPU; a mismatch on load gives VSK_ERR_IMPORT_FAILED.
 * vsk_index_image_size gives the exact byte count vsk_index_export writes.  save/load stream through two
 * 32 MiB pinned buffers and never hold the whole image in host memory. */
int32_t vsk_index_image_size(vsk_index* index, int64_t* bytes);
int32_t vsk_index_export(vsk_index* index, void* dst, int64_t capacity, int64_t* written);
int32_t vsk_index_import(vsk_ctx* ctx, const void* src, int64_t bytes, vsk_index** out_index);
int32_t vsk_index_save(vsk_index* index, const char* path);
int32_t vsk_index_load(vsk_ctx* ctx, const char* path, vsk_index** out_index);

/* out_dist[nq*k], out_ids[nq*k].  qmasks may be NULL.  nq = 1 is VectorStore.search (one query).  Routing of a
 * flat fp32 index: euclidean, cosine and dot-product batches (with or without masks) take the tensor-core path
 * on the default search path; Manhattan batches and VSK_PATH_FP32_SCAN take the fp32 tile, where a batch of one to
 * eight queries streams every row it may see from HBM once instead of padding a query tile. */
int32_t vsk_search(vsk_index* index, const float* queries, int64_t nq, int32_t k,
                   const uint64_t* qmasks, float* out_dist, int64_t* out_ids);
int32_t vsk_search_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k,
                       const uint64_t* qmasks, float* out_dist, int64_t* out_ids);

/* The asynchronous form.  The reference's batch call commits a command buffer and resumes its caller from the
 * buffer's completion handler (MetalAccelerationEngine.swift:139-204, :444-449; MetalDistanceCompute.swift:365-375).
 * These calls return at once; the search runs on the context's worker thread, in submission order, and
 * done(user, status) is then called FROM THAT THREAD with the results complete in out_dist / out_ids (host memory for
 * vsk_search_async, device memory with the stream drained for vsk_search_dev_async).  Every buffer stays valid until
 * the callback.  Between a submission and its callback the context belongs to the worker: no other call on the
 * context or its indices except further *_async submissions and vsk_wait.  A status other than VSK_OK from the
 * submission itself means nothing was queued and `done` will not be called.
 * vsk_wait blocks until nothing is queued or running and returns the first failing status since the previous
 * vsk_wait (VSK_OK if none); vsk_last_error then holds its message.  vsk_close waits for queued work too. */
typedef void (*vsk_done_fn)(void* user, int32_t status);
int32_t vsk_search_async(vsk_index* index, const float* queries, int64_t nq, int32_t k, const uint64_t* qmasks,
                         float* out_dist, int64_t* out_ids, vsk_done_fn done, void* user);
int32_t vsk_search_dev_async(vsk_index* index, const float* queries, int64_t nq, int32_t k, const uint64_t* qmasks,
                             float* out_dist, int64_t* out_ids, vsk_done_fn done, void* user);
int32_t vsk_wait(vsk_ctx* ctx);

/* A shard's search in two halves, for a host that spreads the rows of one database over several GPUs
 * (the multi-GPU form of VectorStore.batchSearch; the reference has no sharded search).
 *   begin:  scans this shard.  bound[q] (device, nq floats) receives a value that this shard's ceil(k / shards)
 *           best rows do not exceed, or +inf when nothing is known (shorter shards, index kinds and search paths
 *           that have no split form).  The units depend on the query only, so the values of one query are
 *           comparable between shards.
 *   host:   element-wise MAXIMUM of `bound` over the shards (one all-reduce): at least k rows of the whole
 *           database lie at or below it.
 *   finish: with the reduced bound, returns this shard's rows among its k best that can still belong to the
 *           overall k best (others are padded with +inf / -1), in the layout of vsk_search_dev.
 * `begin` returns while its kernels still run on the context's stream (vsk_stream): do the reduction on that stream
 * or synchronise it first; `finish` returns with the results complete.
 * The queries, k and the bound buffer of `begin` must stay valid until `finish`, and no other call may be made on
 * the index's context in between.  At most 16 384 queries per call.  Flat fp32 indexes without query masks. */
int32_t vsk_search_shard_begin_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k,
                                   int32_t shards, float* bound);
int32_t vsk_search_shard_finish_dev(vsk_index* index, const float* bound, float* out_dist, int64_t* out_ids);

/* Merge of per-shard results: `g` lists of k (distance, global id) per query, laid out
 * [g][nq][k], into the k best per query by (distance, id) — what one unsharded search returns.
 * Equal distances are ordered by (list, position): give the lists in ascending order of their shards' first
 * global row, each ascending by (distance, id), and that is the (distance, id) order.
 * Device pointers.  The reference has no sharded search; this is the step after the NCCL gather. */
int32_t vsk_merge_topk_dev(vsk_ctx* ctx, const float* dist, const int64_t* ids, int32_t g,
                           int64_t nq, int32_t k, float* out_dist, int64_t* out_ids);

/* --- row-sharded search over several GPUs (one process and one context per GPU) -------------------
 * The database's rows are spread over `nranks` GPUs: rank g's index holds rows [g*N/G, (g+1)*N/G) and its id base
 * (vsk_index_set_id_base) is its first global row.  The reference has no multi-device search; its hosts await one
 * call (MetalAccelerationEngine.batchComputeDistances, Acceleration/MetalAccelerationEngine.swift:139-204,444-449),
 * and so do these.  Collectives are NCCL (libnccl.so.2, loaded when vsk_comm_init is first called; the library has
 * no link-time dependency on it), enqueued on the context's streams; no kernel of this library reads another GPU's
 * memory.
 *   vsk_comm_unique_id  fills 128 bytes (an ncclUniqueId) on ONE rank; the host hands the same bytes to every rank
 *   vsk_comm_init       joins the communicator (every rank calls it, same id, its own rank); collective
 *   vsk_comm_destroy    leaves it (vsk_close does this too)
 *   vsk_search_sharded_dev
 *       Every rank passes the SAME queries (device, [nq][dim]) and k.  Each rank scans its shard; the shards agree on a
 *       per-query bound (one all-reduce of nq floats) so that a shard re-scores only rows that can reach the overall
 *       top-k; the per-shard lists travel as packed 64-bit (distance, global row) keys in ONE all-to-all, so that
 *       rank g receives every shard's lists for its slice of the queries and merges them: ties by global row, what
 *       an unsharded search returns.  Global rows must fit 32 bits (id base + rows <= 2^32 - 1).
 *       layout VSK_SHARDED_SLICE: rank g gets the merged results of queries [first, first + count) (vsk_sharded_slice)
 *                                 at the start of out_dist / out_ids (count * k entries).  No further exchange.
 *       layout VSK_SHARDED_ALL:   an all-gather hands every rank all nq * k results.
 *   vsk_search_sharded  the same with host pointers.  With VSK_SHARDED_QUERIES_SPLIT (flag, or-ed into layout) a
 *       rank copies only its 1/nranks of the host queries to its GPU and an all-gather over NVLink distributes
 *       them (all ranks hold the same host queries; saves PCIe traffic).  Results land in host memory in the
 *       chosen layout.
 * Flat fp32 and int8 indexes; query masks may be NULL. */
enum { VSK_COMM_ID_BYTES = 128 };
typedef enum vsk_sharded_layout { VSK_SHARDED_SLICE = 0, VSK_SHARDED_ALL = 1, VSK_SHARDED_QUERIES_SPLIT = 16 } vsk_sharded_layout;
int32_t vsk_comm_unique_id(void* id_bytes);
int32_t vsk_comm_init(vsk_ctx* ctx, int32_t nranks, int32_t rank, const void* id_bytes);
int32_t vsk_comm_destroy(vsk_ctx* ctx);
/* ranks and this rank of the context's communicator (1, 0 without one) */
int32_t vsk_comm_info(vsk_ctx* ctx, int32_t* nranks, int32_t* rank);
/* the queries whose merged results rank `rank` of `nranks` returns under VSK_SHARDED_SLICE */
void vsk_sharded_slice(int64_t nq, int32_t nranks, int32_t rank, int64_t* first, int64_t* count);
int32_t vsk_search_sharded_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k, const uint64_t* qmasks,
                               int32_t layout, float* out_dist, int64_t* out_ids);
int32_t vsk_search_sharded(vsk_index* index, const float* queries, int64_t nq, int32_t k, const uint64_t* qmasks,
                           int32_t layout, float* out_dist, int64_t* out_ids);
/* The same for an IVF index whose rows are sharded: every rank holds a slice of every list (same centroids on all
 * ranks - train with vsk_kmeans_trainer_* and all-reduced sums - and vsk_index_set_id_base = the shard's first global
 * row).  Each rank probes `nprobe` lists of its shard (IVFIndex.search, Indexes/IVFIndex.swift:124-202), then the
 * exchange and the merge of vsk_search_sharded.  qmasks may be NULL. */
int32_t vsk_ivf_search_sharded_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k, int32_t nprobe,
                                   const uint64_t* qmasks, int32_t layout, float* out_dist, int64_t* out_ids);
int32_t vsk_ivf_search_sharded(vsk_index* index, const float* queries, int64_t nq, int32_t k, int32_t nprobe,
                               const uint64_t* qmasks, int32_t layout, float* out_dist, int64_t* out_ids);
/* Timing of the phases of the last vsk_search_sharded(_dev) call on this context, in milliseconds, from CUDA
 * events on the context's streams (recorded when vsk_profile is on; zeros otherwise):
 *   [0] query copy and exchange  [1] scan and compactions up to the bound  [2] bound all-reduce
 *   [3] certificate, re-scoring, final order, key packing  [4] all-to-all  [5] merge  [6] all-gather / copy out
 * A batch that ran as two halves reports the first half. */
enum { VSK_SHARDED_PHASES = 7 };
int32_t vsk_sharded_phase_ms(vsk_ctx* ctx, float* ms);

/* The tensor path's coarse values, for auditing its error bound (no counterpart in the reference).  For the first
 * `rows` rows of a flat fp32 index (rows <= 4096) and nq queries: coarse[q * rows + r] is the value the
 * contraction's filter sees (fp16 operands, fp32 accumulation on the tensor cores; the squared form for euclidean,
 * without the row-independent |q|^2), eps[q] the bound the certificate assumes on |coarse - exact|.  Device pointers. */
int32_t vsk_coarse_values_dev(vsk_index* index, const float* queries, int64_t nq, int64_t rows, float* coarse,
                              float* eps);

/* --- k-means / IVF -------------------------------------------------------------------------
 * Lloyd iterations from caller-supplied initial centroids.  Replaces KMeansClustering.cluster
 * (Clustering/KMeansClustering.swift:48-113; `.custom` initialisation :189-193) and the shader
 * kernels assign_to_centroids / accumulate_centroids / finalize_centroids
 * (Shaders/ClusteringShaders.metal:29-177).  Assignment: rooted L2, lowest index wins ties.
 * Empty cluster keeps its previous centroid (ClusteringShaders.metal:171-176).  inertia = sum of
 * un-squared distances (KMeansClustering.swift:97).  tolerance < 0: run exactly max_iters. */
int32_t vsk_kmeans(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k,
                   int32_t max_iters, float tolerance, const float* init_centroids,
                   float* centroids, int32_t* assign, float* inertia, int32_t* iters_run);
int32_t vsk_kmeans_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k,
                       int32_t max_iters, float tolerance, const float* init_centroids,
                       float* centroids, int32_t* assign, float* inertia, int32_t* iters_run);
/* k-means++ initial centroids, the reference's default initialisation (KMeansClustering.initializeKMeansPlusPlus,
 * Clustering/KMeansClustering.swift:209-260; shader compute_min_distances, Shaders/ClusteringShaders.metal:205-238).
 * The first centroid is a row drawn uniformly; each next one is drawn with the reference's weights - a row's squared
 * distance to its nearest chosen centroid divided by the SUM OF UN-SQUARED distances (:236-239; the weights do not
 * sum to one, which is kept) - the first row whose running sum exceeds a uniform draw in [0, 1), else the last row.
 * Draws come from the reference's seeded generator (a 64-bit LCG re-seeded with seed + number of centroids so far,
 * :244,480-491) mapped as Swift's standard library maps it.  centroids: [k][dim]; picked (may be NULL): the k chosen
 * row indices, host memory.  Running sums are taken in double precision by a parallel scan where the reference adds
 * floats in sequence, so a draw that lands within rounding of a row boundary may pick the neighbouring row. */
int32_t vsk_kmeans_init_plusplus(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k, uint64_t seed,
                                 float* centroids, int64_t* picked);
int32_t vsk_kmeans_init_plusplus_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k, uint64_t seed,
                                     float* centroids, int64_t* picked);
/* Lloyd iterations over rows that are spread over several GPUs (one shard per context; the reference has no
 * multi-device training).  Each iteration every shard calls step with the current centroids and gets, for its own
 * rows, the per-centroid sums [k][dim], the per-centroid row counts [k] (as floats) and the sum of its rows'
 * un-squared distances (the reference's inertia, KMeansClustering.swift:97); the caller adds these up over the
 * shards (ncclAllReduce) and calls vsk_kmeans_finish_dev, which forms the means (an empty cluster keeps its
 * centroid, Shaders/ClusteringShaders.metal:171-176).  All pointers are device pointers; `rows` must stay valid
 * while the trainer lives.  With one shard the result equals vsk_kmeans_dev's up to the order of the sums. */
typedef struct vsk_kmeans_trainer vsk_kmeans_trainer;
int32_t vsk_kmeans_trainer_create_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t k,
                                      vsk_kmeans_trainer** out_trainer);
int32_t vsk_kmeans_trainer_step_dev(vsk_kmeans_trainer* trainer, const float* centroids, float* sums, float* counts,
                                    float* inertia);
int32_t vsk_kmeans_trainer_assignments_dev(vsk_kmeans_trainer* trainer, int32_t* assign);
int32_t vsk_kmeans_trainer_destroy(vsk_kmeans_trainer* trainer);
int32_t vsk_kmeans_finish_dev(vsk_ctx* ctx, const float* sums, const float* counts, const float* prev_centroids,
                              int32_t k, int32_t dim, float* centroids);
/* Nearest centroid of every row (IVFIndex.findNearestCentroid, Indexes/IVFIndex.swift:514-527). */
int32_t vsk_assign_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim,
                       const float* centroids, int32_t k, int32_t* assign, float* dist);

/* The same result as vsk_assign_dev (device pointers, same outputs) for callers that must not allocate
 * device memory.  It has no counterpart in the reference.  Who needs it: code that places incoming rows
 * into IVF lists from inside a latency-sensitive loop, or on a GPU whose memory has been handed out in full
 * to other buffers.  cudaMalloc and cudaFree stall every stream of the device while they run and fail once
 * memory is exhausted; vsk_assign_dev may call them to grow its scratch.  This entry point calls neither,
 * nor any other allocating routine: its scratch (one 64-bit key per row) is a fixed array inside the library,
 * 8 MB that each GPU using the library keeps until the process ends.
 *   - At most 1 048 576 rows per call; more returns VSK_ERR_INVALID_BUFFER_SIZE (split the rows).
 *   - The first call on a GPU also looks up the array's device address.  Make that first call during
 *     start-up, before any stream capture is begun.
 *   - All calls on a GPU, from every context, share the one array and it keeps the last call's contents; each
 *     call re-initialises the part it uses.  Two calls whose work overlaps on the GPU race on it: run them
 *     one after the other. */
int32_t vsk_assign_static_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim,
                              const float* centroids, int32_t k, int32_t* assign, float* dist);

/* IVF index over trained centroids: rows are assigned to their nearest centroid and stored
 * list by list.  Replaces IVFIndex.train/insert (Indexes/IVFIndex.swift:397-446,80-122). */
int32_t vsk_ivf_build(vsk_ctx* ctx, const float* centroids, int32_t nlist, const float* rows,
                      int64_t n, int32_t dim, vsk_index** out_index);
int32_t vsk_ivf_build_dev(vsk_ctx* ctx, const float* centroids, int32_t nlist, const float* rows,
                          int64_t n, int32_t dim, vsk_index** out_index);
/* Row -> list of the built index (host buffer of n int32). */
int32_t vsk_ivf_assignments(vsk_index* index, int32_t* assign);
/* The index's centroids, [nlist][dim] floats to host memory (what IVFIndex.export keeps, IVFIndex.swift:297-302). */
int32_t vsk_ivf_centroids(vsk_index* index, float* centroids);
/* Probe the nprobe nearest lists, rooted L2, ascending top-k.  Replaces IVFIndex.search
 * (Indexes/IVFIndex.swift:124-202); nprobe == nlist is its `.exact` strategy (:551-560).  The reference's call is
 * the nq = 1 case; up to sixteen queries each stream the rows of their own probed lists. */
int32_t vsk_ivf_search(vsk_index* index, const float* queries, int64_t nq, int32_t k,
                       int32_t nprobe, float* out_dist, int64_t* out_ids);
int32_t vsk_ivf_search_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k,
                           int32_t nprobe, float* out_dist, int64_t* out_ids);
/* Metadata filter on the IVF path.  Replaces the `filter:` argument of IVFIndex.search
 * (Indexes/IVFIndex.swift:128,162-165,564-570): the rows of the probed lists are filtered first, then ranked.
 * vsk_ivf_set_masks gives every row of a built index a 64-bit mask, masks[i] for the i-th row in insertion order
 * (n = vsk_index_size masks); a search keeps row r for query q iff (masks[r] & qmasks[q]) != 0.  qmasks NULL = no
 * filter.  Results with fewer than k eligible rows in the probed lists are padded with id -1, distance +inf. */
int32_t vsk_ivf_set_masks(vsk_index* index, const uint64_t* masks);
int32_t vsk_ivf_set_masks_dev(vsk_index* index, const uint64_t* masks);
int32_t vsk_ivf_search_filtered(vsk_index* index, const float* queries, int64_t nq, int32_t k, int32_t nprobe,
                                const uint64_t* qmasks, float* out_dist, int64_t* out_ids);
int32_t vsk_ivf_search_filtered_dev(vsk_index* index, const float* queries, int64_t nq, int32_t k, int32_t nprobe,
                                    const uint64_t* qmasks, float* out_dist, int64_t* out_ids);
/* Appends n rows to a built index: each goes to the list of its nearest centroid, behind the rows that list already
 * holds, and gets the next insertion indices (vsk_index_size before the call, onward).  Replaces IVFIndex.insert
 * (Indexes/IVFIndex.swift:80-122), which appends one entry at a time; here only the new rows are assigned, the
 * stored rows are regrouped in one pass at copy speed, and nothing is re-trained.  masks: NULL, or one per new row
 * when the index carries masks.  A host that inserts single entries should collect them and add them in blocks. */
int32_t vsk_ivf_add(vsk_index* index, const float* rows, int64_t n, const uint64_t* masks);
int32_t vsk_ivf_add_dev(vsk_index* index, const float* rows, int64_t n, const uint64_t* masks);

/* --- int8 scalar quantiser -----------------------------------------------------------------
 * Replaces ScalarQuantizer.quantizeBatch for `.int8` (Quantization/ScalarQuantizer.swift:129-164):
 *   train   min/max -> scale = 255/(max-min), offset = -min*scale - 128     (:389-451)
 *   encode  code = truncate_toward_zero(x*scale + offset)                   (:251-270)
 *   decode  x^ = (code - offset)/scale                                      (:568-580)
 * scale/offset are arrays of `dim` floats (equal entries in VSK_SQ8_GLOBAL mode).
 * vsk_sq8_index_create accepts host or device scale/offset arrays. */
/* Per-dimension minimum and maximum of device rows into device arrays minv[dim], maxv[dim]; with a
 * row-sharded database the host reduces these across shards (min / max) before vsk_sq8_params_dev. */
int32_t vsk_sq8_minmax_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, float* minv,
                           float* maxv);
int32_t vsk_sq8_params_dev(vsk_ctx* ctx, const float* minv, const float* maxv, int32_t dim,
                           int32_t mode, float* scale, float* offset);
int32_t vsk_sq8_train(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t mode,
                      float* scale, float* offset);
int32_t vsk_sq8_encode(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim,
                       const float* scale, const float* offset, int8_t* codes);
int32_t vsk_sq8_encode_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim,
                           const float* scale, const float* offset, int8_t* codes);
int32_t vsk_sq8_decode(vsk_ctx* ctx, const int8_t* codes, int64_t n, int32_t dim,
                       const float* scale, const float* offset, float* rows);
/* Flat index over int8 codes; search distances are the metric between the fp32 query and the
 * dequantised row.  The reference stores codes but has no scan over them
 * (ScalarQuantizer.swift:453-464 asks for a kernel that does not exist). */
int32_t vsk_sq8_index_create(vsk_ctx* ctx, int32_t metric, int32_t dim, const float* scale,
                             const float* offset, vsk_index** out_index);
int32_t vsk_sq8_index_add(vsk_index* index, const int8_t* codes, int64_t n);
int32_t vsk_sq8_index_add_dev(vsk_index* index, const int8_t* codes, int64_t n);

/* --- product quantisation ---------------------------------------------------------------------
 * Replaces ProductQuantizer (Quantization/ProductQuantizer.swift) and the shaders productQuantize /
 * productDequantize (Acceleration/Metal/Shaders/QuantizationShaders.metal:113-204).
 *   codebooks   [segments][codebook_size][dim / segments] floats (Codebook.centroids,
 *               ProductQuantizerCodebook.swift:8-11); dim % segments == 0, 2 <= codebook_size <= 256
 *               (ProductQuantizationConfig.validate, Config/Quantization/ProductQuantizationConfig.swift:42-49;
 *               a code is one byte, QuantizedVector.codes: [UInt8])
 *   train       one k-means per segment (trainSegmentCodebook :266-312), `iterations` Lloyd steps from
 *               init_codebooks (same layout; NULL = the segments of the first codebook_size rows).  The reference
 *               seeds k-means++ / mini-batch k-means from Swift's random number generator, which cannot be
 *               reproduced; callers that need the reference's codebooks pass them to the calls below.
 *               Needs n >= codebook_size * segments rows (:34-41), else VSK_ERR_INSUFFICIENT_TRAINING_DATA.
 *   encode      codes[n][segments]: per segment the nearest codeword by squared L2 accumulated in dimension
 *               order, lowest code on ties (Codebook.encode :12-30)
 *   decode      rows[n][dim]: the coded codewords side by side (:152-163); the per-vector norm rescale of
 *               :165-180 uses a norm the Swift object stores beside the codes and is the caller's to apply
 *   tables      tables[nq][segments][codebook_size]: squared L2 between each query segment and each codeword
 *               (precomputeDistanceTables :205-233)
 *   index       codes resident on the GPU; vsk_search / vsk_search_dev return per query the k rows with the
 *               smallest asymmetric distance sqrt(sum over segments of table[segment][code])
 *               (DistanceTables.computeDistance, ProductQuantizerTypes.swift:14-20; computeAsymmetricDistance
 *               :341-356), ascending, ties by row.  The reference computes that distance one vector at a time and
 *               has no scan over stored codes.  qmasks must be NULL. */
int32_t vsk_pq_train(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t segments,
                     int32_t codebook_size, int32_t iterations, const float* init_codebooks, float* codebooks);
int32_t vsk_pq_train_dev(vsk_ctx* ctx, const float* rows, int64_t n, int32_t dim, int32_t segments,
                         int32_t codebook_size, int32_t iterations, const float* init_codebooks, float* codebooks);
int32_t vsk_pq_encode(vsk_ctx* ctx, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                      const float* rows, int64_t n, uint8_t* codes);
int32_t vsk_pq_encode_dev(vsk_ctx* ctx, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                          const float* rows, int64_t n, uint8_t* codes);
int32_t vsk_pq_decode(vsk_ctx* ctx, const float* codebooks, int32_t dim, int32_t segments, int32_t codebook_size,
                      const uint8_t* codes, int64_t n, float* rows);
int32_t vsk_pq_distance_tables(vsk_ctx* ctx, const float* codebooks, int32_t dim, int32_t segments,
                               int32_t codebook_size, const float* queries, int64_t nq, float* tables);
/* codebooks: host or device memory, copied. */
int32_t vsk_pq_index_create(vsk_ctx* ctx, int32_t dim, int32_t segments, int32_t codebook_size,
                            const float* codebooks, vsk_index** out_index);
int32_t vsk_pq_index_add(vsk_index* index, const uint8_t* codes, int64_t n);
int32_t vsk_pq_index_add_dev(vsk_index* index, const uint8_t* codes, int64_t n);

#ifdef __cplusplus
}
#endif
#endif /* VSK_CUDA_H_ */
