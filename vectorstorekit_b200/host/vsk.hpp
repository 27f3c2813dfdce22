// Header-only C++ host layer over the C ABI (include/vsk_cuda.h), mirroring the names, argument
// meaning and error behaviour of VectorStoreKit's Swift types for the accelerated search path
// (paths relative to Sources/VectorStoreKit):
//   DistanceMetric                 Core/SearchTypes.swift:105-118
//   CUDAAcceleratorStrategy        a ComputeAccelerator, Core/Protocols.swift:11-20
//   CUDAAccelerationEngine         MetalAccelerationEngine.computeDistances / batchComputeDistances,
//                                  Acceleration/MetalAccelerationEngine.swift:76-204
//   FlatIndex, IVFIndex            VectorStore.search / IVFIndex.train/insert/search,
//                                  API/VectorStore.swift:271-318, Indexes/IVFIndex.swift:80-202,397-446
//   ScalarQuantizer                Quantization/ScalarQuantizer.swift (int8)
// Errors are thrown as exceptions named after MetalComputeError / IVFError cases.
#pragma once
#include <algorithm>
#include <cstdint>
#include <future>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/vsk_cuda.h"

namespace vsk {

enum class DistanceMetric { euclidean = 0, cosine = 1, dotProduct = 2, manhattan = 3,
                            chebyshev, minkowski, hamming, jaccard, mahalanobis, earth_mover, learned, adaptive };

struct Error : std::runtime_error {
  int32_t status;
  Error(int32_t s, const std::string& m) : std::runtime_error(m), status(s) {}
};
struct DeviceNotAvailable : Error { using Error::Error; };
struct DeviceOutOfMemory : Error { using Error::Error; };
struct UnsupportedOperation : Error { using Error::Error; };
struct InvalidInput : Error { using Error::Error; };
struct DimensionMismatch : Error { using Error::Error; };
struct EmptyInput : Error { using Error::Error; };
struct Timeout : Error { using Error::Error; };
struct NotTrained : Error { using Error::Error; };
struct InsufficientTrainingData : Error { using Error::Error; };
struct ImportFailed : Error { using Error::Error; };   // ImportError.decodingFailed (IVFIndex.swift:640-643)
struct ExportFailed : Error { using Error::Error; };   // VectorStoreError.exportError (Errors.swift:661-680)

inline void check(int32_t st, vsk_ctx* ctx) {
  if (st == VSK_OK) return;
  std::string msg = ctx ? vsk_last_error(ctx) : "";
  if (msg.empty()) msg = vsk_status_string(st);
  switch (st) {
    case VSK_ERR_DEVICE_NOT_AVAILABLE: throw DeviceNotAvailable(st, msg);
    case VSK_ERR_OUT_OF_MEMORY: throw DeviceOutOfMemory(st, msg);
    case VSK_ERR_UNSUPPORTED_OPERATION: throw UnsupportedOperation(st, msg);
    case VSK_ERR_DIMENSION_MISMATCH: throw DimensionMismatch(st, msg);
    case VSK_ERR_EMPTY_INPUT: throw EmptyInput(st, msg);
    case VSK_ERR_TIMEOUT: throw Timeout(st, msg);
    case VSK_ERR_NOT_TRAINED: throw NotTrained(st, msg);
    case VSK_ERR_INSUFFICIENT_TRAINING_DATA: throw InsufficientTrainingData(st, msg);
    case VSK_ERR_INVALID_INPUT: case VSK_ERR_INVALID_BUFFER_SIZE: throw InvalidInput(st, msg);
    case VSK_ERR_IMPORT_FAILED: throw ImportFailed(st, msg);
    case VSK_ERR_EXPORT_FAILED: throw ExportFailed(st, msg);
    default: throw Error(st, msg);
  }
}

inline int32_t metric_id(DistanceMetric m) {
  if (static_cast<int>(m) > 3)  // MetalDistanceCompute.swift:342-344
    throw UnsupportedOperation(VSK_ERR_UNSUPPORTED_OPERATION, "Distance metric not supported on GPU");
  return static_cast<int32_t>(m);
}

// What CUDAAcceleratorStrategy::initialize() returns.
class CUDAComputeDevice {
 public:
  explicit CUDAComputeDevice(int device = 0) {
    int32_t st = vsk_open(device, &ctx_);
    if (st != VSK_OK) throw DeviceNotAvailable(st, vsk_status_string(st));
  }
  ~CUDAComputeDevice() { if (ctx_) vsk_close(ctx_); }
  CUDAComputeDevice(const CUDAComputeDevice&) = delete;
  CUDAComputeDevice& operator=(const CUDAComputeDevice&) = delete;
  vsk_ctx* ctx() const { return ctx_; }
  vsk_device_info capabilities() const { vsk_device_info i{}; check(vsk_device_info_get(ctx_, &i), ctx_); return i; }
  vsk_stats statistics() const { vsk_stats s{}; check(vsk_stats_get(ctx_, &s), ctx_); return s; }
  // Row-sharded search: one process and one device object per GPU.  ONE rank makes the id, the host hands the same
  // bytes to every rank, every rank joins with its own rank number.
  static std::vector<uint8_t> communicatorId() {
    std::vector<uint8_t> id(VSK_COMM_ID_BYTES);
    const int32_t st = vsk_comm_unique_id(id.data());
    if (st != VSK_OK) throw Error(st, "NCCL is not available");
    return id;
  }
  void joinCommunicator(int32_t nranks, int32_t rank, const std::vector<uint8_t>& id) {
    check(vsk_comm_init(ctx_, nranks, rank, id.empty() ? nullptr : id.data()), ctx_);
  }
  void leaveCommunicator() { check(vsk_comm_destroy(ctx_), ctx_); }
  // Blocks until every asynchronous call has completed; throws the first failure.
  void wait() { check(vsk_wait(ctx_), ctx_); }
  std::pair<int32_t, int32_t> communicator() const {   // (ranks, this rank)
    int32_t n = 1, r = 0;
    check(vsk_comm_info(ctx_, &n, &r), ctx_);
    return {n, r};
  }
 private:
  vsk_ctx* ctx_ = nullptr;
};

struct CUDAAcceleratorStrategy {
  const char* identifier = "cuda-sm100a";
  int device = 0;
  std::shared_ptr<CUDAComputeDevice> initialize() const { return std::make_shared<CUDAComputeDevice>(device); }
};

struct SearchResults {            // one ascending row of k hits per query
  int64_t nq = 0; int32_t k = 0;
  std::vector<float> distances;   // [nq*k]
  std::vector<int64_t> ids;       // [nq*k], -1 where fewer than k rows were eligible
};

// VectorIndex.export(format: .binary) -> Data (Core/Protocols.swift:157): the index image as bytes.
inline std::vector<uint8_t> exportIndex(vsk_index* ix, vsk_ctx* ctx) {
  int64_t bytes = 0, written = 0;
  check(vsk_index_image_size(ix, &bytes), ctx);
  std::vector<uint8_t> out((size_t)bytes);
  check(vsk_index_export(ix, out.data(), bytes, &written), ctx);
  out.resize((size_t)written);
  return out;
}

class FlatIndex {
 public:
  FlatIndex(std::shared_ptr<CUDAComputeDevice> dev, int32_t dimensions, DistanceMetric metric)
      : dev_(std::move(dev)), dim_(dimensions) {
    check(vsk_flat_create(dev_->ctx(), metric_id(metric), dimensions, &ix_), dev_->ctx());
  }
  // import(data:format: .binary) / a file written by save(): the image must hold a flat fp32 index
  FlatIndex(std::shared_ptr<CUDAComputeDevice> dev, const void* image, int64_t bytes) : dev_(std::move(dev)) {
    check(vsk_index_import(dev_->ctx(), image, bytes, &ix_), dev_->ctx());
    adopt();
  }
  FlatIndex(std::shared_ptr<CUDAComputeDevice> dev, const std::string& path) : dev_(std::move(dev)) {
    check(vsk_index_load(dev_->ctx(), path.c_str(), &ix_), dev_->ctx());
    adopt();
  }
  std::vector<uint8_t> exportBinary() const { return exportIndex(ix_, dev_->ctx()); }
  void save(const std::string& path) const { check(vsk_index_save(ix_, path.c_str()), dev_->ctx()); }
  ~FlatIndex() { if (ix_) vsk_index_destroy(ix_); }
  FlatIndex(const FlatIndex&) = delete;
  FlatIndex& operator=(const FlatIndex&) = delete;
  void add(const float* rows, int64_t n, const uint64_t* masks = nullptr) { check(vsk_flat_add_f32(ix_, rows, n, masks), dev_->ctx()); }
  int64_t count() const { return vsk_index_size(ix_); }
  SearchResults batchSearch(const float* queries, int64_t nq, int32_t k, const uint64_t* filter_masks = nullptr) const {
    SearchResults r; r.nq = nq; r.k = k;
    if (nq <= 0) throw EmptyInput(VSK_ERR_EMPTY_INPUT, "no queries");
    r.distances.resize((size_t)nq * k); r.ids.resize((size_t)nq * k);
    check(vsk_search(ix_, queries, nq, k, filter_masks, r.distances.data(), r.ids.data()), dev_->ctx());
    return r;
  }
  // The awaited form (MetalAccelerationEngine.batchComputeDistances is `async`, :139-204): the library's worker thread
  // fulfils the future.  `queries` (and filter_masks) stay valid until then; until the future is ready the device
  // object takes only further *Async calls and wait().
  std::future<SearchResults> batchSearchAsync(const float* queries, int64_t nq, int32_t k,
                                              const uint64_t* filter_masks = nullptr) const {
    if (nq <= 0) throw EmptyInput(VSK_ERR_EMPTY_INPUT, "no queries");
    struct Pending { std::promise<SearchResults> p; SearchResults r; vsk_ctx* ctx; };
    auto* pend = new Pending();
    pend->ctx = dev_->ctx();
    pend->r.nq = nq; pend->r.k = k;
    pend->r.distances.resize((size_t)nq * k); pend->r.ids.resize((size_t)nq * k);
    auto fut = pend->p.get_future();
    const int32_t st = vsk_search_async(ix_, queries, nq, k, filter_masks, pend->r.distances.data(), pend->r.ids.data(),
        [](void* user, int32_t status) {
          std::unique_ptr<Pending> p(static_cast<Pending*>(user));
          if (status == VSK_OK) { p->p.set_value(std::move(p->r)); return; }
          try { check(status, p->ctx); } catch (...) { p->p.set_exception(std::current_exception()); }
        }, pend);
    if (st != VSK_OK) { delete pend; check(st, dev_->ctx()); }
    return fut;
  }
  // This index holds rows [idBase, idBase + count) of a database spread over the ranks of the device's communicator.
  void setIdBase(int64_t base) { check(vsk_index_set_id_base(ix_, base), dev_->ctx()); }
  // The sharded form of batchSearch: every rank passes the same queries.  gather = false: the merged results of this
  // rank's slice of the queries (firstQuery says where the slice starts); gather = true: all queries on every rank.
  SearchResults shardedSearch(const float* queries, int64_t nq, int32_t k, const uint64_t* filter_masks = nullptr,
                              bool gather = false, int64_t* firstQuery = nullptr) const {
    if (nq <= 0) throw EmptyInput(VSK_ERR_EMPTY_INPUT, "no queries");
    const auto cm = dev_->communicator();
    int64_t first = 0, count = nq;
    if (!gather) vsk_sharded_slice(nq, cm.first, cm.second, &first, &count);
    SearchResults r; r.nq = count; r.k = k;
    r.distances.resize((size_t)std::max<int64_t>(count, 1) * k); r.ids.resize((size_t)std::max<int64_t>(count, 1) * k);
    check(vsk_search_sharded(ix_, queries, nq, k, filter_masks, gather ? VSK_SHARDED_ALL : VSK_SHARDED_SLICE,
                             r.distances.data(), r.ids.data()), dev_->ctx());
    r.distances.resize((size_t)count * k); r.ids.resize((size_t)count * k);
    if (firstQuery) *firstQuery = first;
    return r;
  }
 private:
  void adopt() {
    vsk_index_info info{};
    vsk_index_info_get(ix_, &info);
    if (info.kind != VSK_INDEX_FLAT_F32) {
      vsk_index_destroy(ix_);
      ix_ = nullptr;
      throw ImportFailed(VSK_ERR_IMPORT_FAILED, "the image does not hold a flat fp32 index");
    }
    dim_ = info.dimensions;
  }
  std::shared_ptr<CUDAComputeDevice> dev_;
  vsk_index* ix_ = nullptr;
  int32_t dim_ = 0;
};

// MetalAccelerationEngine's distance surface.
class CUDAAccelerationEngine {
 public:
  explicit CUDAAccelerationEngine(std::shared_ptr<CUDAComputeDevice> dev) : dev_(std::move(dev)) {}
  // batchComputeDistances(queries:candidates:metric:topK: nil): Q x N, row-major
  std::vector<float> batchComputeDistances(const float* q, int64_t nq, const float* x, int64_t nx, int32_t dim,
                                           DistanceMetric metric) const {
    if (nq <= 0 || nx <= 0) throw EmptyInput(VSK_ERR_EMPTY_INPUT, "Empty input provided for distance computation");
    std::vector<float> out((size_t)nq * nx);
    check(vsk_batch_distances(dev_->ctx(), metric_id(metric), q, nq, x, nx, dim, out.data()), dev_->ctx());
    return out;
  }
  // MetalDistanceMatrix.computeDistanceMatrix(vectorsA:vectorsB:metric:) (MetalDistanceMatrix.swift:49-119), row-major
  // na x nb; with b == nullptr the matrix of a against itself, lower triangle mirrored from the upper (:352-381)
  std::vector<float> computeDistanceMatrix(const float* a, int64_t na, const float* b, int64_t nb, int32_t dim,
                                           DistanceMetric metric) const {
    if (!b) {
      std::vector<float> m = batchComputeDistances(a, na, a, na, dim, metric);
      for (int64_t i = 0; i < na; ++i)
        for (int64_t j = 0; j < i; ++j) m[(size_t)(i * na + j)] = m[(size_t)(j * na + i)];
      return m;
    }
    return batchComputeDistances(a, na, b, nb, dim, metric);
  }
  // computeDistances(query:candidates:metric:)
  std::vector<float> computeDistances(const float* query, const float* x, int64_t nx, int32_t dim, DistanceMetric m) const {
    return batchComputeDistances(query, 1, x, nx, dim, m);
  }
  // batchComputeDistances(...topK: k): per query the k smallest distances, ascending (distances only)
  std::vector<float> batchComputeDistances(const float* q, int64_t nq, const float* x, int64_t nx, int32_t dim,
                                           DistanceMetric metric, int32_t topK) const {
    FlatIndex ix(dev_, dim, metric);
    ix.add(x, nx);
    return ix.batchSearch(q, nq, topK < nx ? topK : (int32_t)nx).distances;
  }
 private:
  std::shared_ptr<CUDAComputeDevice> dev_;
};

class IVFIndex {
 public:
  IVFIndex(std::shared_ptr<CUDAComputeDevice> dev, int32_t dimensions, int32_t numberOfCentroids = 1024,
           int32_t numberOfProbes = 10, int32_t maxIterations = 100, float tolerance = 1e-4f)
      : dev_(std::move(dev)), dim_(dimensions), nlist_(numberOfCentroids), nprobe_(numberOfProbes), iters_(maxIterations), tol_(tolerance) {
    if (dimensions <= 0 || numberOfCentroids <= 0 || numberOfProbes <= 0 || numberOfProbes > numberOfCentroids)
      throw InvalidInput(VSK_ERR_INVALID_INPUT, "IVFConfiguration.validate failed");  // IVFConfiguration.swift:49-59
  }
  ~IVFIndex() { if (ix_) vsk_index_destroy(ix_); }
  // train(on:) with `.custom` initial centroids (default: the first numberOfCentroids samples)
  void train(const float* samples, int64_t n, const float* initial = nullptr) {
    if (n < nlist_) throw InsufficientTrainingData(VSK_ERR_INSUFFICIENT_TRAINING_DATA, "insufficient training data");
    centroids_.resize((size_t)nlist_ * dim_);
    std::vector<int32_t> assign((size_t)n);
    float inertia = 0; int32_t iters = 0;
    check(vsk_kmeans(dev_->ctx(), samples, n, dim_, nlist_, iters_, tol_, initial ? initial : samples, centroids_.data(),
                     assign.data(), &inertia, &iters), dev_->ctx());
    trained_ = true;
  }
  // IVFIndex.insert (Indexes/IVFIndex.swift:80-122): the first rows build the lists, later ones are filed behind the
  // rows their lists already hold (no rebuild).  `masks` (one 64-bit filter mask per row) either on every call or on none.
  void insert(const float* rows, int64_t n, const uint64_t* masks = nullptr) {
    if (!trained_) throw NotTrained(VSK_ERR_NOT_TRAINED, "Index must be trained before use");
    if (!ix_) {
      check(vsk_ivf_build(dev_->ctx(), centroids_.data(), nlist_, rows, n, dim_, &ix_), dev_->ctx());
      if (masks) check(vsk_ivf_set_masks(ix_, masks), dev_->ctx());
    } else {
      check(vsk_ivf_add(ix_, rows, n, masks), dev_->ctx());
    }
  }
  // search(query:k:strategy:filter:) for a batch: filter_masks = one mask per query (a row is eligible when it shares a bit)
  SearchResults batchSearch(const float* queries, int64_t nq, int32_t k, bool exact = false,
                            const uint64_t* filter_masks = nullptr) const {
    if (!trained_ || !ix_) throw NotTrained(VSK_ERR_NOT_TRAINED, "Index must be trained before use");
    SearchResults r; r.nq = nq; r.k = k;
    r.distances.resize((size_t)nq * k); r.ids.resize((size_t)nq * k);
    check(vsk_ivf_search_filtered(ix_, queries, nq, k, exact ? nlist_ : nprobe_, filter_masks, r.distances.data(), r.ids.data()),
          dev_->ctx());
    return r;
  }
  // Rows sharded over the ranks of the device's communicator (every rank holds a slice of every list, same centroids):
  // see FlatIndex::shardedSearch for the layouts.
  void setIdBase(int64_t base) { check(vsk_index_set_id_base(ix_, base), dev_->ctx()); }
  SearchResults shardedSearch(const float* queries, int64_t nq, int32_t k, const uint64_t* filter_masks = nullptr,
                              bool gather = false, int64_t* firstQuery = nullptr) const {
    if (!trained_ || !ix_) throw NotTrained(VSK_ERR_NOT_TRAINED, "Index must be trained before use");
    const auto cm = dev_->communicator();
    int64_t first = 0, count = nq;
    if (!gather) vsk_sharded_slice(nq, cm.first, cm.second, &first, &count);
    SearchResults r; r.nq = count; r.k = k;
    r.distances.resize((size_t)std::max<int64_t>(count, 1) * k); r.ids.resize((size_t)std::max<int64_t>(count, 1) * k);
    check(vsk_ivf_search_sharded(ix_, queries, nq, k, nprobe_, filter_masks, gather ? VSK_SHARDED_ALL : VSK_SHARDED_SLICE,
                                 r.distances.data(), r.ids.data()), dev_->ctx());
    r.distances.resize((size_t)count * k); r.ids.resize((size_t)count * k);
    if (firstQuery) *firstQuery = first;
    return r;
  }
  const std::vector<float>& centroids() const { return centroids_; }
 private:
  std::shared_ptr<CUDAComputeDevice> dev_;
  vsk_index* ix_ = nullptr;
  int32_t dim_, nlist_, nprobe_, iters_;
  float tol_;
  bool trained_ = false;
  std::vector<float> centroids_;
};

class ScalarQuantizer {
 public:
  ScalarQuantizer(std::shared_ptr<CUDAComputeDevice> dev, bool per_dim = false) : dev_(std::move(dev)), per_dim_(per_dim) {}
  void train(const float* rows, int64_t n, int32_t dim) {
    scale.resize(dim); offset.resize(dim);
    check(vsk_sq8_train(dev_->ctx(), rows, n, dim, per_dim_ ? VSK_SQ8_PER_DIM : VSK_SQ8_GLOBAL, scale.data(), offset.data()), dev_->ctx());
  }
  std::vector<int8_t> quantizeBatch(const float* rows, int64_t n, int32_t dim) const {
    std::vector<int8_t> codes((size_t)n * dim);
    check(vsk_sq8_encode(dev_->ctx(), rows, n, dim, scale.data(), offset.data(), codes.data()), dev_->ctx());
    return codes;
  }
  std::vector<float> dequantizeBatch(const int8_t* codes, int64_t n, int32_t dim) const {
    std::vector<float> rows((size_t)n * dim);
    check(vsk_sq8_decode(dev_->ctx(), codes, n, dim, scale.data(), offset.data(), rows.data()), dev_->ctx());
    return rows;
  }
  std::vector<float> scale, offset;
 private:
  std::shared_ptr<CUDAComputeDevice> dev_;
  bool per_dim_;
};

// ProductQuantizer (Quantization/ProductQuantizer.swift) with ProductQuantizationConfig's fields; codes are one byte
// per segment, so codeSize is at most 8.
class ProductQuantizer {
 public:
  ProductQuantizer(std::shared_ptr<CUDAComputeDevice> dev, int32_t dimensions, int32_t segments = 8, int32_t codeSize = 8,
                   int32_t trainingIterations = 25)
      : dev_(std::move(dev)), dim_(dimensions), m_(segments), ksub_(1 << codeSize), iters_(trainingIterations) {
    if (dimensions <= 0 || segments <= 0 || dimensions % segments != 0)
      throw InvalidInput(VSK_ERR_INVALID_INPUT, "invalid segmentation");          // QuantizationError.invalidSegmentation
    if (codeSize < 4 || codeSize > 8) throw InvalidInput(VSK_ERR_INVALID_INPUT, "invalid code size");
  }
  // train(on:) from initial codewords [segments][codebookSize][dimensions / segments] (nullptr: the first rows' segments)
  void train(const float* rows, int64_t n, const float* initial = nullptr) {
    codebooks.resize((size_t)ksub_ * dim_);
    check(vsk_pq_train(dev_->ctx(), rows, n, dim_, m_, ksub_, iters_, initial, codebooks.data()), dev_->ctx());
    trained_ = true;
  }
  void setCodebooks(std::vector<float> cb) { codebooks = std::move(cb); trained_ = true; }
  std::vector<uint8_t> encodeBatch(const float* rows, int64_t n) const {
    need();
    std::vector<uint8_t> codes((size_t)n * m_);
    check(vsk_pq_encode(dev_->ctx(), codebooks.data(), dim_, m_, ksub_, rows, n, codes.data()), dev_->ctx());
    return codes;
  }
  std::vector<float> decodeBatch(const uint8_t* codes, int64_t n) const {
    need();
    std::vector<float> rows((size_t)n * dim_);
    check(vsk_pq_decode(dev_->ctx(), codebooks.data(), dim_, m_, ksub_, codes, n, rows.data()), dev_->ctx());
    return rows;
  }
  // precomputeDistanceTables(query:) for a batch: [nq][segments][codebookSize]
  std::vector<float> precomputeDistanceTables(const float* queries, int64_t nq) const {
    need();
    std::vector<float> t((size_t)nq * m_ * ksub_);
    check(vsk_pq_distance_tables(dev_->ctx(), codebooks.data(), dim_, m_, ksub_, queries, nq, t.data()), dev_->ctx());
    return t;
  }
  int32_t segments() const { return m_; }
  int32_t codebookSize() const { return ksub_; }
  int32_t dimensions() const { return dim_; }
  std::vector<float> codebooks;
 private:
  void need() const { if (!trained_) throw NotTrained(VSK_ERR_NOT_TRAINED, "Quantizer must be trained before use"); }
  std::shared_ptr<CUDAComputeDevice> dev_;
  int32_t dim_, m_, ksub_, iters_;
  bool trained_ = false;
};

// Codes resident on the GPU, searched by asymmetric distance (DistanceTables.computeDistance,
// ProductQuantizerTypes.swift:14-20): per query the k nearest rows, ascending, ties by row.
class PQIndex {
 public:
  PQIndex(std::shared_ptr<CUDAComputeDevice> dev, const ProductQuantizer& pq) : dev_(std::move(dev)) {
    check(vsk_pq_index_create(dev_->ctx(), pq.dimensions(), pq.segments(), pq.codebookSize(), pq.codebooks.data(), &ix_), dev_->ctx());
  }
  ~PQIndex() { if (ix_) vsk_index_destroy(ix_); }
  PQIndex(const PQIndex&) = delete;
  PQIndex& operator=(const PQIndex&) = delete;
  void add(const uint8_t* codes, int64_t n) { check(vsk_pq_index_add(ix_, codes, n), dev_->ctx()); }
  int64_t count() const { return vsk_index_size(ix_); }
  SearchResults batchSearch(const float* queries, int64_t nq, int32_t k) const {
    SearchResults r; r.nq = nq; r.k = k;
    r.distances.resize((size_t)nq * k); r.ids.resize((size_t)nq * k);
    check(vsk_search(ix_, queries, nq, k, nullptr, r.distances.data(), r.ids.data()), dev_->ctx());
    return r;
  }
 private:
  std::shared_ptr<CUDAComputeDevice> dev_;
  vsk_index* ix_ = nullptr;
};

// ---- the caller's layer: VectorEntry in, [SearchResult] out -----------------------------------------------------
// VectorEntry(id:vector:metadata:) (Core/VectorTypes.swift:23-45) and SearchResult (Core/SearchTypes.swift:11-55) with
// VectorID = String.  The library works on insertion indices; this class keeps the index -> (VectorID, metadata)
// table on the host, as IVFIndex does (Indexes/IVFIndex.swift:104-111).  A filter is a 64-bit mask here: the caller
// assigns bits to its filters and tags every entry with the bits of the filters it passes (the Python mirror's
// FilterBitmaskCompiler derives them from SearchFilter values); a query passes the bit of its filter.
struct VectorEntry {
  std::string id;
  std::vector<float> vector;
  std::string metadata;        // the entry's metadata as the caller encodes it (JSON in the reference)
  uint64_t filterBits = 0;     // filters this entry passes
};

struct SearchResult {
  std::string id;
  float distance = 0.f;
  std::string metadata;
  const char* tier = "hot";
  float confidence = 1.0f;
};

class VectorStore {   // a flat exact store: VectorStore.search(query:k:strategy:filter:) (API/VectorStore.swift:271-318)
 public:
  VectorStore(std::shared_ptr<CUDAComputeDevice> dev, int32_t dimensions, DistanceMetric metric, bool filtered = false)
      : index_(std::move(dev), dimensions, metric), dim_(dimensions), filtered_(filtered) {}
  int64_t count() const { return (int64_t)ids_.size(); }
  void add(const std::vector<VectorEntry>& entries) {
    if (entries.empty()) return;
    std::vector<float> rows;
    std::vector<uint64_t> masks;
    rows.reserve(entries.size() * (size_t)dim_);
    for (const auto& e : entries) {
      if ((int32_t)e.vector.size() != dim_)
        throw DimensionMismatch(VSK_ERR_DIMENSION_MISMATCH, "expected " + std::to_string(dim_) + ", got " +
                                                                std::to_string(e.vector.size()));
      rows.insert(rows.end(), e.vector.begin(), e.vector.end());
      masks.push_back(e.filterBits);
      ids_.push_back(e.id);
      metadata_.push_back(e.metadata);
    }
    index_.add(rows.data(), (int64_t)entries.size(), filtered_ ? masks.data() : nullptr);
  }
  // one ascending list per query; a list is shorter than k when fewer rows pass the filter
  std::vector<std::vector<SearchResult>> batchSearch(const float* queries, int64_t nq, int32_t k,
                                                     const uint64_t* filterBits = nullptr) const {
    if (filterBits && !filtered_) throw InvalidInput(VSK_ERR_INVALID_INPUT, "the store was created without filters");
    const SearchResults r = index_.batchSearch(queries, nq, k, filterBits);
    std::vector<std::vector<SearchResult>> out((size_t)nq);
    for (int64_t q = 0; q < nq; ++q)
      for (int32_t j = 0; j < k; ++j) {
        const int64_t id = r.ids[(size_t)(q * k + j)];
        if (id < 0) break;
        SearchResult s;
        s.id = ids_[(size_t)id];
        s.distance = r.distances[(size_t)(q * k + j)];
        s.metadata = metadata_[(size_t)id];
        out[(size_t)q].push_back(std::move(s));
      }
    return out;
  }
  std::vector<SearchResult> search(const float* query, int32_t k, uint64_t filterBit = 0) const {
    return batchSearch(query, 1, k, filterBit ? &filterBit : nullptr)[0];
  }
 private:
  FlatIndex index_;
  int32_t dim_;
  bool filtered_;
  std::vector<std::string> ids_, metadata_;
};

}  // namespace vsk
