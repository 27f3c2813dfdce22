// TEST INFRASTRUCTURE — not part of the product.
//
// CPU restatement of VectorStoreKit's batch similarity-search arithmetic, used
// only as the checker for the CUDA path (tests, the smoke check, and the
// cpu-baseline leg of the benchmark).  Nothing in the shipped library links,
// imports or executes this file.
//
// Pinning: every distance / k-means / quantizer function here is checked
//   (1) against the known-answer values in the reference's own tests
//       (Tests/VectorStoreKitTests/ValidationTests/Phase1ValidationTests.swift:143-172,
//        MetalDistance512Tests.swift:50-182, MetalDistanceMatrixTests.swift:27-139,
//        Vector512Tests.swift:61-101, ScalarQuantizerTests.swift:55-94,
//        Sources/VerifyComponents/main.swift:101-119), and
//   (2) bit-for-bit against the reference's Metal shader source compiled as
//       C++ (oracle/_ref, built by oracle/Makefile from the reference tree).
// What stays unpinned because the reference leaves it open: tie order in
// top-k, int8 code bytes at exact .0 boundaries (vDSP_vsmsa may or may not
// fuse), k-means centroids for any seed (the reference's RNG use is not
// reproducible), summation order inside Apple's closed-source vDSP.
//
// All arithmetic is IEEE fp32, accumulated sequentially in index order
// (the order the shader loops and the Swift scalar loops use).  The *_fast
// entry points reassociate the inner sum for SIMD and exist only so the CPU
// baseline can be timed at a realistic speed; they are within 1e-5 relative
// of the strict ones and are never used to judge parity of ids.
//
// Build: g++ -O2 -std=c++17 -fopenmp -ffp-contract=off -shared -fPIC

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// Metric ids shared with include/vsk_cuda.h (the four cases of the reference's
// DistanceMetric enum the accelerated path supports,
// Sources/VectorStoreKit/Core/SearchTypes.swift:105-118).
enum { VSKREF_EUCLIDEAN = 0, VSKREF_COSINE = 1, VSKREF_DOT = 2, VSKREF_MANHATTAN = 3 };

// ---------------------------------------------------------------------------
// Pairwise distances.
// Follows Acceleration/AccelerateOptimizer.swift:251-383 (CPU path) and
// Acceleration/Metal/Shaders/DistanceShaders.metal:62-218 (shader path):
//   euclidean   sqrt(sum (q-x)^2)
//   cosine      1 - q.x / (|q|*|x| + 1e-8)
//   dotProduct  -(q.x)
//   manhattan   sum |q-x|
// ---------------------------------------------------------------------------
float vskref_distance(int metric, const float* q, const float* x, int d) {
  switch (metric) {
    case VSKREF_EUCLIDEAN: {
      float s = 0.0f;
      for (int i = 0; i < d; ++i) { float t = q[i] - x[i]; s += t * t; }
      return std::sqrt(s);
    }
    case VSKREF_COSINE: {
      float dp = 0.0f, qq = 0.0f, xx = 0.0f;
      for (int i = 0; i < d; ++i) { dp += q[i] * x[i]; qq += q[i] * q[i]; xx += x[i] * x[i]; }
      // The literal 1e-8 is a double in both Swift-inferred-Float context
      // (AccelerateOptimizer.swift:316: Float) and MSL (DistanceShaders.metal:131:
      // evaluated in float).  Both end up as fp32 arithmetic.
      float sim = dp / (std::sqrt(qq) * std::sqrt(xx) + 1e-8f);
      return 1.0f - sim;
    }
    case VSKREF_DOT: {
      float dp = 0.0f;
      for (int i = 0; i < d; ++i) dp += q[i] * x[i];
      return -dp;
    }
    case VSKREF_MANHATTAN: {
      float s = 0.0f;
      for (int i = 0; i < d; ++i) s += std::fabs(q[i] - x[i]);
      return s;
    }
    default:
      // AccelerateOptimizer.swift:527-528 returns +inf for unsupported metrics.
      return std::numeric_limits<float>::infinity();
  }
}

// Reassociated variant (8 partial sums) for timing only.
static float distance_fast(int metric, const float* __restrict q, const float* __restrict x, int d,
                           float qnorm) {
  constexpr int L = 16;
  float acc[L] = {0};
  float acc2[L] = {0};
  int i = 0;
  switch (metric) {
    case VSKREF_EUCLIDEAN: {
      for (; i + L <= d; i += L)
        for (int l = 0; l < L; ++l) { float t = q[i + l] - x[i + l]; acc[l] += t * t; }
      float s = 0.0f;
      for (int l = 0; l < L; ++l) s += acc[l];
      for (; i < d; ++i) { float t = q[i] - x[i]; s += t * t; }
      return std::sqrt(s);
    }
    case VSKREF_COSINE: {
      for (; i + L <= d; i += L)
        for (int l = 0; l < L; ++l) { acc[l] += q[i + l] * x[i + l]; acc2[l] += x[i + l] * x[i + l]; }
      float dp = 0.0f, xx = 0.0f;
      for (int l = 0; l < L; ++l) { dp += acc[l]; xx += acc2[l]; }
      for (; i < d; ++i) { dp += q[i] * x[i]; xx += x[i] * x[i]; }
      return 1.0f - dp / (qnorm * std::sqrt(xx) + 1e-8f);
    }
    case VSKREF_DOT: {
      for (; i + L <= d; i += L)
        for (int l = 0; l < L; ++l) acc[l] += q[i + l] * x[i + l];
      float dp = 0.0f;
      for (int l = 0; l < L; ++l) dp += acc[l];
      for (; i < d; ++i) dp += q[i] * x[i];
      return -dp;
    }
    default: {
      for (; i + L <= d; i += L)
        for (int l = 0; l < L; ++l) acc[l] += std::fabs(q[i + l] - x[i + l]);
      float s = 0.0f;
      for (int l = 0; l < L; ++l) s += acc[l];
      for (; i < d; ++i) s += std::fabs(q[i] - x[i]);
      return s;
    }
  }
}

// Full Q x N matrix, row-major out[q*N + c]
// (DistanceShaders.metal:248-379, MetalAccelerationEngine.swift:377-478 with topK == nil).
void vskref_batch_distances(int metric, const float* q, int64_t nq, const float* x, int64_t nx,
                            int d, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t a = 0; a < nq; ++a)
    for (int64_t b = 0; b < nx; ++b)
      out[a * nx + b] = vskref_distance(metric, q + a * d, x + b * d, d);
}

// ---------------------------------------------------------------------------
// Exact flat k-NN: per query, distances to every (eligible) row, ascending
// sort, first k.  This is the intended top-k of the reference
// (MetalAccelerationEngine.swift:465-471, UnifiedDistanceComputation.swift:129-133,
// IVFIndex.swift:175-176); the min-heap branch of
// AccelerateOptimizer.selectTopK (:137-148) evicts the wrong element and is
// not reproduced.  Ties are ordered by row id (the reference leaves tie order
// unspecified).
//
// Optional bitmask pre-filter: row r is eligible for query a iff
// (row_masks[r] & query_masks[a]) != 0.  The reference filters candidates
// before computing distances (IVFIndex.swift:163-172, LLMVectorStore.swift:83-114),
// so the k hits come only from eligible rows.
//
// Slots beyond the number of eligible rows get id -1 and distance +inf.
// mode: 0 = strict sequential sums, 1 = reassociated (timing only).
// nthreads: 1 follows AccelerateOptimizer.batchComputeDistances (sequential
// over queries, :106-118); >1 follows UnifiedDistanceComputation's one task
// per query (:118-146).
// ---------------------------------------------------------------------------
void vskref_flat_search(int metric, const float* q, int64_t nq, const float* x, int64_t nx, int d,
                        int k, const uint64_t* row_masks, const uint64_t* query_masks,
                        float* out_dist, int64_t* out_ids, int mode, int nthreads) {
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
  {
    std::vector<std::pair<float, int64_t>> cand;
    cand.reserve((size_t)nx);
#pragma omp for schedule(dynamic, 1)
    for (int64_t a = 0; a < nq; ++a) {
      const float* qa = q + a * d;
      cand.clear();
      float qn = 0.0f;
      if (mode == 1 && metric == VSKREF_COSINE) {
        for (int i = 0; i < d; ++i) qn += qa[i] * qa[i];
        qn = std::sqrt(qn);
      }
      const bool filt = row_masks && query_masks;
      const uint64_t qm = filt ? query_masks[a] : 0;
      for (int64_t b = 0; b < nx; ++b) {
        if (filt && (row_masks[b] & qm) == 0) continue;
        float dist = mode == 1 ? distance_fast(metric, qa, x + b * d, d, qn)
                               : vskref_distance(metric, qa, x + b * d, d);
        cand.emplace_back(dist, b);
      }
      size_t kk = std::min<size_t>((size_t)k, cand.size());
      std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
      for (size_t j = 0; j < (size_t)k; ++j) {
        out_dist[a * k + j] = j < kk ? cand[j].first : std::numeric_limits<float>::infinity();
        out_ids[a * k + j] = j < kk ? cand[j].second : -1;
      }
    }
  }
}

// In-place row normalisation, EmbeddingVector.normalize (LLM/Vector.swift:25-32):
// x_i /= |x| when |x| > 0; fp32 sum of squares in index order.
void vskref_normalize_rows(float* x, int64_t n, int d) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    float s = 0.0f;
    for (int i = 0; i < d; ++i) s += x[r * d + i] * x[r * d + i];
    float m = std::sqrt(s);
    if (m > 0.0f)
      for (int i = 0; i < d; ++i) x[r * d + i] /= m;
  }
}

// ---------------------------------------------------------------------------
// Lloyd k-means, Clustering/KMeansClustering.swift:48-113 with
//   assignment  :271-295  rooted L2, strict '<' so the lowest index wins ties
//   update      :342-380  fp32 sums in row order, divide by count
//   inertia     :97       sum of the UN-squared distances (reference quirk, kept)
//   stop        :98       |inertia - previous| < tolerance, or max_iters
// Initial centroids are supplied by the caller (the reference's `.custom`
// initialisation, :189-193); its k-means++ path depends on Swift's stdlib RNG
// mapping and cannot be reproduced.
// Empty cluster: the Swift code re-seeds from an unseeded system RNG (:372-376),
// which is not reproducible; this follows the reference's shader rule instead —
// keep the previous centroid (Shaders/ClusteringShaders.metal:171-176).
// tolerance < 0 disables the convergence test (exactly max_iters iterations).
// ---------------------------------------------------------------------------
void vskref_kmeans(const float* x, int64_t n, int d, int k, int max_iters, float tolerance,
                   const float* init_centroids, float* centroids, int32_t* assign,
                   float* inertia_out, int32_t* iters_out) {
  std::vector<float> cur(init_centroids, init_centroids + (size_t)k * d);
  std::vector<float> dist((size_t)n);
  std::vector<int32_t> asg((size_t)n, 0);
  float prev_inertia = std::numeric_limits<float>::infinity();
  int iters = 0;
  bool converged = false;
  while (iters < max_iters && !converged) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      float best = std::numeric_limits<float>::infinity();
      int bi = 0;
      for (int c = 0; c < k; ++c) {
        float s = 0.0f;
        for (int i = 0; i < d; ++i) { float t = x[r * d + i] - cur[(size_t)c * d + i]; s += t * t; }
        float dd = std::sqrt(s);
        if (dd < best) { best = dd; bi = c; }
      }
      asg[r] = bi;
      dist[r] = best;
    }
    std::vector<float> sums((size_t)k * d, 0.0f);
    std::vector<float> counts((size_t)k, 0.0f);
    for (int64_t r = 0; r < n; ++r) {
      float* s = &sums[(size_t)asg[r] * d];
      for (int i = 0; i < d; ++i) s[i] += x[r * d + i] * 1.0f;
      counts[asg[r]] += 1.0f;
    }
    for (int c = 0; c < k; ++c) {
      if (counts[c] > 0.0f)
        for (int i = 0; i < d; ++i) sums[(size_t)c * d + i] /= counts[c];
      else
        for (int i = 0; i < d; ++i) sums[(size_t)c * d + i] = cur[(size_t)c * d + i];
    }
    float inertia = 0.0f;
    for (int64_t r = 0; r < n; ++r) inertia += dist[r];
    converged = tolerance >= 0.0f && std::fabs(inertia - prev_inertia) < tolerance;
    cur.swap(sums);
    prev_inertia = inertia;
    ++iters;
  }
  std::memcpy(centroids, cur.data(), sizeof(float) * (size_t)k * d);
  std::memcpy(assign, asg.data(), sizeof(int32_t) * (size_t)n);
  if (inertia_out) *inertia_out = prev_inertia;
  if (iters_out) *iters_out = iters;
}

// Nearest-centroid assignment alone (IVFIndex.findNearestCentroid, IVFIndex.swift:514-527).
void vskref_assign(const float* x, int64_t n, int d, const float* centroids, int k,
                   int32_t* assign, float* dist) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    float best = std::numeric_limits<float>::infinity();
    int bi = 0;
    for (int c = 0; c < k; ++c) {
      float dd = vskref_distance(VSKREF_EUCLIDEAN, x + r * d, centroids + (size_t)c * d, d);
      if (dd < best) { best = dd; bi = c; }
    }
    assign[r] = bi;
    if (dist) dist[r] = best;
  }
}

// ---------------------------------------------------------------------------
// IVF search, Indexes/IVFIndex.swift:124-202:
//   probes  = the nprobe centroids nearest the query by rooted L2
//             (findNearestCentroids :529-540: all distances, ascending sort, prefix)
//   scan    = every row of the probed lists, rooted L2 (:168-172, :542-549;
//             IVF search is Euclidean whatever the store's metric)
//   result  = ascending sort, first k (:175-176)
// List membership is passed in as `assign` (row -> list) so that the checker
// and the CUDA path search the same lists.  Ties ordered by row id.
// ---------------------------------------------------------------------------
void vskref_ivf_search(const float* q, int64_t nq, const float* x, int64_t n, int d,
                       const float* centroids, int nlist, const int32_t* assign, int nprobe, int k,
                       float* out_dist, int64_t* out_ids) {
  std::vector<std::vector<int64_t>> lists((size_t)nlist);
  for (int64_t r = 0; r < n; ++r) lists[assign[r]].push_back(r);
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t a = 0; a < nq; ++a) {
    const float* qa = q + a * d;
    std::vector<std::pair<float, int>> cd((size_t)nlist);
    for (int c = 0; c < nlist; ++c)
      cd[c] = {vskref_distance(VSKREF_EUCLIDEAN, qa, centroids + (size_t)c * d, d), c};
    int np = std::min(nprobe, nlist);
    std::partial_sort(cd.begin(), cd.begin() + np, cd.end());
    std::vector<std::pair<float, int64_t>> cand;
    for (int p = 0; p < np; ++p)
      for (int64_t r : lists[cd[p].second])
        cand.emplace_back(vskref_distance(VSKREF_EUCLIDEAN, qa, x + r * d, d), r);
    size_t kk = std::min<size_t>((size_t)k, cand.size());
    std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
    for (size_t j = 0; j < (size_t)k; ++j) {
      out_dist[a * k + j] = j < kk ? cand[j].first : std::numeric_limits<float>::infinity();
      out_ids[a * k + j] = j < kk ? cand[j].second : -1;
    }
  }
}

// IVFIndex.search with a metadata filter (Indexes/IVFIndex.swift:128,162-172): the rows of the probed lists are
// collected, the filter drops the ineligible ones (FilterEvaluator.filterVectors, :564-570), distances are computed
// for what is left and sorted.  The filter here is the bitmask form: row r passes for query a iff
// (row_masks[r] & query_masks[a]) != 0.
void vskref_ivf_search_filtered(const float* q, int64_t nq, const float* x, int64_t n, int d,
                                const float* centroids, int nlist, const int32_t* assign, int nprobe, int k,
                                const uint64_t* row_masks, const uint64_t* query_masks,
                                float* out_dist, int64_t* out_ids) {
  std::vector<std::vector<int64_t>> lists((size_t)nlist);
  for (int64_t r = 0; r < n; ++r) lists[assign[r]].push_back(r);
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t a = 0; a < nq; ++a) {
    const float* qa = q + a * d;
    std::vector<std::pair<float, int>> cd((size_t)nlist);
    for (int c = 0; c < nlist; ++c)
      cd[c] = {vskref_distance(VSKREF_EUCLIDEAN, qa, centroids + (size_t)c * d, d), c};
    int np = std::min(nprobe, nlist);
    std::partial_sort(cd.begin(), cd.begin() + np, cd.end());
    std::vector<std::pair<float, int64_t>> cand;
    for (int p = 0; p < np; ++p)
      for (int64_t r : lists[cd[p].second]) {
        if (row_masks && query_masks && (row_masks[r] & query_masks[a]) == 0) continue;   // filtered before distances
        cand.emplace_back(vskref_distance(VSKREF_EUCLIDEAN, qa, x + r * d, d), r);
      }
    size_t kk = std::min<size_t>((size_t)k, cand.size());
    std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
    for (size_t j = 0; j < (size_t)k; ++j) {
      out_dist[a * k + j] = j < kk ? cand[j].first : std::numeric_limits<float>::infinity();
      out_ids[a * k + j] = j < kk ? cand[j].second : -1;
    }
  }
}

// ---------------------------------------------------------------------------
// k-means++ initialisation, Clustering/KMeansClustering.swift:209-260:
//   first centroid  vectors[Int.random(in: 0..<n, using: SeedableRNG(seed))]
//   then, k-1 times: distances[i] = min over the chosen centroids of the un-squared euclidean distance (:397-428,
//                    a float sum in dimension order, sqrt); sumDistances = distances.reduce(0, +);
//                    probabilities[i] = distances[i] * distances[i] / sumDistances   (squared over the sum of
//                    UN-squared ones: they do not sum to one; kept as written);
//                    weightedSample with Float.random(in: 0..<1, using: SeedableRNG(seed + centroids.count)):
//                    the first index whose float running sum exceeds the draw, else the last index (:435-447).
// SeedableRNG is the 64-bit LCG of :480-491.  Swift's standard library maps a generator's output to
// Int.random(in: 0..<n) by multiply-high with rejection, and to Float.random(in: 0..<1) as 24 random bits * 2^-24
// (stdlib/public/core/Integers.swift, FloatingPointRandom.swift); those two mappings are restated from the published
// source of the standard library, which is not part of the reference tree: parity unpinned for them.
// ---------------------------------------------------------------------------
namespace {
struct SwiftLcg {
  uint64_t state;
  uint64_t next() { state = state * 2862933555777941757ull + 3037000493ull; return state; }
};
uint64_t swift_int_below(SwiftLcg& g, uint64_t n) {
  unsigned __int128 m = (unsigned __int128)g.next() * n;
  if ((uint64_t)m < n) {
    const uint64_t t = (0 - n) % n;
    while ((uint64_t)m < t) m = (unsigned __int128)g.next() * n;
  }
  return (uint64_t)(m >> 64);
}
float swift_unit_float(SwiftLcg& g) { return (float)((uint32_t)g.next() & 0xffffffu) * 5.9604645e-8f; }
}  // namespace

void vskref_kmeans_plusplus(const float* x, int64_t n, int d, int k, uint64_t seed, float* centroids, int64_t* picked) {
  SwiftLcg g0{seed};
  std::vector<int64_t> chosen;
  chosen.push_back((int64_t)swift_int_below(g0, (uint64_t)n));
  std::vector<float> dist((size_t)n, std::numeric_limits<float>::infinity());
  while ((int)chosen.size() < k) {
    const float* c = x + chosen.back() * d;   // min over all chosen = running min with the newest
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      float s = 0.f;
      for (int i = 0; i < d; ++i) {
        const float diff = x[r * d + i] - c[i];
        s += diff * diff;
      }
      dist[r] = std::min(dist[r], std::sqrt(s));
    }
    float sum = 0.f;
    for (int64_t r = 0; r < n; ++r) sum += dist[r];
    SwiftLcg g{seed + (uint64_t)chosen.size()};
    const float u = swift_unit_float(g);
    int64_t next = n - 1;
    float cumulative = 0.f;
    for (int64_t r = 0; r < n; ++r) {
      cumulative += dist[r] * dist[r] / sum;
      if (u < cumulative) { next = r; break; }
    }
    chosen.push_back(next);
  }
  for (int j = 0; j < k; ++j) {
    std::memcpy(centroids + (size_t)j * d, x + chosen[j] * d, sizeof(float) * (size_t)d);
    if (picked) picked[j] = chosen[j];
  }
}

// ---------------------------------------------------------------------------
// Scalar int8 quantiser, Quantization/ScalarQuantizer.swift:
//   statistics  :389-418   min / max over the values
//   parameters  :428-431   scale = 255/(max-min); offset = -min*scale - 128
//   encode      :251-270   code = truncate_toward_zero(x*scale + offset) as Int8
//                          (vDSP_vsmsa then vDSP_vfix8); here the multiply and
//                          the add are two separately rounded fp32 operations
//   decode      :568-580   x^ = (code - offset)/scale
// per_dim = 0 is the reference's behaviour: one (scale, offset) pair from the
// min/max over ALL values of the batch, replicated into scale[0..d).
// per_dim = 1 applies the same formulas column by column.
// ---------------------------------------------------------------------------
void vskref_sq8_train(const float* x, int64_t n, int d, int per_dim, float* scale, float* offset) {
  std::vector<float> mn((size_t)d, std::numeric_limits<float>::infinity());
  std::vector<float> mx((size_t)d, -std::numeric_limits<float>::infinity());
  for (int64_t r = 0; r < n; ++r)
    for (int i = 0; i < d; ++i) {
      mn[i] = std::min(mn[i], x[r * d + i]);
      mx[i] = std::max(mx[i], x[r * d + i]);
    }
  if (!per_dim) {
    float a = *std::min_element(mn.begin(), mn.end());
    float b = *std::max_element(mx.begin(), mx.end());
    std::fill(mn.begin(), mn.end(), a);
    std::fill(mx.begin(), mx.end(), b);
  }
  for (int i = 0; i < d; ++i) {
    float range = mx[i] - mn[i];
    scale[i] = 255.0f / range;
    offset[i] = -mn[i] * scale[i] - 128.0f;
  }
}

static inline int8_t fix8(float v) {
  // vDSP_vfix8: round toward zero.  Values outside [-128,127] cannot occur for
  // in-range inputs except by rounding at the top edge; saturate.
  float t = std::trunc(v);
  if (t > 127.0f) t = 127.0f;
  if (t < -128.0f) t = -128.0f;
  return (int8_t)t;
}

void vskref_sq8_encode(const float* x, int64_t n, int d, const float* scale, const float* offset,
                       int8_t* codes) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r)
    for (int i = 0; i < d; ++i) {
      float m = x[r * d + i] * scale[i];
      float v = m + offset[i];
      codes[r * d + i] = fix8(v);
    }
}

void vskref_sq8_decode(const int8_t* codes, int64_t n, int d, const float* scale,
                       const float* offset, float* x) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r)
    for (int i = 0; i < d; ++i) x[r * d + i] = ((float)codes[r * d + i] - offset[i]) / scale[i];
}

// Int8 scan.  The reference stores codes but never searches them; the scan is
// defined as the chosen metric between the fp32 query and the DEQUANTISED row
// (decode per ScalarQuantizer.swift:568-580, then the distance formulas above),
// exact ascending top-k, ties by row id.
void vskref_sq8_search(int metric, const float* q, int64_t nq, const int8_t* codes, int64_t n,
                       int d, const float* scale, const float* offset, int k, float* out_dist,
                       int64_t* out_ids) {
#pragma omp parallel
  {
    std::vector<float> row((size_t)d);
    std::vector<std::pair<float, int64_t>> cand;
#pragma omp for schedule(dynamic, 1)
    for (int64_t a = 0; a < nq; ++a) {
      cand.clear();
      for (int64_t r = 0; r < n; ++r) {
        for (int i = 0; i < d; ++i) row[i] = ((float)codes[r * d + i] - offset[i]) / scale[i];
        cand.emplace_back(vskref_distance(metric, q + a * d, row.data(), d), r);
      }
      size_t kk = std::min<size_t>((size_t)k, cand.size());
      std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
      for (size_t j = 0; j < (size_t)k; ++j) {
        out_dist[a * k + j] = j < kk ? cand[j].first : std::numeric_limits<float>::infinity();
        out_ids[a * k + j] = j < kk ? cand[j].second : -1;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Product quantisation, Quantization/ProductQuantizer.swift.
//   codebooks  [m][ksub][ds] with ds = d / m (Codebook.centroids, ProductQuantizerCodebook.swift:8-11)
//   encode     per segment the nearest codeword by squared L2 accumulated in dimension order, strict '<'
//              so the lowest code wins ties (Codebook.encode :12-30; shader productQuantize,
//              QuantizationShaders.metal:113-156)
//   decode     concatenation of the coded codewords (:152-163).  The optional norm rescale of :165-180 needs
//              the per-vector norm the Swift object carries in customData; it is not part of the code bytes
//              and is left to the caller.
//   tables     tables[s][c] = squared L2 between the query's segment and codeword c (:205-233)
//   distance   sqrt of the sum over segments, in segment order, of tables[s][code[s]]
//              (DistanceTables.computeDistance, ProductQuantizerTypes.swift:14-20; the same value as
//              computeAsymmetricDistance :341-356)
//   search     the reference has no scan over stored codes; defined here as exact ascending top-k of that
//              distance, ties by row id.
//   train      one k-means per segment (trainSegmentCodebook :266-312) with caller-supplied initial
//              codewords: the reference's k-means++ / mini-batch draw from Swift's RNG and cannot be
//              reproduced, so parity runs share the initial codebooks (as the IVF runs share centroids).
// ---------------------------------------------------------------------------
void vskref_pq_encode(const float* x, int64_t n, int d, int m, int ksub, const float* codebooks,
                      uint8_t* codes) {
  const int ds = d / m;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r)
    for (int s = 0; s < m; ++s) {
      const float* seg = x + r * d + (size_t)s * ds;
      float best = std::numeric_limits<float>::infinity();
      int bc = 0;
      for (int c = 0; c < ksub; ++c) {
        const float* cw = codebooks + ((size_t)s * ksub + c) * ds;
        float dist = 0.0f;
        for (int i = 0; i < ds; ++i) { float diff = seg[i] - cw[i]; dist += diff * diff; }
        if (dist < best) { best = dist; bc = c; }
      }
      codes[r * m + s] = (uint8_t)bc;
    }
}

void vskref_pq_decode(const uint8_t* codes, int64_t n, int d, int m, int ksub, const float* codebooks,
                      float* x) {
  const int ds = d / m;
  for (int64_t r = 0; r < n; ++r)
    for (int s = 0; s < m; ++s)
      std::memcpy(x + r * d + (size_t)s * ds, codebooks + ((size_t)s * ksub + codes[r * m + s]) * ds,
                  sizeof(float) * (size_t)ds);
}

void vskref_pq_tables(const float* q, int64_t nq, int d, int m, int ksub, const float* codebooks,
                      float* tables) {
  const int ds = d / m;
  for (int64_t a = 0; a < nq; ++a)
    for (int s = 0; s < m; ++s)
      for (int c = 0; c < ksub; ++c) {
        const float* seg = q + a * d + (size_t)s * ds;
        const float* cw = codebooks + ((size_t)s * ksub + c) * ds;
        float sum = 0.0f;
        for (int i = 0; i < ds; ++i) { float diff = seg[i] - cw[i]; sum += diff * diff; }
        tables[((size_t)a * m + s) * ksub + c] = sum;
      }
}

void vskref_pq_search(const float* q, int64_t nq, const uint8_t* codes, int64_t n, int d, int m, int ksub,
                      const float* codebooks, int k, float* out_dist, int64_t* out_ids) {
#pragma omp parallel
  {
    std::vector<float> table((size_t)m * ksub);
    std::vector<std::pair<float, int64_t>> cand;
#pragma omp for schedule(dynamic, 1)
    for (int64_t a = 0; a < nq; ++a) {
      vskref_pq_tables(q + a * d, 1, d, m, ksub, codebooks, table.data());
      cand.clear();
      for (int64_t r = 0; r < n; ++r) {
        float dist = 0.0f;
        for (int s = 0; s < m; ++s) dist += table[(size_t)s * ksub + codes[r * m + s]];
        cand.emplace_back(std::sqrt(dist), r);
      }
      size_t kk = std::min<size_t>((size_t)k, cand.size());
      std::partial_sort(cand.begin(), cand.begin() + kk, cand.end());
      for (size_t j = 0; j < (size_t)k; ++j) {
        out_dist[a * k + j] = j < kk ? cand[j].first : std::numeric_limits<float>::infinity();
        out_ids[a * k + j] = j < kk ? cand[j].second : -1;
      }
    }
  }
}

void vskref_pq_train(const float* x, int64_t n, int d, int m, int ksub, int iters, const float* init_codebooks,
                     float* codebooks) {
  const int ds = d / m;
  std::vector<float> seg((size_t)n * ds);
  std::vector<int32_t> asg((size_t)n);
  for (int s = 0; s < m; ++s) {
    for (int64_t r = 0; r < n; ++r)
      std::memcpy(&seg[(size_t)r * ds], x + r * d + (size_t)s * ds, sizeof(float) * (size_t)ds);
    vskref_kmeans(seg.data(), n, ds, ksub, iters, -1.0f, init_codebooks + (size_t)s * ksub * ds,
                  codebooks + (size_t)s * ksub * ds, asg.data(), nullptr, nullptr);
  }
}

// Merge of per-shard top-k lists: G lists of k (distance, global id) per query,
// ascending by (distance, id) — what a single unsharded search would return.
void vskref_merge_topk(const float* dist, const int64_t* ids, int g, int64_t nq, int k,
                       float* out_dist, int64_t* out_ids) {
  for (int64_t a = 0; a < nq; ++a) {
    std::vector<std::pair<float, int64_t>> all;
    for (int s = 0; s < g; ++s)
      for (int j = 0; j < k; ++j) {
        int64_t id = ids[((int64_t)s * nq + a) * k + j];
        if (id >= 0) all.emplace_back(dist[((int64_t)s * nq + a) * k + j], id);
      }
    std::sort(all.begin(), all.end());
    for (int j = 0; j < k; ++j) {
      bool ok = j < (int)all.size();
      out_dist[a * k + j] = ok ? all[j].first : std::numeric_limits<float>::infinity();
      out_ids[a * k + j] = ok ? all[j].second : -1;
    }
  }
}

int vskref_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
