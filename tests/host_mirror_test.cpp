// Compiles the header-only C++ host layer and links it against the library.  Without a B200 the
// strategy must refuse to initialise (there is no CPU path); with one, a tiny search is checked
// against values worked out by hand.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "../vectorstorekit_b200/host/vsk.hpp"

int main() {
  vsk::CUDAAcceleratorStrategy strategy;
  std::shared_ptr<vsk::CUDAComputeDevice> dev;
  try {
    dev = strategy.initialize();
  } catch (const vsk::DeviceNotAvailable&) {
    std::puts("no-device");
    return 0;
  }
  try {
    vsk::metric_id(vsk::DistanceMetric::hamming);
    return 2;
  } catch (const vsk::UnsupportedOperation&) {
  }
  const float rows[] = {1, 0, 0, 0, 0, 1, 0, 0, 1, 1, 1, 1};
  const float q[] = {1, 0, 0, 0};
  vsk::CUDAAccelerationEngine engine(dev);
  auto d = engine.computeDistances(q, rows, 3, 4, vsk::DistanceMetric::euclidean);
  if (std::fabs(d[0]) > 1e-6f || std::fabs(d[1] - std::sqrt(2.0f)) > 1e-4f) return 3;
  auto m = engine.computeDistances(q, rows, 3, 4, vsk::DistanceMetric::manhattan);
  if (std::fabs(m[2] - 3.0f) > 1e-4f) return 4;
  vsk::FlatIndex ix(dev, 4, vsk::DistanceMetric::cosine);
  ix.add(rows, 3);
  auto r = ix.batchSearch(q, 1, 2);
  if (r.ids[0] != 0 || r.ids[1] != 2) return 5;
  // export -> import: the rebuilt index answers the same
  auto image = ix.exportBinary();
  if (image.size() < 16 || std::memcmp(image.data(), "VSTR", 4) != 0) return 6;
  vsk::FlatIndex back(dev, image.data(), (int64_t)image.size());
  auto r2 = back.batchSearch(q, 1, 2);
  if (back.count() != 3 || r2.ids != r.ids || r2.distances != r.distances) return 7;
  image[image.size() - 60] ^= 1;   // inside the rows section (48 bytes of rows + 16 of padding end the image)
  try {
    vsk::FlatIndex broken(dev, image.data(), (int64_t)image.size());
    return 8;
  } catch (const vsk::ImportFailed&) {
  }
  // the awaited form: two submissions queue behind one another, both futures resolve to the blocking call's result
  {
    auto f1 = ix.batchSearchAsync(q, 1, 2);
    auto f2 = ix.batchSearchAsync(q, 1, 2);
    auto a1 = f1.get();
    auto a2 = f2.get();
    dev->wait();
    if (a1.ids != r.ids || a1.distances != r.distances || a2.ids != r.ids) return 12;
    auto bad = ix.batchSearchAsync(q, 1, 0);   // k = 0: the failure arrives through the future
    try {
      bad.get();
      return 13;
    } catch (const vsk::Error&) {
    }
    try {
      dev->wait();                              // ...and once more as the first failure since the last wait
      return 14;
    } catch (const vsk::Error&) {
    }
  }
  // the caller's layer: string ids and metadata back, the filter as a bit (the reference's filter test:
  // category == "A" keeps v1 and v3, Tests/VectorStoreKitTests/IVFIndexTests.swift:536-590)
  {
    vsk::VectorStore store(dev, 4, vsk::DistanceMetric::euclidean, true);
    const uint64_t categoryA = 1;
    store.add({{"v1", {1, 0, 0, 0}, "{\"category\":\"A\"}", categoryA},
               {"v2", {0.9f, 0.1f, 0, 0}, "{\"category\":\"B\"}", 0},
               {"v3", {0, 1, 0, 0}, "{\"category\":\"A\"}", categoryA}});
    auto all = store.search(q, 3);
    if (all.size() != 3 || all[0].id != "v1" || all[1].id != "v2" || all[2].id != "v3") return 15;
    auto onlyA = store.search(q, 3, categoryA);
    if (onlyA.size() != 2 || onlyA[0].id != "v1" || onlyA[1].id != "v3" ||
        onlyA[1].metadata.find("\"A\"") == std::string::npos) return 16;
    if (std::fabs(onlyA[1].distance - std::sqrt(2.0f)) > 1e-4f) return 17;
  }
  // a communicator of one rank: the sharded call is the plain search, in both layouts
  dev->joinCommunicator(1, 0, {});
  int64_t first = -1;
  auto s1 = ix.shardedSearch(q, 1, 2, nullptr, false, &first);
  auto s2 = ix.shardedSearch(q, 1, 2, nullptr, true);
  if (first != 0 || s1.ids != r.ids || s1.distances != r.distances || s2.ids != r.ids) return 11;
  dev->leaveCommunicator();
  // IVF mirror: two centroids, rows filed in two inserts (the second without a rebuild), a filter on the second
  // batch's rows, and the one-rank sharded form (the reference's flow: IVFIndexTests.swift:60-140, :536-590)
  {
    vsk::IVFIndex ivf(dev, 4, 2, 2, 5);
    const float train[] = {1, 0, 0, 0, 0, 1, 0, 0, 0.9f, 0.1f, 0, 0, 0.1f, 0.9f, 0, 0};
    try {
      ivf.batchSearch(q, 1, 1);
      return 18;                                // search before train must be refused
    } catch (const vsk::NotTrained&) {
    }
    ivf.train(train, 4);
    const uint64_t m1[] = {1, 1}, m2[] = {2, 2};
    ivf.insert(train, 2, m1);                   // rows 0, 1
    ivf.insert(train + 8, 2, m2);               // rows 2, 3 behind them
    auto a = ivf.batchSearch(q, 1, 4);
    if (a.ids[0] != 0 || a.ids[1] != 2 || a.ids[2] != 3 || a.ids[3] != 1) return 19;
    const uint64_t only2[] = {2};
    auto f = ivf.batchSearch(q, 1, 2, false, only2);
    if (f.ids[0] != 2 || f.ids[1] != 3) return 20;
    dev->joinCommunicator(1, 0, {});
    auto sh = ivf.shardedSearch(q, 1, 4, nullptr, true);
    dev->leaveCommunicator();
    if (sh.ids != a.ids || sh.distances != a.distances) return 21;
  }
  // product quantiser: 2 segments of 2 dimensions, 16 codewords; row 1 sits on codewords (3, 5)
  vsk::ProductQuantizer pq(dev, 4, 2, 4);
  std::vector<float> cb(2 * 16 * 2);
  for (size_t i = 0; i < cb.size(); ++i) cb[i] = (float)((i * 7) % 13) - 6.0f + 0.01f * (float)i;
  pq.setCodebooks(cb);
  const float pr[] = {cb[0], cb[1], cb[32], cb[33], cb[3 * 2], cb[3 * 2 + 1], cb[32 + 5 * 2], cb[32 + 5 * 2 + 1]};
  auto codes = pq.encodeBatch(pr, 2);
  if (codes[0] != 0 || codes[1] != 0 || codes[2] != 3 || codes[3] != 5) return 9;
  vsk::PQIndex pix(dev, pq);
  pix.add(codes.data(), 2);
  auto pr2 = pix.batchSearch(pr + 4, 1, 2);
  if (pr2.ids[0] != 1 || pr2.distances[0] != 0.0f || pr2.ids[1] != 0) return 10;
  std::puts("ok");
  return 0;
}
