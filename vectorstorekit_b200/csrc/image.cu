// Index image: a flat fp32, flat int8 or IVF index written to (and rebuilt from) one self-describing byte
// stream, so that a built index survives the process.  The reference exports an index as
// "VSTR" + version + JSON metadata + index data (API/VectorStore.swift:707-727) and its IVF export carries
// the centroids but not the inverted lists (Indexes/IVFIndex.swift:297-326, 612-616); this image keeps the same
// envelope and carries everything a search needs.
//
//   offset 0   "VSTR"
//   offset 4   version bytes 1,0,0,0
//   offset 8   u64 little-endian: length L of the metadata text
//   offset 16  metadata: JSON (ASCII), padded with spaces so that the data starts on a 64-byte boundary
//   then       the sections named in the metadata, in that order, raw little-endian arrays, each padded with
//              zero bytes to a multiple of 64
//
// Every section carries a 64-bit checksum computed ON THE DEVICE (before the download when saving, after the
// upload when loading), so a bit that flips on disk, in host memory or on the way over PCIe is caught.
//   checksum(bytes) = sum over i of mix(w_i + (i + 1) * 0x9E3779B97F4A7C15)  (mod 2^64)
// where w_i is the i-th little-endian 64-bit word of the section (the last one padded with zero bytes) and mix is
// the splitmix64 finaliser.  A sum of per-word hashes needs no ordering, so the reduction is deterministic.
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"

namespace vsk {

// adopters of uploaded storage, defined next to each index kind
int32_t flat_reserve(Index* ix, int64_t need);
int32_t flat_adopt_rows(Index* ix, int64_t n, bool has_masks);
int32_t sq8_reserve(Index* ix, int64_t need);
int32_t sq8_adopt_rows(Index* ix, int64_t n);
int32_t pq_adopt_rows(Index* ix, int64_t n);

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;
constexpr size_t kChunk = (size_t)32 << 20;   // staging buffer: 32 MiB of pinned host memory, two of them
constexpr int64_t kAlign = 64;

__host__ __device__ inline uint64_t mix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

// grid-stride over the whole words; thread 0 of block 0 adds the padded tail word
__global__ void __launch_bounds__(256) checksum_kernel(const uint64_t* __restrict__ words, int64_t nwords,
                                                       const uint8_t* __restrict__ tail, int tail_bytes,
                                                       unsigned long long* out) {
  uint64_t acc = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += stride)
    acc += mix64(__ldg(words + i) + (uint64_t)(i + 1) * kGolden);
  if (blockIdx.x == 0 && threadIdx.x == 0 && tail_bytes > 0) {
    uint64_t w = 0;
    for (int b = 0; b < tail_bytes; ++b) w |= (uint64_t)tail[b] << (8 * b);
    acc += mix64(w + (uint64_t)(nwords + 1) * kGolden);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ uint64_t part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint64_t s = 0;
    for (int w = 0; w < 8; ++w) s += part[w];
    atomicAdd(out, (unsigned long long)s);
  }
}

int32_t device_checksum(Ctx* ctx, const void* dev, int64_t bytes, uint64_t* out) {
  unsigned long long* acc = nullptr;
  VSK_TRY(dev_alloc(ctx, (void**)&acc, 8));
  cudaMemsetAsync(acc, 0, 8, ctx->stream);
  const int64_t nwords = bytes / 8;
  const int tail = (int)(bytes - nwords * 8);
  const unsigned grid = (unsigned)std::min<int64_t>(std::max<int64_t>(1, ceil_div(nwords, 256 * 8)),
                                                    (int64_t)ctx->prop.multiProcessorCount * 8);
  checksum_kernel<<<grid, 256, 0, ctx->stream>>>((const uint64_t*)dev, nwords, (const uint8_t*)dev + nwords * 8, tail, acc);
  ctx->stats.kernel_launches++;
  unsigned long long h = 0;
  cudaError_t e = cudaMemcpyAsync(&h, acc, 8, cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  dev_free(acc);
  if (e != cudaSuccess) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "checksum failed: %s", cudaGetErrorString(e));
  *out = (uint64_t)h;
  return VSK_OK;
}

// ---- byte sinks and sources ------------------------------------------------------------------
struct Sink {
  virtual ~Sink() {}
  virtual bool write(const void* p, size_t n) = 0;
};
struct FileSink : Sink {
  FILE* f;
  explicit FileSink(FILE* f_) : f(f_) {}
  bool write(const void* p, size_t n) override { return n == 0 || fwrite(p, 1, n, f) == n; }
};
struct MemSink : Sink {
  uint8_t* dst;
  int64_t cap, pos = 0;
  MemSink(void* d, int64_t c) : dst((uint8_t*)d), cap(c) {}
  bool write(const void* p, size_t n) override {
    if (pos + (int64_t)n > cap) return false;
    memcpy(dst + pos, p, n);
    pos += (int64_t)n;
    return true;
  }
};
struct Source {
  virtual ~Source() {}
  virtual bool read(void* p, size_t n) = 0;
};
struct FileSource : Source {
  FILE* f;
  explicit FileSource(FILE* f_) : f(f_) {}
  bool read(void* p, size_t n) override { return n == 0 || fread(p, 1, n, f) == n; }
};
struct MemSource : Source {
  const uint8_t* src;
  int64_t size, pos = 0;
  MemSource(const void* s, int64_t n) : src((const uint8_t*)s), size(n) {}
  bool read(void* p, size_t n) override {
    if (pos + (int64_t)n > size) return false;
    memcpy(p, src + pos, n);
    pos += (int64_t)n;
    return true;
  }
};

// ---- the sections of an index ------------------------------------------------------------------
struct Section {
  std::string name;
  void* dev = nullptr;
  int64_t bytes = 0;
  uint64_t checksum = 0;
};

const char* kind_name(int kind) {
  return kind == INDEX_FLAT_F32 ? "flat_f32" : kind == INDEX_FLAT_I8 ? "flat_i8" : kind == INDEX_IVF ? "ivf" : kind == INDEX_PQ ? "pq" : "?";
}
const char* metric_name(int m) {
  static const char* names[] = {"euclidean", "cosine", "dotProduct", "manhattan"};   // DistanceMetric raw values
  return (m >= 0 && m < 4) ? names[m] : "?";
}

std::vector<Section> sections_of(const Index* ix) {
  std::vector<Section> s;
  auto add = [&](const char* name, void* p, int64_t bytes) {
    Section x;
    x.name = name;
    x.dev = p;
    x.bytes = bytes;
    s.push_back(x);
  };
  const int64_t n = ix->n, d = ix->dim;
  if (ix->kind == INDEX_FLAT_F32) {
    add("rows", ix->rows, n * d * 4);
    if (ix->has_masks) add("masks", ix->masks, n * 8);
  } else if (ix->kind == INDEX_FLAT_I8) {
    add("sq_scale", ix->sq_scale, d * 4);
    add("sq_offset", ix->sq_offset, d * 4);
    add("codes", ix->codes, n * d);
  } else if (ix->kind == INDEX_IVF) {
    add("centroids", ix->centroids, (int64_t)ix->nlist * d * 4);
    add("list_offsets", ix->list_offsets, ((int64_t)ix->nlist + 1) * 8);
    add("list_rows", ix->list_rows, n * 4);
    add("assignments", ix->assign, n * 4);
    add("rows", ix->rows, n * d * 4);   // in list order
    if (ix->has_masks) add("masks", ix->masks, n * 8);   // in list order too
  } else if (ix->kind == INDEX_PQ) {
    add("pq_codebooks", ix->pq_codebooks, (int64_t)ix->pq_ksub * d * 4);   // [m][ksub][d / m]
    add("pq_codes", ix->pq_codes, n * ix->pq_m);
  }
  return s;
}

inline int64_t padded(int64_t b) { return ceil_div(b, kAlign) * kAlign; }

std::string metadata_text(const Index* ix, const std::vector<Section>& secs) {
  char buf[512];
  std::string m;
  snprintf(buf, sizeof buf,
           "{\"format\":\"vsk-b200-index-image\",\"format_version\":1,\"kind\":\"%s\",\"metric\":\"%s\","
           "\"dimensions\":%d,\"count\":%lld,\"id_base\":%lld,\"has_masks\":%s,\"nlist\":%d,\"pq_segments\":%d,"
           "\"pq_codebook_size\":%d,\"sections\":[",
           kind_name(ix->kind), metric_name(ix->metric), ix->dim, (long long)ix->n, (long long)ix->id_base,
           ix->has_masks ? "true" : "false", ix->nlist, ix->pq_m, ix->pq_ksub);
  m = buf;
  for (size_t i = 0; i < secs.size(); ++i) {
    snprintf(buf, sizeof buf, "%s{\"name\":\"%s\",\"bytes\":%lld,\"checksum\":\"%016llx\"}", i ? "," : "",
             secs[i].name.c_str(), (long long)secs[i].bytes, (unsigned long long)secs[i].checksum);
    m += buf;
  }
  m += "]}";
  // data starts on a 64-byte boundary: 16 header bytes + metadata length
  while ((16 + m.size()) % kAlign) m += ' ';
  return m;
}

struct Pinned {
  uint8_t* p[2] = {nullptr, nullptr};
  cudaEvent_t ev[2] = {nullptr, nullptr};
  ~Pinned() {
    for (int i = 0; i < 2; ++i) {
      if (p[i]) cudaFreeHost(p[i]);
      if (ev[i]) cudaEventDestroy(ev[i]);
    }
  }
  bool init() {
    for (int i = 0; i < 2; ++i) {
      if (cudaHostAlloc((void**)&p[i], kChunk, cudaHostAllocDefault) != cudaSuccess) return false;
      if (cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming) != cudaSuccess) return false;
    }
    return true;
  }
};

int32_t write_image(Index* ix, Sink& sink, int64_t* written) {
  Ctx* ctx = ix->ctx;
  if (ix->n <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "the index is empty");
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::vector<Section> secs = sections_of(ix);
  if (secs.empty()) return fail(ctx, VSK_ERR_EXPORT_FAILED, "this kind of index has no image format");
  for (auto& s : secs) VSK_TRY(device_checksum(ctx, s.dev, s.bytes, &s.checksum));
  const std::string meta = metadata_text(ix, secs);
  uint8_t head[16] = {'V', 'S', 'T', 'R', 1, 0, 0, 0};
  const uint64_t len = meta.size();
  for (int b = 0; b < 8; ++b) head[8 + b] = (uint8_t)(len >> (8 * b));
  int64_t total = 0;
  if (!sink.write(head, 16) || !sink.write(meta.data(), meta.size()))
    return fail(ctx, VSK_ERR_EXPORT_FAILED, "write failed (header)");
  total += 16 + (int64_t)meta.size();
  Pinned pin;
  if (!pin.init()) return fail(ctx, VSK_ERR_OUT_OF_MEMORY, "pinned staging buffers");
  static const uint8_t zeros[kAlign] = {0};
  for (auto& s : secs) {
    // download chunk i+1 while chunk i is written
    const int64_t chunks = ceil_div(s.bytes, (int64_t)kChunk);
    auto issue = [&](int64_t c) {
      const int64_t off = c * (int64_t)kChunk, nb = std::min<int64_t>(kChunk, s.bytes - off);
      cudaMemcpyAsync(pin.p[c & 1], (const uint8_t*)s.dev + off, (size_t)nb, cudaMemcpyDeviceToHost, ctx->stream);
      cudaEventRecord(pin.ev[c & 1], ctx->stream);
    };
    if (chunks > 0) issue(0);
    for (int64_t c = 0; c < chunks; ++c) {
      VSK_CUDA(ctx, cudaEventSynchronize(pin.ev[c & 1]));
      if (c + 1 < chunks) issue(c + 1);
      const int64_t off = c * (int64_t)kChunk, nb = std::min<int64_t>(kChunk, s.bytes - off);
      if (!sink.write(pin.p[c & 1], (size_t)nb)) {
        cudaStreamSynchronize(ctx->stream);
        return fail(ctx, VSK_ERR_EXPORT_FAILED, "write failed in section %s", s.name.c_str());
      }
    }
    ctx->stats.d2h_bytes += s.bytes;
    const int64_t pad = padded(s.bytes) - s.bytes;
    if (pad && !sink.write(zeros, (size_t)pad)) return fail(ctx, VSK_ERR_EXPORT_FAILED, "write failed (padding)");
    total += padded(s.bytes);
  }
  if (written) *written = total;
  return VSK_OK;
}

// ---- a reader for the metadata text: objects, arrays, strings, integers, true/false -----------------
struct Json {
  enum Type { NUL, BOOL, NUM, STR, ARR, OBJ } type = NUL;
  bool b = false;
  long long num = 0;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;
  const Json* get(const char* k) const {
    auto it = obj.find(k);
    return it == obj.end() ? nullptr : &it->second;
  }
};
struct JsonReader {
  const char* p;
  const char* end;
  int depth = 0;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(const char* s) {
    const size_t n = strlen(s);
    if ((size_t)(end - p) < n || memcmp(p, s, n) != 0) return false;
    p += n;
    return true;
  }
  bool string(std::string& out) {
    if (p >= end || *p != '"') return false;
    ++p;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return false;
      }
      out += *p++;
    }
    if (p >= end) return false;
    ++p;
    return true;
  }
  bool value(Json& v) {
    if (++depth > 8) return false;
    ws();
    if (p >= end) return false;
    bool ok = false;
    if (*p == '{') {
      ++p;
      v.type = Json::OBJ;
      ws();
      if (p < end && *p == '}') { ++p; ok = true; }
      else
        for (;;) {
          std::string k;
          ws();
          if (!string(k)) break;
          ws();
          if (p >= end || *p++ != ':') break;
          Json c;
          if (!value(c)) break;
          v.obj[k] = c;
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == '}') { ++p; ok = true; }
          break;
        }
    } else if (*p == '[') {
      ++p;
      v.type = Json::ARR;
      ws();
      if (p < end && *p == ']') { ++p; ok = true; }
      else
        for (;;) {
          Json c;
          if (!value(c)) break;
          v.arr.push_back(c);
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == ']') { ++p; ok = true; }
          break;
        }
    } else if (*p == '"') {
      v.type = Json::STR;
      ok = string(v.str);
    } else if (lit("true")) {
      v.type = Json::BOOL; v.b = true; ok = true;
    } else if (lit("false")) {
      v.type = Json::BOOL; v.b = false; ok = true;
    } else if (lit("null")) {
      v.type = Json::NUL; ok = true;
    } else {
      const char* s = p;
      if (p < end && *p == '-') ++p;
      while (p < end && *p >= '0' && *p <= '9') ++p;
      if (p > s && !(p - s == 1 && *s == '-') && p - s < 20) {
        v.type = Json::NUM;
        v.num = atoll(std::string(s, p).c_str());
        ok = true;
      }
    }
    --depth;
    return ok;
  }
};

int32_t upload_section(Ctx* ctx, Source& src, Pinned& pin, void* dev, int64_t bytes, const char* name) {
  const int64_t chunks = ceil_div(bytes, (int64_t)kChunk);
  for (int64_t c = 0; c < chunks; ++c) {
    const int64_t off = c * (int64_t)kChunk, nb = std::min<int64_t>(kChunk, bytes - off);
    if (c >= 2) VSK_CUDA(ctx, cudaEventSynchronize(pin.ev[c & 1]));   // the copy that last used this buffer
    if (!src.read(pin.p[c & 1], (size_t)nb)) {
      cudaStreamSynchronize(ctx->stream);
      return fail(ctx, VSK_ERR_IMPORT_FAILED, "the image ends inside section %s", name);
    }
    VSK_CUDA(ctx, cudaMemcpyAsync((uint8_t*)dev + off, pin.p[c & 1], (size_t)nb, cudaMemcpyHostToDevice, ctx->stream));
    VSK_CUDA(ctx, cudaEventRecord(pin.ev[c & 1], ctx->stream));
  }
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.h2d_bytes += bytes;
  uint8_t skip[kAlign];
  const int64_t pad = padded(bytes) - bytes;
  if (pad && !src.read(skip, (size_t)pad)) return fail(ctx, VSK_ERR_IMPORT_FAILED, "the image ends after section %s", name);
  return VSK_OK;
}

int32_t read_image(Ctx* ctx, Source& src, Index** out) {
  *out = nullptr;
  uint8_t head[16];
  if (!src.read(head, 16)) return fail(ctx, VSK_ERR_IMPORT_FAILED, "the image is shorter than its header");
  if (memcmp(head, "VSTR", 4) != 0) return fail(ctx, VSK_ERR_IMPORT_FAILED, "not an index image (magic)");
  if (head[4] != 1) return fail(ctx, VSK_ERR_IMPORT_FAILED, "image version %d is not supported", (int)head[4]);
  uint64_t len = 0;
  for (int b = 0; b < 8; ++b) len |= (uint64_t)head[8 + b] << (8 * b);
  if (len == 0 || len > (1u << 20)) return fail(ctx, VSK_ERR_IMPORT_FAILED, "implausible metadata length");
  std::string meta((size_t)len, '\0');
  if (!src.read(&meta[0], (size_t)len)) return fail(ctx, VSK_ERR_IMPORT_FAILED, "the image ends inside its metadata");
  Json root;
  JsonReader rd{meta.data(), meta.data() + meta.size()};
  if (!rd.value(root) || root.type != Json::OBJ) return fail(ctx, VSK_ERR_IMPORT_FAILED, "metadata is not valid JSON");
  auto str = [&](const char* k) -> std::string {
    const Json* j = root.get(k);
    return j && j->type == Json::STR ? j->str : std::string();
  };
  auto num = [&](const char* k, long long dflt) -> long long {
    const Json* j = root.get(k);
    return j && j->type == Json::NUM ? j->num : dflt;
  };
  if (str("format") != "vsk-b200-index-image" || num("format_version", 0) != 1)
    return fail(ctx, VSK_ERR_IMPORT_FAILED, "metadata does not describe an index image of this library");
  const std::string kind = str("kind"), metric_s = str("metric");
  int metric = -1;
  for (int m = 0; m < 4; ++m)
    if (metric_s == metric_name(m)) metric = m;
  const long long dim = num("dimensions", 0), n = num("count", 0), nlist = num("nlist", 0);
  const Json* hm = root.get("has_masks");
  const bool has_masks = hm && hm->type == Json::BOOL && hm->b;
  if (metric < 0 || dim <= 0 || dim > (1 << 20) || n <= 0 || n > 0x7fffffffLL || nlist < 0 || nlist > 0x7fffffffLL)
    return fail(ctx, VSK_ERR_IMPORT_FAILED, "metadata holds an impossible shape");
  const Json* sj = root.get("sections");
  if (!sj || sj->type != Json::ARR) return fail(ctx, VSK_ERR_IMPORT_FAILED, "metadata lists no sections");
  struct Want { std::string name; int64_t bytes; uint64_t checksum; };
  std::vector<Want> want;
  for (const Json& e : sj->arr) {
    const Json *jn = e.get("name"), *jb = e.get("bytes"), *jc = e.get("checksum");
    if (!jn || !jb || !jc || jn->type != Json::STR || jb->type != Json::NUM || jc->type != Json::STR)
      return fail(ctx, VSK_ERR_IMPORT_FAILED, "a section entry is malformed");
    want.push_back({jn->str, (int64_t)jb->num, (uint64_t)strtoull(jc->str.c_str(), nullptr, 16)});
  }

  // build the empty index of that kind and learn where its sections go
  Index* ix = nullptr;
  int32_t st = VSK_OK;
  if (kind == "flat_f32") {
    vsk_index* h = nullptr;
    st = vsk_flat_create(reinterpret_cast<vsk_ctx*>(ctx), metric, (int32_t)dim, &h);
    ix = reinterpret_cast<Index*>(h);
    if (st == VSK_OK) st = flat_reserve(ix, n);
  } else if (kind == "flat_i8") {
    ix = new Index();
    ix->ctx = ctx;
    ix->kind = INDEX_FLAT_I8;
    ix->metric = metric;
    ix->dim = (int32_t)dim;
    if ((st = dev_alloc(ctx, (void**)&ix->sq_scale, (size_t)dim * 4)) == VSK_OK &&
        (st = dev_alloc(ctx, (void**)&ix->sq_offset, (size_t)dim * 4)) == VSK_OK)
      st = sq8_reserve(ix, n);
  } else if (kind == "ivf") {
    if (nlist <= 0) return fail(ctx, VSK_ERR_IMPORT_FAILED, "an IVF image without lists");
    ix = new Index();
    ix->ctx = ctx;
    ix->kind = INDEX_IVF;
    ix->metric = VSK_METRIC_EUCLIDEAN;
    ix->dim = (int32_t)dim;
    ix->nlist = (int32_t)nlist;
    ix->capacity = n;
    if ((st = dev_alloc(ctx, (void**)&ix->centroids, (size_t)nlist * dim * 4)) == VSK_OK &&
        (st = dev_alloc(ctx, (void**)&ix->list_offsets, (size_t)(nlist + 1) * 8)) == VSK_OK &&
        (st = dev_alloc(ctx, (void**)&ix->list_rows, (size_t)n * 4)) == VSK_OK &&
        (st = dev_alloc(ctx, (void**)&ix->assign, (size_t)n * 4)) == VSK_OK &&
        (st = has_masks ? dev_alloc(ctx, (void**)&ix->masks, (size_t)n * 8) : VSK_OK) == VSK_OK)
      st = dev_alloc(ctx, (void**)&ix->rows, (size_t)n * dim * 4);
  } else if (kind == "pq") {
    const long long pm = num("pq_segments", 0), pk = num("pq_codebook_size", 0);
    if (pm <= 0 || dim % pm != 0 || pk < 2 || pk > 256) return fail(ctx, VSK_ERR_IMPORT_FAILED, "an impossible product quantiser");
    ix = new Index();
    ix->ctx = ctx;
    ix->kind = INDEX_PQ;
    ix->metric = VSK_METRIC_EUCLIDEAN;
    ix->dim = (int32_t)dim;
    ix->pq_m = (int32_t)pm;
    ix->pq_ksub = (int32_t)pk;
    if ((st = dev_alloc(ctx, (void**)&ix->pq_codebooks, (size_t)pk * dim * 4)) == VSK_OK) st = pq_reserve(ix, n);
  } else {
    return fail(ctx, VSK_ERR_IMPORT_FAILED, "unknown index kind '%s'", kind.c_str());
  }
  auto bail = [&](int32_t s) {
    if (ix) vsk_index_destroy(reinterpret_cast<vsk_index*>(ix));
    return s;
  };
  if (st != VSK_OK) return bail(st);
  ix->n = n;   // sections_of sizes the sections from it
  ix->has_masks = has_masks;
  std::vector<Section> secs = sections_of(ix);
  ix->n = 0;
  if (secs.size() != want.size()) return bail(fail(ctx, VSK_ERR_IMPORT_FAILED, "the image's sections do not fit its kind"));
  Pinned pin;
  if (!pin.init()) return bail(fail(ctx, VSK_ERR_OUT_OF_MEMORY, "pinned staging buffers"));
  for (size_t i = 0; i < secs.size(); ++i) {
    if (secs[i].name != want[i].name || secs[i].bytes != want[i].bytes)
      return bail(fail(ctx, VSK_ERR_IMPORT_FAILED, "section %s: unexpected name or size", want[i].name.c_str()));
    if ((st = upload_section(ctx, src, pin, secs[i].dev, secs[i].bytes, secs[i].name.c_str())) != VSK_OK) return bail(st);
    uint64_t h = 0;
    if ((st = device_checksum(ctx, secs[i].dev, secs[i].bytes, &h)) != VSK_OK) return bail(st);
    if (h != want[i].checksum)
      return bail(fail(ctx, VSK_ERR_IMPORT_FAILED, "section %s is corrupt: checksum %016llx, expected %016llx",
                       secs[i].name.c_str(), (unsigned long long)h, (unsigned long long)want[i].checksum));
  }
  // derived state
  if (ix->kind == INDEX_FLAT_F32) st = flat_adopt_rows(ix, n, has_masks);
  else if (ix->kind == INDEX_FLAT_I8) st = sq8_adopt_rows(ix, n);
  else if (ix->kind == INDEX_PQ) st = pq_adopt_rows(ix, n);
  else {
    ix->n = n;
    ix->list_offsets_h.resize((size_t)nlist + 1);
    cudaError_t e = cudaMemcpy(ix->list_offsets_h.data(), ix->list_offsets, (size_t)(nlist + 1) * 8, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) st = fail(ctx, VSK_ERR_EXECUTION_FAILED, "%s", cudaGetErrorString(e));
    // the offsets must describe n rows in ascending order, or a later scan would read outside the arrays
    if (st == VSK_OK) {
      bool good = ix->list_offsets_h.front() == 0 && ix->list_offsets_h.back() == n;
      for (size_t l = 0; l + 1 < ix->list_offsets_h.size() && good; ++l)
        good = ix->list_offsets_h[l] <= ix->list_offsets_h[l + 1];
      if (!good) st = fail(ctx, VSK_ERR_IMPORT_FAILED, "list offsets are not a partition of the rows");
    }
  }
  if (st != VSK_OK) return bail(st);
  ix->id_base = num("id_base", 0);
  *out = ix;
  return VSK_OK;
}

}  // namespace
}  // namespace vsk

using namespace vsk;

extern "C" {

int32_t vsk_index_info_get(vsk_index* i, vsk_index_info* info) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix || !info) return VSK_ERR_INVALID_INPUT;
  info->kind = ix->kind == INDEX_FLAT_F32 ? VSK_INDEX_FLAT_F32 : ix->kind == INDEX_FLAT_I8 ? VSK_INDEX_FLAT_I8 : ix->kind == INDEX_PQ ? VSK_INDEX_PQ : VSK_INDEX_IVF;
  info->pq_segments = ix->pq_m;
  info->pq_codebook_size = ix->pq_ksub;
  info->metric = ix->metric;
  info->dimensions = ix->dim;
  info->count = ix->n;
  info->id_base = ix->id_base;
  info->nlist = ix->nlist;
  info->has_masks = ix->has_masks ? 1 : 0;
  return VSK_OK;
}

int32_t vsk_index_image_size(vsk_index* i, int64_t* bytes) {
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix || !bytes) return VSK_ERR_INVALID_INPUT;
  if (ix->n <= 0) return fail(ix->ctx, VSK_ERR_EMPTY_INPUT, "the index is empty");
  std::vector<Section> secs = sections_of(ix);
  int64_t total = 16 + (int64_t)metadata_text(ix, secs).size();   // checksums have a fixed width
  for (auto& s : secs) total += padded(s.bytes);
  *bytes = total;
  return VSK_OK;
}

int32_t vsk_index_export(vsk_index* i, void* dst, int64_t capacity, int64_t* written) {
  VSK_TRACE("vsk_index_export");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  if (!dst || capacity <= 0) return fail(ix->ctx, VSK_ERR_INVALID_INPUT, "null or empty destination");
  MemSink sink(dst, capacity);
  return write_image(ix, sink, written);
}

int32_t vsk_index_import(vsk_ctx* c, const void* src, int64_t bytes, vsk_index** out) {
  VSK_TRACE("vsk_index_import");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  *out = nullptr;
  if (!src || bytes <= 0) return fail(ctx, VSK_ERR_EMPTY_INPUT, "no image bytes");
  MemSource source(src, bytes);
  return read_image(ctx, source, reinterpret_cast<Index**>(out));
}

int32_t vsk_index_save(vsk_index* i, const char* path) {
  VSK_TRACE("vsk_index_save");
  Index* ix = reinterpret_cast<Index*>(i);
  if (!ix) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ix->ctx->device);
  if (!path) return fail(ix->ctx, VSK_ERR_INVALID_INPUT, "null path");
  FILE* f = fopen(path, "wb");
  if (!f) return fail(ix->ctx, VSK_ERR_EXPORT_FAILED, "cannot open %s for writing", path);
  FileSink sink(f);
  int32_t st = write_image(ix, sink, nullptr);
  if (fclose(f) != 0 && st == VSK_OK) st = fail(ix->ctx, VSK_ERR_EXPORT_FAILED, "closing %s failed", path);
  if (st != VSK_OK) remove(path);   // never leave half an image behind
  return st;
}

int32_t vsk_index_load(vsk_ctx* c, const char* path, vsk_index** out) {
  VSK_TRACE("vsk_index_load");
  Ctx* ctx = reinterpret_cast<Ctx*>(c);
  if (!ctx || !out) return VSK_ERR_INVALID_INPUT;
  cudaSetDevice(ctx->device);
  *out = nullptr;
  if (!path) return fail(ctx, VSK_ERR_INVALID_INPUT, "null path");
  FILE* f = fopen(path, "rb");
  if (!f) return fail(ctx, VSK_ERR_IMPORT_FAILED, "cannot open %s", path);
  FileSource source(f);
  const int32_t st = read_image(ctx, source, reinterpret_cast<Index**>(out));
  fclose(f);
  return st;
}

}  // extern "C"
