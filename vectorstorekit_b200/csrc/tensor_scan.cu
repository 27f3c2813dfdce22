// Tensor-core search path for euclidean, cosine and dot-product over a flat fp32 index.
//
//   coarse   queries x rows contraction on the 5th-generation tensor cores (tcgen05.mma, fp16
//            operands, fp32 accumulators in tensor memory), operands staged by TMA into
//            128-byte-swizzled shared-memory tiles.  The epilogue turns each accumulator into a
//            coarse distance and appends only the rows at or below the query's running threshold
//            to that query's candidate list: the query x row matrix never reaches HBM.
//   bound    every operand is the fp16 rounding of a power-of-two scaled fp32 value, and the
//            rounding residuals are measured when the operands are made, so |coarse - exact| <= eps
//            holds with eps computed per query from measured norms (see prep kernels).
//   rerank   the few candidates per query that can still be in the true top-k are re-scored with
//            the reference's direct fp32 formulas (AccelerateOptimizer.swift:251-383) and sorted.
//   proof    a query's result is accepted only if  c_k + 2 eps < t,  where c_k is the k-th smallest
//            coarse value kept and t the threshold below which no row was ever dropped; then every
//            true top-k row is among the re-scored candidates.  Otherwise the query is re-run on
//            the fp32 scan.
//
// Kernel structure (one CTA per SM, persistent over 128-query x 256-row tiles, query tile fastest
// so that concurrently running CTAs share the same rows in L2):
//   warp 0      TMA producer: 4-stage ring of {128 x 64 query, 256 x 64 row} fp16 tiles
//   warp 1      tensor-memory allocation; one lane issues tcgen05.mma (M128 N256 K16 x 4 per stage)
//   warps 2..   epilogue (8 warps for long contractions, 16 up to d = 256): tcgen05.ld of the thread's
//               accumulator row (one query per thread; the warps of a lane quarter split the tile's columns),
//               threshold filter, candidate append; double-buffered accumulators (2 x 256 columns)
// The same kernel scans the probed lists of an IVF index (tile-table mode: an explicit list of tiles over a
// query operand gathered per (query, list) pair) and assigns rows to centroids for k-means (argmin mode and a
// threshold mode whose tiles walk the centroids for a fixed block of rows).
// Every mbarrier wait is bounded: on expiry the kernel raises an error word, stops issuing work,
// drains its copies and frees tensor memory, and the host call returns VSK_ERR_TIMEOUT.
#include <cuda.h>
#include <math_constants.h>

#include <cmath>

#include "common.cuh"
#include "tensor_scan.cuh"
#include "tc_ptx.cuh"

namespace vsk {
namespace {

using namespace tc;   // tile geometry and the tcgen05 / TMA / mbarrier wrappers (tc_ptx.cuh)
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;              // operand ring: 4 stages of 48 KB
constexpr int RING_BYTES = STAGES * STAGE_BYTES;
// (A variant on pairs of CTAs - tcgen05.mma.cta_group::2, a 256-query tile, each CTA staging half of the rows -
// was built and measured 2 - 3 % slower on the headline workload: the kernel is bound by the power cap, not by
// operand traffic from L2.  It was removed.)
// Warp 0 is the TMA producer, warp 1 the MMA issuer, then EW epilogue warps: EW / 4 per tensor-memory lane quarter,
// each taking one of EW / 4 equal parts of the tile's columns.  EW = 8 for long contractions (the epilogue hides
// behind the MMAs, and fewer warps cost less issue and power); EW = 16 for short ones (d <= 256), where a tile's
// MMAs take about a microsecond and the epilogue warps' serial chain of tensor-memory loads sets the pace.
template <int EW> struct Epi {
  static constexpr int WARPS = EW;
  static constexpr int PARTS = EW / 4;
  static constexpr int COLS = TN / PARTS;      // columns per epilogue warp
  static constexpr int GROUPS = COLS / 32;
  static constexpr int THREADS = 64 + 32 * EW;
};

template <int EW>
struct TcSmemT {
  // stage buffers first: each must start on a 1024-byte boundary for the 128B swizzle
  uint8_t ring[RING_BYTES];
  float beta[2][EW][Epi<EW>::COLS];   // per accumulator buffer and epilogue warp: its columns' per-row terms
  uint32_t masks[EW * 32][Epi<EW>::GROUPS + 1];  // per epilogue thread: pass bits of its values (padded row)
  float hitval[EW * 32][Epi<EW>::GROUPS + 1];    // ... and per group the value of its last hit
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  volatile int abort_flag;
};
template <int EW> constexpr size_t tc_smem_bytes() { return sizeof(TcSmemT<EW>) + 1024; }   // + alignment slack

struct TcArgs {
  int64_t nq;                 // queries (list positions)
  int64_t row_begin, row_end; // rows of this launch
  int32_t kblocks;            // dim16 / 64
  int32_t k16_last;           // K16 steps of the last K block that hold operand columns (the rest is padding); 0 = all 4
  int32_t stage_kblocks;      // K blocks per ring stage: 1 (four stages of 48 KB) or 2 (two stages of 96 KB: half the
                              // hand-overs between producer, MMA issuer and ring)
  int mode;                   // SCAN_DENSE or SCAN_THRESHOLD
  const float* alpha;         // device scalar: value = alpha * acc + beta[row]
  const float* beta;          // [n] or null (treated as 0)
  CandLists cand;
  int32_t cap;                // keys per candidate list (SCAN_THRESHOLD)
  unsigned long long* best;   // SCAN_ARGMIN: [nq] smallest (value, row) key, pre-set to all ones
  int32_t row_tile_fastest;   // tile order: 0 = query tile fastest (rows are the operand streamed once),
                              //             1 = row tile fastest (the "queries" are the operand streamed once)
  int32_t* err;               // device error word
  // Tile-table mode (IVF list scan): the launch walks an explicit list of tiles instead of the full
  // (query tile) x (row tile) grid, and the "query" operand holds one row per (query, probed list) pair, grouped
  // by list.  tiles[t] = {first pair, first row, valid rows | in-pilot-window << 30, valid pairs};
  // pair_info[p] = list position of the pair's query | remainder item << 31 (the rest of a query's nearest list
  // after the pilot window: such a pair skips the tiles inside the window).
  const int4* tiles;          // or null
  int64_t num_tiles;
  const uint32_t* pair_info;
  const float* pair_thr;      // [pairs] coarse threshold of the pair's query for this launch
  // Filter (HAS_MASK kernels): operand row r may be appended for query q iff (row_masks[r] & q_masks[q]) != 0.
  const uint64_t* row_masks;  // [rows of the row operand]
  const uint64_t* q_masks;    // [nq] by list position
  // Bounded waits: polls before a wait gives up (0 = WAIT_LIMIT).  stall_kblock >= 0 (testing only): the producer of
  // CTA 0 leaves out the copies of that k-block of its first tile, so that the consumer's wait for them runs out and
  // the time-out path (error word, abort flag, drain, tensor-memory release, VSK_ERR_TIMEOUT) can be exercised.
  uint32_t wait_limit;
  int32_t stall_kblock;
};


template <int MODE, bool HAS_BETA, bool HAS_MASK, int EW>
__global__ void __launch_bounds__(Epi<EW>::THREADS, 1)
tc_scan_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_x, TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  using TcSmem = TcSmemT<EW>;
  constexpr int EPI_WARPS = EW, EPI_COLS = Epi<EW>::COLS, EPI_GROUPS = Epi<EW>::GROUPS, EPI_PARTS = Epi<EW>::PARTS;
  TcSmem* sm = reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t unit = blockIdx.x;
  const int64_t units = gridDim.x;
  constexpr int QT = TM;  // queries per tile
  const uint32_t wait_limit = a.wait_limit ? a.wait_limit : WAIT_LIMIT;
  const int kps = a.stage_kblocks == 2 ? 2 : 1;   // K blocks per ring stage
  const int nstages = STAGES / kps;

  const int64_t qtiles = (a.nq + QT - 1) / QT;
  const int64_t ntiles = (a.row_end - a.row_begin + TN - 1) / TN;
  const int64_t tiles = qtiles * ntiles;
  // i-th tile of this unit.  Query-tile-fastest order interleaves units over the tile list (units that run
  // together read the same rows).  In row-tile-fastest order a unit OWNS whole query tiles and walks all their
  // row tiles in turn, so a query's running state (slot count, best key) stays in its thread's registers.
  auto tile_at = [&](int64_t i, int64_t& qt, int64_t& nt) -> bool {
    if (a.tiles) {   // explicit tile list: nt is the tile's index in the table
      const int64_t t = unit + i * units;
      if (t >= a.num_tiles) return false;
      nt = t;
      qt = 0;
      return true;
    }
    if (a.row_tile_fastest) {
      const int64_t qi = i / ntiles;
      nt = i - qi * ntiles;
      qt = unit + qi * units;
      return qt < qtiles;
    }
    const int64_t t = unit + i * units;
    if (t >= tiles) return false;
    nt = t / qtiles;
    qt = t - nt * qtiles;
    return true;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm->full[s], 1);
      mbar_init(&sm->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm->tmem_full[b], 1);
      mbar_init(&sm->tmem_empty[b], EPI_WARPS);
    }
    mbar_init(&sm->drain, 1);
    sm->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t issued = 0;       // bit s: a copy into stage s was issued ...
      uint32_t issued_ph = 0;    // ... with this full-barrier parity
      bool ok = true;
      // tile-table mode: the entry of the next tile is loaded while this tile's copies are issued, so that the
      // table look-up (a global load) is not on the producer's critical path
      int4 entry_next = make_int4(0, 0, 0, 0);
      if (a.tiles && unit < a.num_tiles) entry_next = __ldg(&a.tiles[unit]);
      for (int64_t i = 0; ok; ++i) {
        int64_t qt, nt;
        if (!tile_at(i, qt, nt)) break;
        const int4 entry = entry_next;
        if (a.tiles && nt + units < a.num_tiles) entry_next = __ldg(&a.tiles[nt + units]);
        const int32_t qrow = a.tiles ? entry.x : (int32_t)(qt * QT);
        const int32_t xrow = a.tiles ? entry.y : (int32_t)(a.row_begin + nt * TN);
        for (int kb = 0; kb < a.kblocks; kb += kps) {
          if (!mbar_wait(&sm->empty[s], ph ^ 1, &sm->abort_flag, a.err, 1, wait_limit)) { ok = false; break; }
          uint8_t* st = sm->ring + s * kps * STAGE_BYTES;
          const int nkb = min(kps, a.kblocks - kb);
          if (a.stall_kblock >= 0 && unit == 0 && i == 0 && kb == a.stall_kblock) {
            // testing only: this stage is never filled, the consumer's bounded wait for it runs out
          } else {
            mbar_expect_tx(&sm->full[s], (uint32_t)(nkb * STAGE_BYTES));
            for (int j = 0; j < nkb; ++j) {
              tma_load_2d(st + j * STAGE_BYTES, &map_q, &sm->full[s], (kb + j) * TK, qrow);
              tma_load_2d(st + j * STAGE_BYTES + A_BYTES, &map_x, &sm->full[s], (kb + j) * TK, xrow);
            }
            issued |= 1u << s;
            issued_ph = (issued_ph & ~(1u << s)) | (ph << s);
          }
          if (++s == nstages) { s = 0; ph ^= 1; }
        }
      }
      // copies still in flight must land before the CTA's shared memory is released
      for (int i = 0; i < STAGES; ++i)
        if (issued & (1u << i)) {
          for (uint32_t it = 0; it < wait_limit; ++it) {
            if (mbar_try_wait(&sm->full[i], (issued_ph >> i) & 1)) break;
            __nanosleep(64);
          }
        }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // One lane, loop state in 32-bit registers, the number of tiles worked out once (the tile's coordinates, which
    // cost a 64-bit division per tile, are of no use to this role).  A converged warp with an elected lane and a
    // look-ahead at the next stage's barriers was measured 2 - 3 % slower here and is not used.
    if (lane == 0) {
      int64_t count;
      if (a.tiles) count = unit < a.num_tiles ? (a.num_tiles - unit + units - 1) / units : 0;
      else if (a.row_tile_fastest) count = unit < qtiles ? ((qtiles - unit + units - 1) / units) * ntiles : 0;
      else count = unit < tiles ? (tiles - unit + units - 1) / units : 0;
      const uint32_t ring_lo = desc_lo(smem_u32(sm->ring));
      const uint32_t full0 = smem_u32(&sm->full[0]), empty0 = smem_u32(&sm->empty[0]), tfull0 = smem_u32(&sm->tmem_full[0]);
      const int last_nk4 = a.k16_last > 0 ? a.k16_last : TK / 16;
      uint32_t s = 0, ph = 0, acc = 0, aph = 0;
      bool ok = true;
      for (int64_t left = count; ok && left > 0; --left) {
        if (!mbar_wait(&sm->tmem_empty[acc], aph ^ 1, &sm->abort_flag, a.err, 2, wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * (uint32_t)TN;
        for (int kb0 = 0; kb0 < a.kblocks; kb0 += kps) {
          if (!mbar_wait(&sm->full[s], ph, &sm->abort_flag, a.err, 3, wait_limit)) { ok = false; break; }
          tc_fence_after();
          const int nkb = min(kps, a.kblocks - kb0);
          for (int j = 0; j < nkb; ++j) {
            const int kb = kb0 + j;
            const uint32_t a_lo = ring_lo + (uint32_t)((s * kps + j) * (STAGE_BYTES >> 4));
            const uint32_t b_lo = a_lo + (uint32_t)(A_BYTES >> 4);
            const int nk4 = kb == a.kblocks - 1 ? last_nk4 : TK / 16;
#pragma unroll
            for (int k4 = 0; k4 < TK / 16; ++k4) {
              // 16 fp16 = 32 bytes further along K inside the swizzle atom: +2 in 16-byte units
              if (k4 < nk4)
                tc_mma(tmem_d, desc_pack(a_lo + (uint32_t)(k4 * 2), kDescHi), desc_pack(b_lo + (uint32_t)(k4 * 2), kDescHi), kIdesc,
                       (kb | k4) ? 1u : 0u);
            }
          }
          tc_commit_a(empty0 + s * 8u);   // the stage is free once these MMAs have read it
          if (++s == (uint32_t)nstages) { s = 0; ph ^= 1u; }
        }
        if (ok) tc_commit_a(tfull0 + acc * 8u);
        aph = acc ? aph ^ 1u : aph;
        acc ^= 1u;
      }
      // all issued MMAs must retire before tensor memory is freed
      tc_commit(&sm->drain);
      for (uint32_t it = 0; it < wait_limit; ++it) {
        if (mbar_try_wait(&sm->drain, 0)) break;
        __nanosleep(64);
      }
    }
  } else {
    // ---------------- epilogue: one query per thread, half of the tile's columns per warp ----------------
    const int quarter = warp & 3;                 // tensor-memory lanes this warp may read
    const int et = quarter * 32 + lane;           // row of the tile owned by this thread
    const int ew = warp - 2;                      // epilogue warp 0..7
    const int part = ew >> 2;                     // which part of the tile's columns this warp takes
    const int c0 = part * EPI_GROUPS;             // first 32-column group of that part
    const float alpha = __ldg(a.alpha);
    int64_t local = 0;
    bool ok = true;
    int run_cnt = 0;                 // row-tile-fastest order: keys this thread has stored for its query so far
    float run_bv = CUDART_INF_F;     // ... and its best value / row so far (SCAN_ARGMIN)
    int64_t run_bn = 0;
    // Tile-table mode: the tile's entry, then this lane's pair and threshold (both indexed by the entry), are a
    // chain of dependent global loads.  The chain is pipelined over the tiles: the entry is loaded two tiles ahead,
    // the pair and threshold one tile ahead, so neither load is waited for (with short contractions the epilogue,
    // not the MMA, sets the pace).  pair_info / pair_thr are padded by one tile, so the loads need no bounds test.
    struct Ahead { int4 e; uint32_t info; float thr; };
    auto entry_at = [&](int64_t i) {
      const int64_t t = unit + i * units;
      return (a.tiles && t < a.num_tiles) ? __ldg(&a.tiles[t]) : make_int4(0, 0, 0, 0);
    };
    auto pair_at = [&](const int4& e) {
      Ahead h{e, 0u, -CUDART_INF_F};
      if (a.tiles) {
        h.info = __ldg(a.pair_info + e.x + et);
        if (MODE == SCAN_THRESHOLD) h.thr = __ldg(a.pair_thr + e.x + et);
      }
      return h;
    };
    Ahead ahead = pair_at(entry_at(0));
    int4 entry_next = entry_at(1);
    for (;; ++local) {
      int64_t qt, nt;
      if (!ok || !tile_at(local, qt, nt)) break;
      const int acc = (int)(local & 1);
      const uint32_t aph = (uint32_t)((local >> 1) & 1);
      const Ahead cur = ahead;
      if (a.tiles) {
        ahead = pair_at(entry_next);
        entry_next = entry_at(local + 2);
      }
      int64_t q = qt * QT + et;
      const bool owned = a.row_tile_fastest != 0;
      if (owned && nt == 0) { run_cnt = 0; run_bv = CUDART_INF_F; run_bn = 0; }
      int64_t n0 = a.row_begin + nt * TN;
      int64_t row_end = a.row_end;
      bool qok = q < a.nq;
      float thr_tile = -CUDART_INF_F;
      if (a.tiles) {
        n0 = cur.e.y;
        row_end = (int64_t)cur.e.y + (cur.e.z & 0x3fffffff);
        qok = et < cur.e.w;
        q = cur.info & 0x7fffffffu;
        // a remainder item (the rest of a query's nearest list) skips the tiles inside the pilot window
        const bool skip = (cur.info >> 31) != 0u && ((cur.e.z >> 30) & 1) != 0;
        if (qok && !skip) thr_tile = cur.thr;
      }
      // The tile's per-row terms; each warp stages its own copy, so no CTA-wide barrier is needed.  The first tile
      // loads them directly; after that they are fetched one tile ahead into registers (the loads fly while this
      // tile is processed) and stored to the other buffer at the end of the iteration.
      float beta_next[EPI_COLS / 32];
      if (HAS_BETA) {
        if (local == 0) {
          for (int i = lane; i < EPI_COLS; i += 32)
            sm->beta[acc][ew][i] = (n0 + c0 * 32 + i < row_end) ? __ldg(a.beta + n0 + c0 * 32 + i) : 0.f;
          __syncwarp();
        }
        int64_t nqt, nnt, nn0 = 0, nrow_end = 0;
        if (tile_at(local + 1, nqt, nnt)) {
          if (a.tiles) { nn0 = ahead.e.y; nrow_end = (int64_t)ahead.e.y + (ahead.e.z & 0x3fffffff); }
          else { nn0 = a.row_begin + nnt * TN; nrow_end = a.row_end; }
        }
#pragma unroll
        for (int i = 0; i < EPI_COLS / 32; ++i) {
          const int64_t r = nn0 + c0 * 32 + lane + 32 * i;
          beta_next[i] = r < nrow_end ? __ldg(a.beta + r) : 0.f;
        }
      }
      float thr = CUDART_INF_F;
      if (MODE == SCAN_THRESHOLD && qok) thr = a.tiles ? thr_tile : a.cand.thr[q];
      uint64_t qm = 0ull;   // this query's filter mask: a row is eligible iff (row mask & qm) != 0
      if (HAS_MASK && qok) qm = __ldg(a.q_masks + q);
      // every lane of the warp must take part in the wait result
      bool got = mbar_wait(&sm->tmem_full[acc], aph, &sm->abort_flag, a.err, 4, wait_limit);
      got = __all_sync(0xffffffffu, got);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TN);
      if (MODE == SCAN_DENSE) {
#pragma unroll 1
        for (int c = c0; c < c0 + EPI_GROUPS; ++c) {
          float v[32];
          tc_ld32(trow + (uint32_t)(c * 32), v);
          const int64_t nc = n0 + c * 32;
          if (!qok) continue;
          uint64_t* dst = a.cand.keys + q * kCandCap + (nc - a.row_begin);
          // a query's keys are contiguous (16-byte aligned at every even column): two keys per store halve the
          // number of scattered store transactions, which is what bounds this epilogue
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float v0 = HAS_BETA ? fmaf(v[j], alpha, sm->beta[acc][ew][(c - c0) * 32 + j]) : v[j] * alpha;
            const float v1 = HAS_BETA ? fmaf(v[j + 1], alpha, sm->beta[acc][ew][(c - c0) * 32 + j + 1]) : v[j + 1] * alpha;
            uint64_t k0 = make_key(v0, (uint32_t)(nc + j)), k1 = make_key(v1, (uint32_t)(nc + j + 1));
            if (HAS_MASK) {
              // the same row mask for every lane (a broadcast load); an ineligible row leaves an empty slot
              if (nc + j < a.row_end && (__ldg(a.row_masks + nc + j) & qm) == 0ull) k0 = kEmptyKey;
              if (nc + j + 1 < a.row_end && (__ldg(a.row_masks + nc + j + 1) & qm) == 0ull) k1 = kEmptyKey;
            }
            if (nc + j + 1 < a.row_end)
              *reinterpret_cast<ulonglong2*>(dst + j) = make_ulonglong2(k0, k1);
            else if (nc + j < a.row_end)
              dst[j] = k0;
          }
        }
      } else if (MODE == SCAN_ARGMIN) {
        // smallest (value, row) key of this query over the tile's 256 rows, merged into best[q]
        float bv = CUDART_INF_F;
        int bj = 0;
#pragma unroll 1
        for (int c = c0; c < c0 + EPI_GROUPS; ++c) {
          float v[32];
          tc_ld32(trow + (uint32_t)(c * 32), v);
          const int64_t left = a.row_end - (n0 + c * 32);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = HAS_BETA ? fmaf(v[j], alpha, sm->beta[acc][ew][(c - c0) * 32 + j]) : v[j] * alpha;
            if (j < left && val < bv) { bv = val; bj = c * 32 + j; }   // strict '<': the lowest row wins ties
          }
        }
        if (owned) {
          if (bv < run_bv) { run_bv = bv; run_bn = n0 + bj; }   // row tiles come in ascending order: '<' keeps the lowest row
          if (nt == ntiles - 1 && qok && run_bv < CUDART_INF_F)
            atomicMin(a.best + q, (unsigned long long)make_key(run_bv, (uint32_t)run_bn));
        } else if (qok && bv < CUDART_INF_F) {
          atomicMin(a.best + q, (unsigned long long)make_key(bv, (uint32_t)(n0 + bj)));
        }
      } else {
        // Pass 1: which of this query's 256 values pass the threshold (one bit each).  A thread then
        // reserves all its slots with ONE atomic per tile; pass 2 re-reads the accumulator groups that
        // have a passing value and stores the keys.  A per-value atomic would serialise the warp on an
        // L2 round trip for every column in which any of its 32 queries has a hit.
        // The masks live in shared memory so that both loops stay rolled (small code, no dynamic
        // register indexing).
        uint32_t* m = sm->masks[ew * 32 + lane];
        float* mv = sm->hitval[ew * 32 + lane];
        int cnt = 0;
#pragma unroll 1
        for (int c = c0; c < c0 + EPI_GROUPS; ++c) {
          float v[32];
          tc_ld32(trow + (uint32_t)(c * 32), v);
          const int64_t left = row_end - (n0 + c * 32);   // columns of this group inside the launch (tile)
          // Cheap test first: the smallest of the group's 32 values against the threshold.  Most groups of a late
          // chunk hold no hit for any of the warp's queries and then cost two instructions per value, not five.
          float vmin = CUDART_INF_F;
          if (!HAS_BETA && alpha < 0.f) {
            // value = alpha * accumulator with alpha < 0: the smallest value is alpha times the largest accumulator
            // (the multiplication is monotone, so this is the same number), one instruction per value; the values
            // themselves are only formed for a group that has a hit
            float amax = v[0];
#pragma unroll
            for (int j = 1; j < 32; ++j) amax = fmaxf(amax, v[j]);
            vmin = amax * alpha;
            if (left >= 32 && !__any_sync(0xffffffffu, qok && vmin <= thr)) {
              m[c - c0] = 0u;
              continue;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= alpha;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = HAS_BETA ? fmaf(v[j], alpha, sm->beta[acc][ew][(c - c0) * 32 + j]) : v[j] * alpha;
              vmin = fminf(vmin, v[j]);
            }
            if (left >= 32 && !__any_sync(0xffffffffu, qok && vmin <= thr)) {
              m[c - c0] = 0u;
              continue;
            }
          }
          const uint32_t colmask = left >= 32 ? 0xffffffffu : (left > 0 ? ((1u << (int)left) - 1u) : 0u);
          uint32_t bits = 0;
          float hv = 0.f;   // the value of the (last) hit: all that pass 2 needs when a query has one hit in the group
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float val = v[j];
            const bool hit = val <= thr;
            bits |= hit ? (1u << j) : 0u;
            hv = hit ? val : hv;
          }
          bits = qok ? (bits & colmask) : 0u;
          if (HAS_MASK) {
            // Only hits are tested against the filter (a few per query and tile once the threshold is tight): the
            // row masks of a tile are 2 KB and stay in L1 for the CTA's 128 queries.
            uint32_t b = bits;
            while (b) {
              const int j = __ffs((int)b) - 1;
              b &= b - 1u;
              if ((__ldg(a.row_masks + n0 + c * 32 + j) & qm) == 0ull) bits &= ~(1u << j);
            }
          }
          m[c - c0] = bits;
          mv[c - c0] = hv;
          cnt += __popc(bits);
        }
        // Slot reservation.  Interleaved order: one atomic per tile.  Owned order: this warp's half of the
        // columns appends to its own half of the query's list, counted in a register; the two 16-bit counts are
        // stored after the last row tile.
        int base = 0;
        const int cap_here = owned ? a.cap / EPI_PARTS : a.cap;
        if (owned) base = run_cnt;
        else if (cnt) base = atomicAdd(&a.cand.count[q], cnt);
#pragma unroll 1
        for (int c = c0; c < c0 + EPI_GROUPS; ++c) {
          const uint32_t bits = m[c - c0];
          const uint32_t colbits = __reduce_or_sync(0xffffffffu, bits);   // columns in which any query has a hit
          if (colbits == 0u) continue;
          if (!HAS_MASK && !__any_sync(0xffffffffu, (bits & (bits - 1u)) != 0u) && n0 + c * 32 + 32 <= row_end) {
            // no query has more than one hit in this (whole) group: its value was kept by pass 1
            const uint32_t ok1 = (bits != 0u && base < cap_here) ? 1u : 0u;
            const uint64_t key1 = make_key(mv[c - c0], (uint32_t)(n0 + c * 32 + (__ffs((int)bits) - 1)));
            uint64_t* d1 = a.cand.keys + q * a.cap + (owned ? part * cap_here : 0) + base;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.ne.u32 p, %2, 0;\n\t"
                "@p st.global.u64 [%0], %1;\n\t}" ::"l"(d1),
                "l"(key1), "r"(ok1)
                : "memory");
            base += bits != 0u ? 1 : 0;
            continue;
          }
          float v[32];
          tc_ld32(trow + (uint32_t)(c * 32), v);
          const int64_t nc = n0 + c * 32;
          uint64_t* dst = a.cand.keys + q * a.cap + (owned ? part * cap_here : 0) + base;
          // Straight-line code with predicated stores: a branch around every store makes the warp wait out each
          // store's address chain in turn (measured: four times the cost of this form at 1 hit in 150 values).
          // Only whole octets of columns without any hit are skipped, on a warp-uniform test.
#pragma unroll
          for (int o = 0; o < 4; ++o) {
            if (((colbits >> (8 * o)) & 0xffu) == 0u) continue;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int j = o * 8 + jj;
              const float val = HAS_BETA ? fmaf(v[j], alpha, sm->beta[acc][ew][(c - c0) * 32 + j]) : v[j] * alpha;
              const int rank = __popc(bits & ((1u << j) - 1u));
              const uint32_t ok = (((bits >> j) & 1u) != 0u && base + rank < cap_here) ? 1u : 0u;
              const uint64_t key = make_key(val, (uint32_t)(nc + j));
              asm volatile(
                  "{\n\t.reg .pred p;\n\t"
                  "setp.ne.u32 p, %2, 0;\n\t"
                  "@p st.global.u64 [%0], %1;\n\t}" ::"l"(dst + rank),
                  "l"(key), "r"(ok)
                  : "memory");
            }
          }
          base += __popc(bits);
        }
        if (owned) {
          run_cnt += cnt;
          if (nt == ntiles - 1 && qok)
            reinterpret_cast<unsigned char*>(a.cand.count)[q * 4 + part] = (unsigned char)min(run_cnt, 255);
        }
      }
      if (HAS_BETA) {
#pragma unroll
        for (int i = 0; i < EPI_COLS / 32; ++i) sm->beta[acc ^ 1][ew][lane + 32 * i] = beta_next[i];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->tmem_empty[acc]);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- nearest-centroid assignment with a STATIONARY centroid block ---------------------------------------
// k-means assignment is a contraction of 10^7 data rows against a few thousand centroids with a short inner
// dimension (d = 128: two or three 64-wide k-blocks).  In the general kernel every 128 x 256 tile re-fetches both
// operands from L2 - 96 KB for 8 Mflop - and at that ratio the L2 -> shared-memory fill, not the tensor pipe, sets the
// pace (measured: 1.44 us per tile against 0.53 us of MMAs).  Here a CTA keeps one block of 256 centroids (all its
// k-blocks, up to 128 KB) resident in shared memory and streams 128-row data tiles past it: 16 KB per k-block and
// tile, a third of the traffic (a sixth with the row term folded in), so the MMAs set the pace again.
//   grid      blocks of 256 centroids x groups of CTAs; CTA (b, g) holds centroid block b and takes data tiles
//             g, g + groups, ...  (more blocks than SMs: a CTA takes several blocks in turn)
//   warp 0    TMA producer: the centroid block once, then the data tiles through a ring whose stage holds a whole
//             data tile (a K block where a tile is too large for two such stages); fold columns that begin a K block
//             of their own travel as a 16-column tile
//   warp 1    tcgen05.mma issuer: per data tile M128 N256 K16 x 4 per k-block against the resident block; it looks at
//             the next tile's barriers while this tile's last MMAs are still to be issued
//   warps 2.. epilogue (16 warps): the centroid's |c|^2 / 2 rides inside the contraction (fold columns), so a value
//             is alpha * accumulator and "no hit in these eight columns" is their largest accumulator against a bar.
//             Threshold mode: a hit (rare: the threshold is the row's previous assignment plus the error band)
//             is logged as {row, centroid} in the CTA's own stretch of a log, its slot taken from a shared-memory
//             counter; arg-min mode (first iteration): one atomicMin per row, centroid block and column part.
// Every mbarrier wait is bounded like the general kernel's.
constexpr int AS_EW = 16;
constexpr int AS_THREADS = 64 + 32 * AS_EW;
constexpr int AS_MAX_KB = 4;                       // k-blocks of the resident block (d + 16 fold columns <= 256)
constexpr int AS_RING_BYTES = 216 * 1024;          // resident block + data-tile stages
constexpr int AS_MAX_STAGES = 8;
// The 16-column fold tile is only loaded and issued in whole-tile stages: two such stages must fit beside the largest
// resident block that has one (the condition is tightest at the largest number of K blocks).
static_assert(2 * ((AS_MAX_KB - 1) * A_BYTES + A_NARROW_BYTES) <= AS_RING_BYTES - ((AS_MAX_KB - 1) * B_BYTES + B_NARROW_BYTES),
              "a 16-column fold tile implies whole-tile stages");

struct AsSmem {
  uint8_t ring[AS_RING_BYTES];   // [kblocks x 32 KB centroid block][stages x 16 KB data k-blocks]
  uint64_t a_full[AS_MAX_STAGES];
  uint64_t a_empty[AS_MAX_STAGES];
  uint64_t b_full, b_empty;
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  volatile int abort_flag;
  int log_n;                     // hits this CTA has logged so far
};
constexpr size_t kAsSmemBytes = sizeof(AsSmem) + 1024;

struct AsArgs {
  int64_t n;                  // data rows
  int32_t k;                  // centroids
  int32_t kblocks;            // dim16 / 64, <= AS_MAX_KB
  int32_t k16_last;           // K16 steps of the last K block that hold operand columns; 0 = all 4
  int32_t max_stages;         // measurement: cap on the data-tile stages (0 = as many as fit)
  int32_t narrow_ok;          // the two 16-column tensor maps are valid (see `narrow` in the kernel)
  int32_t groups;             // CTAs per centroid block (1 when there are more blocks than CTAs)
  const float* alpha;         // value = alpha * accumulator = |c|^2 - 2 x.c
  const float* thr;           // [n] SCAN_THRESHOLD: a centroid is listed for a row iff value <= thr[row]
  // SCAN_THRESHOLD: every hit is logged as {row, centroid} in this CTA's own stretch of the log; the slot comes from a
  // shared-memory counter, so an append never waits for a round trip to L2 (with 32 rows x 64 columns per warp and
  // step, half of the steps hold a hit somewhere: a global atomic per hit made the epilogue wait out its latency)
  uint2* log;                 // [gridDim.x][log_cap]
  int32_t* log_count;         // [gridDim.x] entries written (capped); a CTA that ran out of room raises err = 9
  int64_t log_cap;            // entries per CTA = log_total / gridDim.x (set at launch)
  int64_t log_total;
  unsigned long long* best;   // [n] SCAN_ARGMIN: smallest (value, centroid) key, pre-set to all ones
  int32_t* err;
  uint32_t wait_limit;
};

// The accumulator a value must reach to be a hit: alpha * acc <= thr with alpha < 0 holds for every acc >= thr / alpha;
// thr * (1 / alpha) and the product alpha * acc each differ from the exact quotient by a few units in the last place,
// so the bar is lowered by 2^-20 of its size (and a denormal's worth): no hit of the product form is lost.
__device__ __forceinline__ float as_bar(float thr, float inv_alpha) {
  const float b = thr * inv_alpha;
  return b - fabsf(b) * 9.5367431640625e-7f - 1e-37f;
}

template <int MODE>
__global__ void __launch_bounds__(AS_THREADS, 1)
assign_scan_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_c,
                   const __grid_constant__ CUtensorMap map_xn, const __grid_constant__ CUtensorMap map_cn, AsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  AsSmem* sm = reinterpret_cast<AsSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t wait_limit = a.wait_limit ? a.wait_limit : WAIT_LIMIT;
  const int nb = (a.k + TN - 1) / TN;                       // centroid blocks
  const int64_t qtiles = (a.n + TM - 1) / TM;               // data tiles
  // When only the first K16 step of the last K block holds operand columns (d a multiple of 64: the 16 fold columns
  // start a block of their own), that block is fetched and kept as a 16-column tile (32-byte swizzle: 4 KB of a data
  // tile, 8 KB of the centroid block) instead of 64 columns of which 48 are zeros: a quarter less to fetch per data
  // tile at d = 128, and room for four whole-tile stages instead of two.
  const bool narrow = a.narrow_ok != 0 && a.max_stages == 0 && a.k16_last == 1 && a.kblocks >= 2;
  const int nfull = narrow ? a.kblocks - 1 : a.kblocks;   // K blocks held as 64-column tiles
  const int bres_bytes = nfull * B_BYTES + (narrow ? B_NARROW_BYTES : 0);
  const int tile_bytes = nfull * A_BYTES + (narrow ? A_NARROW_BYTES : 0);
  // A stage of the data ring holds ALL K blocks of a data tile when two such stages fit (one wait, one batch of MMAs
  // and one commit per tile instead of per K block); otherwise, or when max_stages asks for it, one K block.
  const int skb = (a.max_stages == 0 && 2 * tile_bytes <= AS_RING_BYTES - bres_bytes) ? a.kblocks : 1;
  const int stage_bytes = skb == a.kblocks ? tile_bytes : A_BYTES;
  int stages = min(AS_MAX_STAGES, (AS_RING_BYTES - bres_bytes) / stage_bytes);
  if (a.max_stages > 0) stages = max(2, min(stages, a.max_stages));
  // this CTA's centroid blocks and its share of the data tiles
  const bool one_block = a.groups >= 1 && nb <= (int)gridDim.x;
  const int b_first = one_block ? (int)(blockIdx.x % nb) : (int)blockIdx.x;
  const int b_step = one_block ? (1 << 30) : (int)gridDim.x;
  const int64_t t_first = one_block ? (int64_t)(blockIdx.x / nb) : 0;
  const int64_t t_step = one_block ? a.groups : 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < AS_MAX_STAGES; ++s) {
      mbar_init(&sm->a_full[s], 1);
      mbar_init(&sm->a_empty[s], 1);
    }
    mbar_init(&sm->b_full, 1);
    mbar_init(&sm->b_empty, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm->tmem_full[b], 1);
      mbar_init(&sm->tmem_empty[b], AS_EW);
    }
    mbar_init(&sm->drain, 1);
    sm->abort_flag = 0;
    sm->log_n = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;
  uint8_t* a_ring = sm->ring + bres_bytes;
  uint2* my_log = MODE == SCAN_THRESHOLD ? a.log + (int64_t)blockIdx.x * a.log_cap : nullptr;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0, bph = 0;
      uint32_t issued = 0, issued_ph = 0;
      bool b_issued = false;
      uint32_t b_issued_ph = 0;
      bool ok = true;
      for (int b = b_first; ok && b < nb; b += b_step) {
        // the resident block may be replaced once every MMA that read the previous one has retired
        if (!mbar_wait(&sm->b_empty, bph ^ 1, &sm->abort_flag, a.err, 5, wait_limit)) { ok = false; break; }
        mbar_expect_tx(&sm->b_full, (uint32_t)bres_bytes);
        for (int kb = 0; kb < nfull; ++kb) tma_load_2d(sm->ring + kb * B_BYTES, &map_c, &sm->b_full, kb * TK, b * TN);
        if (narrow) tma_load_2d(sm->ring + nfull * B_BYTES, &map_cn, &sm->b_full, nfull * TK, b * TN);
        b_issued = true;
        b_issued_ph = bph;
        bph ^= 1;
        for (int64_t t = t_first; ok && t < qtiles; t += t_step) {
          for (int kb = 0; kb < a.kblocks; kb += skb) {
            if (!mbar_wait(&sm->a_empty[s], ph ^ 1, &sm->abort_flag, a.err, 1, wait_limit)) { ok = false; break; }
            mbar_expect_tx(&sm->a_full[s], (uint32_t)stage_bytes);
            const int nj = skb == a.kblocks ? nfull : 1;
            for (int j = 0; j < nj; ++j)
              tma_load_2d(a_ring + s * stage_bytes + j * A_BYTES, &map_x, &sm->a_full[s], (kb + j) * TK, (int32_t)(t * TM));
            if (narrow) tma_load_2d(a_ring + s * stage_bytes + nfull * A_BYTES, &map_xn, &sm->a_full[s], nfull * TK, (int32_t)(t * TM));
            issued |= 1u << s;
            issued_ph = (issued_ph & ~(1u << s)) | (ph << s);
            if (++s == stages) { s = 0; ph ^= 1; }
          }
        }
      }
      // copies still in flight must land before the CTA's shared memory is released
      if (b_issued)
        for (uint32_t it = 0; it < wait_limit; ++it) {
          if (mbar_try_wait(&sm->b_full, b_issued_ph)) break;
          __nanosleep(64);
        }
      for (int i = 0; i < stages; ++i)
        if (issued & (1u << i))
          for (uint32_t it = 0; it < wait_limit; ++it) {
            if (mbar_try_wait(&sm->a_full[i], (issued_ph >> i) & 1)) break;
            __nanosleep(64);
          }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // Measured with clock stamps in this warp: an M128 N256 K16 MMA executes in 128 cycles and the pipe queues only a
    // few, so the nine MMAs of a d = 128 tile are issued over about 1 250 cycles, and every cycle this warp then spends
    // before the next tile's first MMA (commits, loop, two barrier waits of 200 - 250 cycles each even when the barrier
    // has long completed) is a cycle the pipe idles: 2 130 cycles per tile at first, 1 152 of them MMA execution.
    if (skb == a.kblocks) {
      // A whole data tile per ring stage (the usual case): one lane, all loop state in 32-bit registers.  What this
      // thread executes between the last MMA of a tile and the first of the next is time the tensor pipe idles once
      // its short queue has drained, so the barriers of the next tile are looked at (one test, never a wait) while
      // this tile's last MMAs are still to be issued, and nothing is recomputed that can be carried along.
      if (lane == 0) {
        const uint32_t a_lo0 = desc_lo(smem_u32(a_ring)), stage_lo = (uint32_t)stage_bytes >> 4;
        uint32_t b_lo[AS_MAX_KB];
#pragma unroll
        for (int kb = 0; kb < AS_MAX_KB; ++kb) b_lo[kb] = desc_lo(smem_u32(sm->ring + kb * B_BYTES));
        const uint32_t bn_lo = desc_lo(smem_u32(sm->ring + nfull * B_BYTES));
        const uint32_t full0 = smem_u32(&sm->a_full[0]), empty0 = smem_u32(&sm->a_empty[0]);
        const uint32_t tfull0 = smem_u32(&sm->tmem_full[0]), tempty0 = smem_u32(&sm->tmem_empty[0]);
        const int last_nk4 = (!narrow && a.k16_last > 0) ? a.k16_last : TK / 16;   // MMAs of the last 64-column block
        const int32_t tiles_cta = t_first < qtiles ? (int32_t)((qtiles - t_first + t_step - 1) / t_step) : 0;
        uint32_t s = 0, ph = 0, bph = 0, acc = 0, aph = 0;
        bool ok = true, pre_acc = false, pre_stage = false;
        for (int b = b_first; ok && b < nb; b += b_step) {
          if (!mbar_wait(&sm->b_full, bph, &sm->abort_flag, a.err, 6, wait_limit)) { ok = false; break; }
          bph ^= 1;
          for (int32_t left = tiles_cta; left > 0; --left) {
            if (!pre_acc && !mbar_wait(&sm->tmem_empty[acc], aph ^ 1, &sm->abort_flag, a.err, 2, wait_limit)) { ok = false; break; }
            if (!pre_stage && !mbar_wait(&sm->a_full[s], ph, &sm->abort_flag, a.err, 3, wait_limit)) { ok = false; break; }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + acc * (uint32_t)TN;
            const uint32_t a_lo = a_lo0 + s * stage_lo;
            const uint32_t ns = s + 1 == (uint32_t)stages ? 0u : s + 1;
            const uint32_t nph = s + 1 == (uint32_t)stages ? ph ^ 1u : ph;
            const uint32_t naph = acc ? aph ^ 1u : aph;   // the other accumulator's use count flips parity every second tile
            const bool more = left > 1;                   // the next tile belongs to this centroid block
            pre_acc = false;
            pre_stage = false;
#pragma unroll
            for (int kb = 0; kb < AS_MAX_KB; ++kb) {
              if (kb < nfull) {
                if (kb == nfull - 1 && more) {
                  pre_stage = mbar_test_wait_a(full0 + ns * 8u, nph);
                  pre_acc = mbar_test_wait_a(tempty0 + (acc ^ 1u) * 8u, naph ^ 1u);
                }
                const int nk4 = kb == nfull - 1 ? last_nk4 : TK / 16;
#pragma unroll
                for (int k4 = 0; k4 < TK / 16; ++k4)
                  if (k4 < nk4)
                    tc_mma(tmem_d, desc_pack(a_lo + (uint32_t)(kb * (A_BYTES >> 4) + k4 * 2), kDescHi),
                           desc_pack(b_lo[kb] + (uint32_t)(k4 * 2), kDescHi), kIdesc, (kb | k4) ? 1u : 0u);
              }
            }
            if (narrow) {
              // a second look for what the first one came too early for
              if (more && !pre_stage) pre_stage = mbar_test_wait_a(full0 + ns * 8u, nph);
              if (more && !pre_acc) pre_acc = mbar_test_wait_a(tempty0 + (acc ^ 1u) * 8u, naph ^ 1u);
              tc_mma(tmem_d, desc_pack(a_lo + (uint32_t)(nfull * (A_BYTES >> 4)), kDescHiNarrow), desc_pack(bn_lo, kDescHiNarrow), kIdesc, 1u);
            }
            tc_commit_a(empty0 + s * 8u);
            tc_commit_a(tfull0 + acc * 8u);
            s = ns;
            ph = nph;
            aph = naph;
            acc ^= 1u;
          }
          if (ok) tc_commit(&sm->b_empty);   // arrives when every MMA issued so far (all readers of this block) has retired
        }
        tc_commit(&sm->drain);
        for (uint32_t it = 0; it < wait_limit; ++it) {
          if (mbar_try_wait(&sm->drain, 0)) break;
          __nanosleep(64);
        }
      }
      __syncwarp();
    } else {
      // One K block per ring stage (long rows, or a stage cap set for measurement): the whole warp runs the loop
      // converged and one elected lane issues; the same look-ahead, per stage.
      int s = 0;
      uint32_t ph = 0, bph = 0;
      int64_t local = 0;
      bool ok = true;
      bool pre_acc = false, pre_stage = false;
      for (int b = b_first; ok && b < nb; b += b_step) {
        if (!__all_sync(0xffffffffu, mbar_wait(&sm->b_full, bph, &sm->abort_flag, a.err, 6, wait_limit))) { ok = false; break; }
        bph ^= 1;
        tc_fence_after();
        for (int64_t t = t_first; ok && t < qtiles; t += t_step, ++local) {
          const int acc = (int)(local & 1);
          const uint32_t aph = (uint32_t)((local >> 1) & 1);
          if (!pre_acc && !__all_sync(0xffffffffu, mbar_wait(&sm->tmem_empty[acc], aph ^ 1, &sm->abort_flag, a.err, 2, wait_limit))) { ok = false; break; }
          pre_acc = false;
          const uint32_t tmem_d = tmem_base + (uint32_t)(acc * TN);
          for (int kb0 = 0; kb0 < a.kblocks; kb0 += skb) {
            if (!pre_stage && !__all_sync(0xffffffffu, mbar_wait(&sm->a_full[s], ph, &sm->abort_flag, a.err, 3, wait_limit))) { ok = false; break; }
            pre_stage = false;
            tc_fence_after();
            // The barriers of the NEXT step are looked at (one test, never a wait) before the last MMAs of this step are
            // issued, while the tensor pipe still has work queued: what is seen complete there is not waited for again,
            // so the next step's MMAs follow without the pipe running dry over two barrier waits.
            const bool tile_ends = kb0 + skb >= a.kblocks;
            const int ns = s + 1 == stages ? 0 : s + 1;
            const uint32_t nph = s + 1 == stages ? ph ^ 1 : ph;
            const bool more = !tile_ends || t + t_step < qtiles;   // the next step belongs to this centroid block
            const int nj = skb == a.kblocks ? nfull : 1;
            for (int j = 0; j < nj; ++j) {
              const int kb = kb0 + j;
              const uint64_t adesc = make_desc(smem_u32(a_ring + s * stage_bytes + j * A_BYTES));
              const uint64_t bdesc = make_desc(smem_u32(sm->ring + kb * B_BYTES));
              const int nk4 = (kb == a.kblocks - 1 && a.k16_last > 0) ? a.k16_last : TK / 16;
              if (j == nj - 1 && more) {
                pre_stage = __all_sync(0xffffffffu, mbar_test_wait(&sm->a_full[ns], nph));
                if (tile_ends)
                  pre_acc = __all_sync(0xffffffffu, mbar_test_wait(&sm->tmem_empty[acc ^ 1], (uint32_t)(((local + 1) >> 1) & 1) ^ 1u));
              }
              if (elect_one()) {
#pragma unroll
                for (int k4 = 0; k4 < TK / 16; ++k4)
                  if (k4 < nk4) tc_mma(tmem_d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), kIdesc, (kb | k4) ? 1u : 0u);
              }
              __syncwarp();
            }
            if (narrow) {
              const uint64_t adesc = make_desc_narrow(smem_u32(a_ring + s * stage_bytes + nfull * A_BYTES));
              const uint64_t bdesc = make_desc_narrow(smem_u32(sm->ring + nfull * B_BYTES));
              // a second look for what the first one came too early for (the other accumulator is handed back about
              // four MMAs after this tile's first)
              if (more && !pre_stage) pre_stage = __all_sync(0xffffffffu, mbar_test_wait(&sm->a_full[ns], nph));
              if (more && tile_ends && !pre_acc)
                pre_acc = __all_sync(0xffffffffu, mbar_test_wait(&sm->tmem_empty[acc ^ 1], (uint32_t)(((local + 1) >> 1) & 1) ^ 1u));
              if (elect_one()) tc_mma(tmem_d, adesc, bdesc, kIdesc, 1u);
              __syncwarp();
            }
            if (elect_one()) tc_commit(&sm->a_empty[s]);
            __syncwarp();
            s = ns;
            ph = nph;
          }
          if (ok && elect_one()) tc_commit(&sm->tmem_full[acc]);
          __syncwarp();
        }
        if (ok && elect_one()) tc_commit(&sm->b_empty);   // arrives when every MMA issued so far (all readers of this block) has retired
        __syncwarp();
      }
      if (lane == 0) {
        tc_commit(&sm->drain);
        for (uint32_t it = 0; it < wait_limit; ++it) {
          if (mbar_try_wait(&sm->drain, 0)) break;
          __nanosleep(64);
        }
      }
      __syncwarp();
    }
  } else {
    // ---------------- epilogue: one data row per thread, a quarter of the block's columns per warp ----------------
    constexpr int PARTS = AS_EW / 4, GROUPS = TN / PARTS / 32;
    const int quarter = warp & 3;
    const int et = quarter * 32 + lane;
    const int ew = warp - 2;
    const int part = ew >> 2;
    const int c0 = part * GROUPS;
    const float alpha = __ldg(a.alpha);
    const float inv_alpha = 1.0f / alpha;
    int64_t local = 0;
    bool ok = true;
    for (int b = b_first; ok && b < nb; b += b_step) {
      const int col_base = b * TN;
      float thr_next = CUDART_INF_F;
      if (MODE == SCAN_THRESHOLD && t_first < qtiles && t_first * TM + et < a.n) thr_next = __ldg(a.thr + t_first * TM + et);
      for (int64_t t = t_first; t < qtiles; t += t_step, ++local) {
        const int acc = (int)(local & 1);
        const uint32_t aph = (uint32_t)((local >> 1) & 1);
        const int64_t q = t * TM + et;
        const bool qok = q < a.n;
        const float thr = thr_next;
        const float bar = as_bar(thr, inv_alpha);
        if (MODE == SCAN_THRESHOLD) {   // the next tile's threshold is in flight while this tile is processed
          const int64_t qn = (t + t_step) * TM + et;
          thr_next = (t + t_step < qtiles && qn < a.n) ? __ldg(a.thr + qn) : CUDART_INF_F;
        }
        bool got = mbar_wait(&sm->tmem_full[acc], aph, &sm->abort_flag, a.err, 4, wait_limit);
        got = __all_sync(0xffffffffu, got);
        if (!got) { ok = false; break; }
        tc_fence_after();
        const uint32_t trow = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TN);
        if (MODE == SCAN_THRESHOLD) {
          // Both 32-column groups of this warp are read at once and the accumulator is handed back BEFORE the values
          // are looked at: the next tile's MMAs never wait for the tests below (with a short contraction the
          // epilogue's own latency, not the MMAs and not the operand fill, sets the pace of this kernel).
          static_assert(GROUPS == 2, "two groups per warp");
          float v0[32], v1[32];
          tc_ld32_issue(trow + (uint32_t)(c0 * 32), v0);
          tc_ld32_issue(trow + (uint32_t)((c0 + 1) * 32), v1);
          tc_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm->tmem_empty[acc]);
          const int left0 = a.k - (col_base + c0 * 32), left1 = left0 - 32;
          // value = alpha * accumulator <= thr with alpha < 0 is accumulator >= bar (bar = thr / alpha, lowered by more
          // than the roundings of either form can differ: the hits are a superset, and every logged hit is evaluated
          // exactly afterwards).  Eight columns at a time: the largest of eight costs four instructions, and only a
          // set of eight that holds a hit is searched for its columns.
          const float m00 = max8<0>(v0), m01 = max8<8>(v0), m02 = max8<16>(v0), m03 = max8<24>(v0);
          const float m10 = max8<0>(v1), m11 = max8<8>(v1), m12 = max8<16>(v1), m13 = max8<24>(v1);
          const bool mine0 = qok && left0 > 0 && max3(m00, m01, fmaxf(m02, m03)) >= bar;
          const bool mine1 = qok && left1 > 0 && max3(m10, m11, fmaxf(m12, m13)) >= bar;
          if (!__any_sync(0xffffffffu, mine0 || mine1)) continue;
          auto log_hits = [&](uint32_t bits, int first_col) {   // one or two hits as a rule
            bits = (first_col + 8 <= a.k) ? bits : (first_col < a.k ? bits & ((1u << (a.k - first_col)) - 1u) : 0u);
            while (bits) {
              const int j = __ffs((int)bits) - 1;
              bits &= bits - 1u;
              const int slot = atomicAdd(&sm->log_n, 1);
              if (slot < a.log_cap) my_log[slot] = make_uint2((uint32_t)q, (uint32_t)(first_col + j));
            }
          };
          const int col0 = col_base + c0 * 32;
          if (mine0) {
            if (m00 >= bar) log_hits(ge_bits8<0>(v0, bar), col0);
            if (m01 >= bar) log_hits(ge_bits8<8>(v0, bar), col0 + 8);
            if (m02 >= bar) log_hits(ge_bits8<16>(v0, bar), col0 + 16);
            if (m03 >= bar) log_hits(ge_bits8<24>(v0, bar), col0 + 24);
          }
          if (mine1) {
            if (m10 >= bar) log_hits(ge_bits8<0>(v1, bar), col0 + 32);
            if (m11 >= bar) log_hits(ge_bits8<8>(v1, bar), col0 + 40);
            if (m12 >= bar) log_hits(ge_bits8<16>(v1, bar), col0 + 48);
            if (m13 >= bar) log_hits(ge_bits8<24>(v1, bar), col0 + 56);
          }
          continue;
        }
        float bv = CUDART_INF_F;   // SCAN_ARGMIN: this thread's best over its columns of the block
        int bj = 0;
#pragma unroll 1
        for (int c = c0; c < c0 + GROUPS; ++c) {
          float v[32];
          tc_ld32(trow + (uint32_t)(c * 32), v);
          const int left = a.k - (col_base + c * 32);   // valid centroids from this group's first column on
          if (left <= 0) continue;
          // alpha < 0: the smallest value of the group is alpha times its largest accumulator - one max per value;
          // the column is looked for only when the group beats the best so far (ever more rarely as groups go by)
          float amax = -CUDART_INF_F;
          if (left >= 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, v[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = j < left ? fmaxf(amax, v[j]) : amax;
          }
          const float gmin = amax * alpha;
          if (gmin < bv) {   // strict '<': an earlier (lower) centroid keeps a tie
            bv = gmin;
            int jj = 31;
#pragma unroll
            for (int j = 31; j >= 0; --j) jj = (j < left && v[j] == amax) ? j : jj;   // the lowest column holding the max
            bj = c * 32 + jj;
          }
        }
        if (qok && bv < CUDART_INF_F)
          atomicMin(a.best + q, (unsigned long long)make_key(bv, (uint32_t)(col_base + bj)));
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->tmem_empty[acc]);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (MODE == SCAN_THRESHOLD && threadIdx.x == 0) {
    const int logged = sm->log_n;
    a.log_count[blockIdx.x] = (int32_t)min((int64_t)logged, a.log_cap);
    if (logged > a.log_cap) atomicCAS(a.err, 0, 9);
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// One warp per logged hit: the exact squared distance of the row to the listed centroid, direct fp32 formula, merged
// into best[row] - smallest (value, centroid), the reference's strict '<' scan (KMeansClustering.swift:283-288).
template <bool VEC>
__global__ void __launch_bounds__(256, 6) assign_log_exact_kernel(const float* __restrict__ x, int dim, const float* __restrict__ cent,
                                        const uint2* __restrict__ log, const int32_t* __restrict__ log_count, int64_t log_cap,
                                        unsigned long long* __restrict__ best) {
  const int cta = blockIdx.y;
  const int cnt = log_count[cta];
  const uint2* mine = log + (int64_t)cta * log_cap;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (VEC) {
    // 16-byte loads (dim a multiple of 4, aligned rows), two hits per step: four independent loads in flight per lane
    const int nv = dim >> 2;
    for (int e = 2 * w; e < cnt; e += 2 * warps) {
      const bool two = e + 1 < cnt;
      const uint2 h0 = mine[e], h1 = two ? mine[e + 1] : h0;
      const float4* x0 = reinterpret_cast<const float4*>(x + (int64_t)h0.x * dim);
      const float4* c0 = reinterpret_cast<const float4*>(cent + (int64_t)h0.y * dim);
      const float4* x1 = reinterpret_cast<const float4*>(x + (int64_t)h1.x * dim);
      const float4* c1 = reinterpret_cast<const float4*>(cent + (int64_t)h1.y * dim);
      float s0 = 0.f, s1 = 0.f;
      for (int i = lane; i < nv; i += 32) {
        const float4 a0 = __ldg(x0 + i), b0 = __ldg(c0 + i), a1 = __ldg(x1 + i), b1 = __ldg(c1 + i);
        float d;
        d = a0.x - b0.x; s0 = fmaf(d, d, s0);
        d = a0.y - b0.y; s0 = fmaf(d, d, s0);
        d = a0.z - b0.z; s0 = fmaf(d, d, s0);
        d = a0.w - b0.w; s0 = fmaf(d, d, s0);
        d = a1.x - b1.x; s1 = fmaf(d, d, s1);
        d = a1.y - b1.y; s1 = fmaf(d, d, s1);
        d = a1.z - b1.z; s1 = fmaf(d, d, s1);
        d = a1.w - b1.w; s1 = fmaf(d, d, s1);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      }
      if (lane == 0) {
        atomicMin(best + h0.x, (unsigned long long)make_key(s0, h0.y));
        if (two) atomicMin(best + h1.x, (unsigned long long)make_key(s1, h1.y));
      }
    }
    return;
  }
  for (int e = w; e < cnt; e += warps) {
    const uint2 h = mine[e];
    const float* xr = x + (int64_t)h.x * dim;
    const float* cr = cent + (int64_t)h.y * dim;
    float s = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float d = __ldg(xr + i) - __ldg(cr + i);
      s = fmaf(d, d, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) atomicMin(best + h.x, (unsigned long long)make_key(s, h.y));
  }
}

// best[row] -> assignment and rooted distance; a row without any logged hit is handed to the exact scan
// (`err` given and raised: the scan's log is incomplete - nothing is written, so that the previous assignment and its
// distances survive for the repeat)
__global__ void assign_log_decode_kernel(const unsigned long long* __restrict__ best, int64_t n, int32_t* __restrict__ assign,
                                         float* __restrict__ dist, int32_t* __restrict__ bad_rows, int32_t* bad_count,
                                         const int32_t* __restrict__ err) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  if (err != nullptr && *err != 0) return;
  const unsigned long long b = best[r];
  if (b == ~0ull) {
    bad_rows[atomicAdd(bad_count, 1)] = (int32_t)r;
    return;
  }
  assign[r] = (int32_t)(uint32_t)b;
  if (dist) dist[r] = sqrtf(ordered_to_float((uint32_t)(b >> 32)));
}

// ---- operand preparation --------------------------------------------------------------------
// Statistics accumulated with atomics on order-preserving integer images of non-negative floats.
struct PrepStats {
  unsigned absmax;      // max |x_i|
  unsigned max_norm16;  // max over rows of |x'| (operand units)
  unsigned max_err16;   // max over rows of |s*x - x'|
  unsigned max_norm;    // max |x|
  unsigned min_norm_nz; // min nonzero |x| (initialised to +inf)
};

__global__ void absmax_kernel(const float* __restrict__ x, int64_t total, unsigned* out) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(__ldg(x + i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));  // non-negative floats order as uints
}

// scale = 2^e with 2^13 < absmax * scale <= 2^14 (1 when absmax is 0 or not finite); cosine: 2^14
// fold != 0 (queries against folded rows, see FoldArgs): the scale is also kept where the folded constant
// s 2^-exp is a normal fp16 number.
__global__ void choose_scale_kernel(const unsigned* absmax, int cosine, float* scale, int fold = 0, int fold_exp = 0) {
  float s = 16384.f;
  if (!cosine) {
    const float m = __uint_as_float(*absmax);
    s = 1.f;
    if (m > 0.f && m < CUDART_INF_F) {
      int e;
      frexpf(m, &e);               // m = f * 2^e, f in [0.5, 1)
      s = ldexpf(1.f, 14 - e);
    }
  }
  if (fold) s = fmaxf(fminf(s, ldexpf(1.f, fold_exp + 13)), ldexpf(1.f, fold_exp - 14));   // 4u <= 2^15, 2u normal
  *scale = s;
}

// One warp per row: fp32 row -> fp16 operand row x' = fp16(s * x) (cosine: s * x/|x|), padded with
// zeros to dim16, and the measured quantities the error bound needs.
//   aux[row]   = |x|^2 (euclidean), unused otherwise
//   nrm16[row] = |x'|, err16[row] = |s*x^ - x'|   (optional per-row outputs, used for queries)
// Euclidean operands can carry the per-row term of the value inside the contraction.  Sixteen columns - one K16
// step of the MMA, placed right behind the data columns (fold_col0) - hold, on the row side, R = -(s_x |x|^2 / 2) 2^exp
// split into three fp16 pieces p0 + p1 + p2 = R / 16 (p0 in columns 0-3, p1 in 4-7, p2 in 8-15), and on the query
// side the constants 4u (columns 0-7) and 2u (columns 8-15), u = s_q 2^-exp a power of two: the sixteen products add
// up to 16 u (p0 + p1 + p2) = -s_q s_x |x|^2 / 2, so the accumulator is s_q s_x (q.x - |x|^2 / 2) and the value
// alpha * accumulator needs no per-row term in the epilogue.  Columns behind the sixteen are zero and the MMA issuer
// skips K16 steps that hold nothing but padding (kvalid), so the term costs one K16 step, not a K block.
constexpr int kFoldCols = 16;
__host__ __device__ inline int fold_col0(int dim) { return (dim + 15) / 16 * 16; }
// K16 steps of the last 64-column K block that hold operand columns, for `kvalid` columns in a width of dim16
inline int k16_last_of(int kvalid, int dim16) {
  const int steps = (kvalid + 15) / 16, before = 4 * (dim16 / 64 - 1);
  return std::max(1, std::min(4, steps - before));
}
struct FoldArgs {
  int side;   // 0: none, 1: rows (pieces of the term), 2: queries (the constants)
  int col0;   // first of the kFoldCols columns (fold_col0(dim))
  int exp;
  const int* exp_dev = nullptr;   // when given, the exponent is read from device memory instead
};

template <int METRIC>
__global__ void prep_rows_kernel(const float* __restrict__ x, int64_t n, int dim, int dim16, const float* scale_p,
                                 __half* __restrict__ out, float* __restrict__ aux, float* __restrict__ nrm16,
                                 float* __restrict__ err16, float* __restrict__ nrm, PrepStats* stats, FoldArgs fold) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float s = *scale_p;
  const float* p = x + row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = __ldg(p + i);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float norm = sqrtf(ss);
  const float inv = (METRIC == VSK_METRIC_COSINE) ? (norm > 0.f ? 1.0f / norm : 0.f) : 1.0f;
  float n2 = 0.f, e2 = 0.f;
  for (int i = lane; i < dim16; i += 32) {
    float t = 0.f;
    if (i < dim) t = (METRIC == VSK_METRIC_COSINE) ? (__ldg(p + i) * inv) * s : __ldg(p + i) * s;
    const __half h = __float2half_rn(t);
    if (fold.side == 0 || i < fold.col0 || i >= fold.col0 + kFoldCols) out[row * dim16 + i] = h;
    const float back = __half2float(h);
    n2 = fmaf(back, back, n2);
    const float e = t - back;
    e2 = fmaf(e, e, e2);
  }
  const int fold_exp = fold.exp_dev ? *fold.exp_dev : fold.exp;
  if (fold.side == 1) {
    // pieces of R = s_x (|x|^2 / 2) 2^exp: p0 = fp16(R/16), then the same of what is left, twice (the remainders are
    // exact in fp32); what is left after three pieces is below 2^-33 R
    const float R = ldexpf(0.5f * ss * s, fold_exp);
    const __half p0 = __float2half_rn(R * 0.0625f);
    const float r1 = R - 16.0f * __half2float(p0);
    const __half p1 = __float2half_rn(r1 * 0.0625f);
    const float r2 = r1 - 16.0f * __half2float(p1);
    const __half p2 = __float2half_rn(r2 * 0.0625f);
    if (lane < kFoldCols) {
      const __half p = lane < 4 ? p0 : (lane < 8 ? p1 : p2);
      out[row * dim16 + fold.col0 + lane] = __hneg(p);
    }
  } else if (fold.side == 2) {
    // 4u against the four copies of p0 and of p1, 2u against the eight copies of p2
    if (lane < kFoldCols) out[row * dim16 + fold.col0 + lane] = __float2half_rn(ldexpf(s, (lane < 8 ? 2 : 1) - fold_exp));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    n2 += __shfl_xor_sync(0xffffffffu, n2, o);
    e2 += __shfl_xor_sync(0xffffffffu, e2, o);
  }
  if (lane == 0) {
    // round the measured norms up a little: they are used as upper bounds
    const float up = 1.0f + 1e-5f;
    const float a16 = sqrtf(n2) * up, r16 = sqrtf(e2) * up;
    if (aux && METRIC == VSK_METRIC_EUCLIDEAN) aux[row] = ss;
    if (nrm16) nrm16[row] = a16;
    if (err16) err16[row] = r16;
    if (nrm) nrm[row] = norm;
    if (stats) {
      atomicMax(&stats->max_norm16, __float_as_uint(a16));
      atomicMax(&stats->max_err16, __float_as_uint(r16));
      atomicMax(&stats->max_norm, __float_as_uint(norm));
      if (norm > 0.f) atomicMin(&stats->min_norm_nz, __float_as_uint(norm));
    }
  }
}

struct BoundConsts {
  float scale_x;       // s_x
  float max_norm16;    // X' = max |x'|
  float max_err16;     // E' = max |s_x x - x'|
  float max_norm;      // max |x|
  float min_norm_nz;   // min nonzero |x|
  int dim16;
  float fold_bmax;     // folded rows: max |x|^2 / 2 (0 otherwise)
};

// eps[q]: |coarse - exact| <= eps for every row, in the units of the stored coarse value.
//   contraction error (operand units) <= |q'| E' + |e_q| X' + |e_q| E'      (Cauchy-Schwarz on the residuals)
//                                       + dim16 * 2^-22 * |q'| X'            (fp32 accumulation in the tensor core)
//   divided by s_q s_x; doubled for euclidean (value = |x|^2 - 2 q.x) plus the fp32 rounding of |x|^2;
//   cosine adds the effect of the reference's +1e-8 in the denominator and of normalising in fp32.
// Also writes alpha = coefficient / (s_q s_x).
template <int METRIC>
__global__ void bound_kernel(const float* __restrict__ qn16, const float* __restrict__ qe16,
                             const float* __restrict__ qnorm, int64_t nq, const float* scale_q, BoundConsts c,
                             float* __restrict__ eps, float* alpha) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float inv = 1.0f / ((*scale_q) * c.scale_x);
  if (q == 0) *alpha = (METRIC == VSK_METRIC_EUCLIDEAN ? -2.0f : -1.0f) * inv;
  if (q >= nq) return;
  const float a = qn16[q], e = qe16[q];
  float dot_err = (a * c.max_err16 + e * c.max_norm16 + e * c.max_err16) + (float)c.dim16 * 2.3841858e-7f * a * c.max_norm16;
  dot_err *= inv;
  // folded per-row term (true units): its products pass through the same fp32 accumulation, and three fp16 pieces
  // leave less than 2^-30 of it unrepresented
  dot_err += ((float)c.dim16 * 2.3841858e-7f + 9.3132257e-10f) * c.fold_bmax;
  float r;
  if (METRIC == VSK_METRIC_EUCLIDEAN) {
    // + fp32 rounding of the stored |x|^2 (a sum of dim squares) and of the final multiply-add
    const float qn = qnorm[q];
    r = 2.0f * dot_err + 4.0f * 5.9604645e-8f * (float)c.dim16 * c.max_norm * c.max_norm +
        2.0f * 5.9604645e-8f * (c.max_norm * c.max_norm + 2.0f * qn * c.max_norm);
  } else if (METRIC == VSK_METRIC_COSINE) {
    const float qn = qnorm[q];
    const float den = qn * c.min_norm_nz;
    r = dot_err + 1e-8f / (den + 1e-8f) + 4.0f * 5.9604645e-8f;
    if (!(den > 0.f)) r = dot_err + 4.0f * 5.9604645e-8f;  // zero query (or no nonzero row): every value is exactly 0
  } else {
    r = dot_err;
  }
  eps[q] = r * 1.0001f + 1e-30f;
}

// ---- int8-coded rows -----------------------------------------------------------------------
// One warp per row of int8 codes: the fp16 operand row is the code itself (exact: |code| <= 128), so the
// operand residual of the rows is zero.  aux = |x^|^2 of the dequantised row x^ = (code - offset)/scale
// (euclidean); stats: max |code row|, max |x^|.
__global__ void prep_codes_kernel(const int8_t* __restrict__ codes, int64_t n, int dim, int dim16,
                                  const float* __restrict__ scale, const float* __restrict__ offset,
                                  __half* __restrict__ out, float* __restrict__ aux, PrepStats* stats) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const int8_t* p = codes + row * dim;
  float c2 = 0.f, x2 = 0.f;
  for (int i = lane; i < dim16; i += 32) {
    float c = 0.f;
    if (i < dim) {
      c = (float)p[i];
      const float xh = __fdiv_rn(__fsub_rn(c, __ldg(offset + i)), __ldg(scale + i));
      x2 = fmaf(xh, xh, x2);
    }
    out[row * dim16 + i] = __float2half_rn(c);
    c2 = fmaf(c, c, c2);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c2 += __shfl_xor_sync(0xffffffffu, c2, o);
    x2 += __shfl_xor_sync(0xffffffffu, x2, o);
  }
  if (lane == 0) {
    const float up = 1.0f + 1e-5f;
    aux[row] = x2;
    atomicMax(&stats->max_norm16, __float_as_uint(sqrtf(c2) * up));
    atomicMax(&stats->max_norm, __float_as_uint(sqrtf(x2) * up));
  }
}

// q~ = q / scale per dimension: sum_i q_i x^_i = sum_i q~_i code_i - sum_i q_i offset_i / scale_i, and the
// second term does not depend on the row.
__global__ void scale_queries_kernel(const float* __restrict__ q, int64_t total, int dim,
                                     const float* __restrict__ scale, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) out[i] = __fdiv_rn(q[i], __ldg(scale + (int)(i % dim)));
}

// eps for int8-coded rows (operand residual of the rows is zero; the query operand is fp16(s_q q~)):
//   contraction   |e_q| C + dim16 2^-22 |q'| C, divided by s_q          (C = max |code row|)
//   formula       2^-22 (|q| max|x^| + |q~| C): fp32 rounding of x^ = (code - offset)/scale and of q~
// doubled for euclidean (value = |x^|^2 - 2 q.x^) plus the rounding of |x^|^2 and of the final multiply-add.
template <int METRIC>
__global__ void bound_i8_kernel(const float* __restrict__ qn16, const float* __restrict__ qe16,
                                const float* __restrict__ qt_norm, const float* __restrict__ q_norm, int64_t nq,
                                const float* scale_q, BoundConsts c, float* __restrict__ eps, float* alpha) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float inv = 1.0f / (*scale_q);
  if (q == 0) *alpha = (METRIC == VSK_METRIC_EUCLIDEAN ? -2.0f : -1.0f) * inv;
  if (q >= nq) return;
  const float a = qn16[q], e = qe16[q];
  float dot_err = (e * c.max_norm16 + (float)c.dim16 * 2.3841858e-7f * a * c.max_norm16) * inv;
  dot_err += 2.3841858e-7f * (q_norm[q] * c.max_norm + qt_norm[q] * c.max_norm16);
  float r = dot_err;
  if (METRIC == VSK_METRIC_EUCLIDEAN)
    r = 2.0f * dot_err + 4.0f * 5.9604645e-8f * (float)c.dim16 * c.max_norm * c.max_norm +
        2.0f * 5.9604645e-8f * (c.max_norm * c.max_norm + 2.0f * q_norm[q] * c.max_norm);
  eps[q] = r * 1.0001f + 1e-30f;
}

// Exact re-scoring against dequantised rows (the int8 scan's definition: the metric between the fp32 query
// and x^ = (code - offset)/scale, ScalarQuantizer.swift:576-578).
template <int METRIC>
__global__ void __launch_bounds__(256) rerank_i8_kernel(const float* __restrict__ q, const int8_t* __restrict__ codes,
                                                        int dim, const float* __restrict__ scale,
                                                        const float* __restrict__ offset, CandLists cand,
                                                        unsigned long long* total) {
  extern __shared__ float qs[];
  const int64_t qi = blockIdx.x;
  const int cnt = min(cand.count[qi], kCandCap);
  uint64_t* keys = cand.keys + qi * kCandCap;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) qs[i] = q[qi * dim + i];
  if (threadIdx.x == 0) atomicAdd(total, (unsigned long long)cnt);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int c = warp; c < cnt; c += nwarps) {
    const uint32_t id = (uint32_t)keys[c];
    const int8_t* xr = codes + (int64_t)id * dim;
    float s = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float xv = __fdiv_rn(__fsub_rn((float)xr[i], __ldg(offset + i)), __ldg(scale + i));
      const float qv = qs[i];
      if (METRIC == VSK_METRIC_EUCLIDEAN) {
        const float d = qv - xv;
        s = fmaf(d, d, s);
      } else {
        s = fmaf(qv, xv, s);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) keys[c] = make_key(METRIC == VSK_METRIC_EUCLIDEAN ? s : -s, id);
  }
}

// ---- exact rerank -------------------------------------------------------------------------
// One CTA per query: replaces every kept candidate's coarse value with the reference's direct fp32 value:
//   euclidean sum (q-x)^2 (rooted at output), cosine 1 - q.x/(|q||x| + 1e-8), dotProduct -(q.x).
template <int METRIC>
__global__ void __launch_bounds__(256) rerank_kernel(const float* __restrict__ q, const float* __restrict__ x, int dim,
                                                     const float* __restrict__ qnorm, const float* __restrict__ xnorm,
                                                     CandLists cand, unsigned long long* total) {
  extern __shared__ float qs[];
  const int64_t qi = blockIdx.x;
  const int cnt = min(cand.count[qi], kCandCap);
  uint64_t* keys = cand.keys + qi * kCandCap;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) qs[i] = q[qi * dim + i];
  if (threadIdx.x == 0) atomicAdd(total, (unsigned long long)cnt);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const float qn = (METRIC == VSK_METRIC_COSINE) ? qnorm[qi] : 0.f;
  // four candidate rows per warp step: their key loads and row loads are independent chains, which is what keeps
  // enough bytes in flight when a row is only a few hundred bytes
  constexpr int RR = 4;
  for (int c0 = warp * RR; c0 < cnt; c0 += nwarps * RR) {
    uint32_t id[RR];
    const float* xr[RR];
    float s[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      id[r] = c0 + r < cnt ? (uint32_t)keys[c0 + r] : 0u;
      xr[r] = x + (int64_t)id[r] * dim;
      s[r] = 0.f;
    }
    for (int i = lane; i < dim; i += 32) {
      const float qv = qs[i];
#pragma unroll
      for (int r = 0; r < RR; ++r) {
        const float xv = __ldg(xr[r] + i);
        if (METRIC == VSK_METRIC_EUCLIDEAN) {
          const float d = qv - xv;
          s[r] = fmaf(d, d, s[r]);
        } else {
          s[r] = fmaf(qv, xv, s[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RR; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s[r] += __shfl_xor_sync(0xffffffffu, s[r], o);
      if (lane == 0 && c0 + r < cnt) {
        float v;
        if (METRIC == VSK_METRIC_COSINE) v = 1.0f - s[r] / (qn * xnorm[id[r]] + 1e-8f);
        else if (METRIC == VSK_METRIC_DOT_PRODUCT) v = -s[r];
        else v = s[r];
        keys[c0 + r] = make_key(v, id[r]);
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// fp16 matrix [rows][dim16] row-major; box = 64 columns x box_rows, 128-byte swizzle, zero fill
int32_t make_map(Ctx* ctx, const __half* base, int64_t rows, int32_t dim16, int box_rows, CUtensorMap* map) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)dim16, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)dim16 * 2};
  cuuint32_t box[2] = {(cuuint32_t)TK, (cuuint32_t)box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return VSK_OK;
}

// The same matrix seen through a box of 16 columns x box_rows with the 32-byte swizzle: one K16 step of a tile.
int32_t make_map_narrow(Ctx* ctx, const __half* base, int64_t rows, int32_t dim16, int box_rows, CUtensorMap* map) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)dim16, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)dim16 * 2};
  cuuint32_t box[2] = {16u, (cuuint32_t)box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(base), gdim, gstride, box, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, VSK_ERR_EXECUTION_FAILED, "cuTensorMapEncodeTiled (16-column box) failed with %d", (int)r);
  return VSK_OK;
}

template <int METRIC>
void launch_prep(Ctx* ctx, const float* x, int64_t n, int dim, int dim16, const float* scale, __half* out, float* aux,
                 float* nrm16, float* err16, float* nrm, PrepStats* stats, FoldArgs fold = FoldArgs{0, 0, 0}) {
  prep_rows_kernel<METRIC><<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(x, n, dim, dim16, scale, out, aux, nrm16,
                                                                               err16, nrm, stats, fold);
  ctx->stats.kernel_launches++;
}

// max over rows of |x|^2, summed as prep_rows_kernel sums it (one warp per row)
__global__ void max_sq_kernel(const float* __restrict__ x, int64_t n, int dim, unsigned* out) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  const float* p = x + row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = __ldg(p + i);
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) atomicMax(out, __float_as_uint(ss));
}

// fp16 operand copy of the index rows + the constants of the error bound (once per index state)
int32_t tensor_prepare(Index* ix) {
  Ctx* ctx = ix->ctx;
  if (ix->n16 == ix->n && ix->rows16) return VSK_OK;
  dev_free(ix->rows16);
  dev_free(ix->row_aux);
  ix->rows16 = nullptr;
  ix->row_aux = nullptr;
  ix->dim16 = (int32_t)(ceil_div(ix->dim, TK) * TK);
  // Folding the per-row term into the operands (FoldArgs) pays where the epilogue, not the MMAs, sets the pace
  // (up to four K blocks), and is free where the padding already has room for it.
  ix->fold16 = ctx->tuning.fold_row_term != 0 && ix->kind != INDEX_FLAT_I8 && ix->metric == VSK_METRIC_EUCLIDEAN &&
               (ix->dim16 / TK <= 4 || ix->dim16 - fold_col0(ix->dim) >= kFoldCols);
  if (ix->fold16 && ix->dim16 - fold_col0(ix->dim) < kFoldCols) ix->dim16 += TK;
  VSK_TRY(dev_alloc(ctx, (void**)&ix->rows16, (size_t)ix->n * ix->dim16 * sizeof(__half)));
  VSK_TRY(dev_alloc(ctx, (void**)&ix->row_aux, (size_t)ix->n * sizeof(float)));
  void* p;
  VSK_TRY(scratch(ctx, SLOT_TC_A, sizeof(PrepStats) + 32, &p));
  PrepStats* st = (PrepStats*)p;
  float* scale = (float*)((char*)p + sizeof(PrepStats));
  unsigned* max_sq = (unsigned*)((char*)p + sizeof(PrepStats) + 16);
  PrepStats init{0u, 0u, 0u, 0u, 0x7f800000u};
  VSK_CUDA(ctx, cudaMemcpyAsync(st, &init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
  const bool cosine = ix->metric == VSK_METRIC_COSINE;
  if (ix->kind == INDEX_FLAT_I8) {
    const float one = 1.0f;
    VSK_CUDA(ctx, cudaMemcpyAsync(scale, &one, 4, cudaMemcpyHostToDevice, ctx->stream));
    prep_codes_kernel<<<(unsigned)ceil_div(ix->n, 8), 256, 0, ctx->stream>>>(ix->codes, ix->n, ix->dim, ix->dim16, ix->sq_scale,
                                                                            ix->sq_offset, ix->rows16, ix->row_aux, st);
    ctx->stats.kernel_launches++;
  } else {
  if (!cosine) {
    absmax_kernel<<<1184, 256, 0, ctx->stream>>>(ix->rows, ix->n * (int64_t)ix->dim, &st->absmax);
    ctx->stats.kernel_launches++;
  }
  choose_scale_kernel<<<1, 1, 0, ctx->stream>>>(&st->absmax, cosine ? 1 : 0, scale);
  ctx->stats.kernel_launches++;
  FoldArgs fold{0, 0, 0};
  ix->fold_exp = 0;
  ix->fold_bmax = 0.f;
  if (ix->fold16) {
    // the exponent that brings the largest piece, s_x (|x|^2 / 2) 2^exp / 16, just below 2^14
    VSK_CUDA(ctx, cudaMemsetAsync(max_sq, 0, 4, ctx->stream));
    max_sq_kernel<<<(unsigned)ceil_div(ix->n, 8), 256, 0, ctx->stream>>>(ix->rows, ix->n, ix->dim, max_sq);
    ctx->stats.kernel_launches++;
    float hmax = 0.f, hscale = 1.f;
    VSK_CUDA(ctx, cudaMemcpyAsync(&hmax, max_sq, 4, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaMemcpyAsync(&hscale, scale, 4, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const double top = 0.5 * (double)hmax * (double)hscale / 16.0;
    int e = 0;
    if (top > 0.0 && std::isfinite(top)) e = 14 - (int)std::ceil(std::log2(top));
    ix->fold_exp = std::max(-100, std::min(100, e));
    ix->fold_bmax = 0.5f * hmax;
    if (!std::isfinite(top)) ix->fold16 = false;   // the plain form copes with what overflows here no better, but is the known path
    fold = FoldArgs{ix->fold16 ? 1 : 0, fold_col0(ix->dim), ix->fold_exp};
  }
  switch (ix->metric) {
    case VSK_METRIC_EUCLIDEAN:
      launch_prep<VSK_METRIC_EUCLIDEAN>(ctx, ix->rows, ix->n, ix->dim, ix->dim16, scale, ix->rows16, ix->row_aux, nullptr, nullptr, nullptr, st, fold);
      break;
    case VSK_METRIC_COSINE:
      launch_prep<VSK_METRIC_COSINE>(ctx, ix->rows, ix->n, ix->dim, ix->dim16, scale, ix->rows16, ix->row_aux, nullptr, nullptr, nullptr, st);
      break;
    default:
      launch_prep<VSK_METRIC_DOT_PRODUCT>(ctx, ix->rows, ix->n, ix->dim, ix->dim16, scale, ix->rows16, ix->row_aux, nullptr, nullptr, nullptr, st);
      break;
  }
  }
  VSK_CUDA(ctx, cudaGetLastError());
  PrepStats h;
  float hs;
  VSK_CUDA(ctx, cudaMemcpyAsync(&h, st, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(&hs, scale, 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  auto f = [](unsigned u) { float v; memcpy(&v, &u, 4); return v; };
  ix->scale16 = hs;
  ix->max_xnorm16 = f(h.max_norm16);
  ix->max_xerr16 = f(h.max_err16);
  ix->max_xnorm = f(h.max_norm);
  ix->min_xnorm_nz = h.min_norm_nz == 0x7f800000u ? 0.f : f(h.min_norm_nz);
  ix->n16 = ix->n;
  return VSK_OK;
}

// Launches the scan over tiles (persistent: one CTA per SM, or per tile when there are fewer tiles).
template <int MODE, int EW>
int32_t launch_tc_ew(Ctx* ctx, const CUtensorMap& mq, const CUtensorMap& mx, const TcArgs& a, bool has_beta) {
  static bool attr_done[2][2] = {};
  const bool has_mask = MODE != SCAN_ARGMIN && a.row_masks != nullptr && a.q_masks != nullptr;
  void (*kern)(CUtensorMap, CUtensorMap, TcArgs);
  if constexpr (MODE == SCAN_ARGMIN) {
    kern = has_beta ? tc_scan_kernel<MODE, true, false, EW> : tc_scan_kernel<MODE, false, false, EW>;
  } else {
    kern = has_mask ? (has_beta ? tc_scan_kernel<MODE, true, true, EW> : tc_scan_kernel<MODE, false, true, EW>)
                    : (has_beta ? tc_scan_kernel<MODE, true, false, EW> : tc_scan_kernel<MODE, false, false, EW>);
  }
  constexpr size_t smem = tc_smem_bytes<EW>();
  if (!attr_done[has_beta][has_mask]) {
    VSK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[has_beta][has_mask] = true;
  }
  const int64_t tiles = a.tiles ? a.num_tiles : ceil_div(a.nq, TM) * ceil_div(a.row_end - a.row_begin, TN);
  if (tiles <= 0) return VSK_OK;
  const int sms = ctx->prop.multiProcessorCount;
  const unsigned grid = (unsigned)std::min<int64_t>(tiles, sms);
  TcArgs la = a;
  la.wait_limit = ctx->tuning.wait_limit_log2 > 0 ? (1u << std::min(ctx->tuning.wait_limit_log2, 30)) : 0u;
  la.stall_kblock = -1;
  la.stage_kblocks = ctx->tuning.stage_kblocks == 2 ? 2 : 1;
  if (ctx->tuning.test_stall_scan > 0) {   // testing only, one shot
    la.stall_kblock = 0;
    ctx->tuning.test_stall_scan = 0;
  }
  prof_begin(ctx);
  kern<<<grid, Epi<EW>::THREADS, smem, ctx->stream>>>(mq, mx, la);
  prof_end(ctx);
  tl_mark(ctx, MODE == SCAN_DENSE ? "scan_dense" : (MODE == SCAN_ARGMIN ? "scan_argmin" : "scan"));
  ctx->stats.kernel_launches++;
  ctx->stats.tensor_tiles += tiles;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

// Epilogue warps by contraction length (see Epi): 16 up to four K blocks (d <= 256), 8 beyond.
inline int tc_epilogue_warps(int kblocks) { return kblocks <= 4 ? 16 : 8; }

template <int MODE>
int32_t launch_tc(Ctx* ctx, const CUtensorMap& mq, const CUtensorMap& mx, const TcArgs& a, bool has_beta) {
  if (tc_epilogue_warps(a.kblocks) == 16) return launch_tc_ew<MODE, 16>(ctx, mq, mx, a, has_beta);
  return launch_tc_ew<MODE, 8>(ctx, mq, mx, a, has_beta);
}

// ---- k-means assignment on the tensor cores ----------------------------------------------------
// Data rows are the streamed operand (the "query" side of the tile), centroids the small one.
//   pass 1  coarse arg-min: best[row] = smallest coarse (|c|^2 - 2 x.c, centroid) key
//   pass 2  every centroid whose coarse value is within 2 eps(row) of that minimum is appended to the
//           row's short list (the true nearest centroid is among them: its exact value is <= the exact
//           value of the coarse winner <= coarse minimum + eps, so its coarse value <= minimum + 2 eps)
//   exact   the listed centroids are compared with the direct fp32 formula sum (x-c)^2; the smallest
//           (value, index) wins, as the reference's strict '<' scan does (KMeansClustering.swift:283-288)
// A row whose list overflows (more near-ties than a sub-list holds) is re-done by the fp32 tile.
constexpr int kAssignLogPerRow = 6;
constexpr int kAssignCap = 32;   // split into one sub-list per column part of a tile (2 parts of 16, or 4 of 8)

// eps per data row against the current centroids; stats of the centroid operand are read on the device.
__global__ void assign_bound_kernel(const float* __restrict__ xn16, const float* __restrict__ xe16,
                                    const float* __restrict__ xnorm, int64_t n, const float* scale_x,
                                    const float* scale_c, const PrepStats* cs, int dim16, float* __restrict__ eps,
                                    float* alpha, int folded) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float inv = 1.0f / ((*scale_x) * (*scale_c));
  if (r == 0) *alpha = -2.0f * inv;
  if (r >= n) return;
  const float C16 = __uint_as_float(cs->max_norm16), E16 = __uint_as_float(cs->max_err16);
  const float Cn = __uint_as_float(cs->max_norm);
  const float a = xn16[r], e = xe16[r];
  float dot_err = ((a * E16 + e * C16 + e * E16) + (float)dim16 * 2.3841858e-7f * a * C16) * inv;
  // |c|^2 / 2 carried inside the contraction: its products pass through the same fp32 accumulation, and three fp16
  // pieces leave less than 2^-30 of it unrepresented
  if (folded) dot_err += ((float)dim16 * 2.3841858e-7f + 9.3132257e-10f) * 0.5f * Cn * Cn;
  const float v = 2.0f * dot_err + 4.0f * 5.9604645e-8f * (float)dim16 * Cn * Cn +
                  2.0f * 5.9604645e-8f * (Cn * Cn + 2.0f * xnorm[r] * Cn);
  eps[r] = v * 1.0001f + 1e-30f;
}

__global__ void assign_threshold_kernel(const unsigned long long* __restrict__ best, const float* __restrict__ eps,
                                        int64_t n, float* __restrict__ thr, int32_t* __restrict__ count) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  thr[r] = ordered_to_float((uint32_t)(best[r] >> 32)) + 2.0f * eps[r];
  count[r] = 0;
}

// Thresholds of the next scan from the previous assignment (Lloyd iterations after the first).  With u the exact value
// |c_p|^2 - 2 x.c_p = |x - c_p|^2 - |x|^2 of the centroid the row was assigned to last time, the nearest centroid c* has
// exact value <= u, hence coarse value <= u + eps; the threshold is u + 2 eps (the second eps covers the fp32 rounding
// of u itself).  Two ways to u, chosen per row:
//   exact   one read of the row: sum (x - c_p)^2 and sum x^2 in fp32 (a warp per row, four rows in flight);
//   bound   no read at all, when the centroid has moved by no more than `ratio` of the row's distance to it: the
//           triangle inequality, |x - c_new| <= |x - c_old| + |c_new - c_old|, with the distance the last iteration
//           left in `dist_old`, the shifts in `shift` and the row norms measured when the operand was made.  The bound
//           is looser than the exact value by at most (2 ratio + ratio^2) of the squared distance, which lists a few
//           more centroids for the exact decision and costs nothing in correctness.
// A lane takes one of 32 consecutive rows; the rows that need the exact form are then done by the whole warp.
template <bool VEC>
__global__ void __launch_bounds__(256) assign_prev_threshold_kernel(
    const float* __restrict__ x, int64_t n, int dim, const float* __restrict__ cent, const int32_t* __restrict__ prev,
    const float* __restrict__ eps, float* __restrict__ thr, int32_t* __restrict__ count, const float* __restrict__ dist_old,
    const float* __restrict__ shift, const float* __restrict__ xnorm, float ratio) {
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 32;
  if (row0 >= n) return;
  const int64_t mine = row0 + lane;
  const bool have = mine < n;
  bool need = have;
  if (have && dist_old != nullptr) {
    const float d = dist_old[mine], sft = shift[prev[mine]];
    if (d > 0.f && d < CUDART_INF_F && sft <= ratio * d) {
      const float xn = xnorm[mine], x2 = xn * xn;
      const float ub = (d + sft) * (1.0f + 1e-5f);
      const float ub2 = ub * ub;
      thr[mine] = (ub2 - x2) + 2.0f * eps[mine] + 1e-5f * (ub2 + x2);
      count[mine] = 0;
      need = false;
    }
  }
  unsigned todo = __ballot_sync(0xffffffffu, need);
  while (todo) {
    // up to four rows per step, each read by the whole warp
    int64_t rr[4];
    int nr = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      rr[r] = row0;
      if (todo) {
        const int l = __ffs((int)todo) - 1;
        todo &= todo - 1u;
        rr[r] = row0 + l;
        nr = r + 1;
      }
    }
    float d2[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
    if (VEC) {
      const int nv = dim >> 2;
      const float4* xr[4];
      const float4* cr[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        xr[r] = reinterpret_cast<const float4*>(x + rr[r] * dim);
        cr[r] = reinterpret_cast<const float4*>(cent + (int64_t)prev[rr[r]] * dim);
      }
      for (int i = lane; i < nv; i += 32) {
        float4 a[4], b[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) { a[r] = __ldg(xr[r] + i); b[r] = __ldg(cr[r] + i); }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float d;
          d = a[r].x - b[r].x; d2[r] = fmaf(d, d, d2[r]); x2[r] = fmaf(a[r].x, a[r].x, x2[r]);
          d = a[r].y - b[r].y; d2[r] = fmaf(d, d, d2[r]); x2[r] = fmaf(a[r].y, a[r].y, x2[r]);
          d = a[r].z - b[r].z; d2[r] = fmaf(d, d, d2[r]); x2[r] = fmaf(a[r].z, a[r].z, x2[r]);
          d = a[r].w - b[r].w; d2[r] = fmaf(d, d, d2[r]); x2[r] = fmaf(a[r].w, a[r].w, x2[r]);
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float* xr = x + rr[r] * dim;
        const float* cr = cent + (int64_t)prev[rr[r]] * dim;
        for (int i = lane; i < dim; i += 32) {
          const float xv = __ldg(xr + i), d = xv - __ldg(cr + i);
          d2[r] = fmaf(d, d, d2[r]);
          x2[r] = fmaf(xv, xv, x2[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        d2[r] += __shfl_xor_sync(0xffffffffu, d2[r], o);
        x2[r] += __shfl_xor_sync(0xffffffffu, x2[r], o);
      }
      if (lane == 0 && r < nr) {
        thr[rr[r]] = (d2[r] - x2[r]) + 2.0f * eps[rr[r]] + 4.0f * 5.9604645e-8f * (d2[r] + x2[r]);
        count[rr[r]] = 0;
      }
    }
  }
}

// |c_new - c_old| per centroid (one warp each), a hair above its fp32 value
__global__ void assign_shift_kernel(const float* __restrict__ cent, const float* __restrict__ old, int k, int dim,
                                    float* __restrict__ shift) {
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= k) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float d = cent[(int64_t)c * dim + i] - old[(int64_t)c * dim + i];
    s = fmaf(d, d, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) shift[c] = sqrtf(s) * (1.0f + 1e-5f);
}

// launches the vector form when the rows allow 16-byte loads; dist_old == nullptr: every row takes the exact form
static void launch_prev_threshold(Ctx* ctx, const float* rows, int64_t n, int dim, const float* centroids, const int32_t* assign,
                                  const float* eps, float* thr, int32_t* count, const float* dist_old, const float* shift,
                                  const float* xnorm, float ratio) {
  const bool vec = dim % 4 == 0 && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)centroids & 15) == 0;
  const unsigned grid = (unsigned)ceil_div(n, 256);
  if (vec)
    assign_prev_threshold_kernel<true><<<grid, 256, 0, ctx->stream>>>(rows, n, dim, centroids, assign, eps, thr, count, dist_old, shift, xnorm, ratio);
  else
    assign_prev_threshold_kernel<false><<<grid, 256, 0, ctx->stream>>>(rows, n, dim, centroids, assign, eps, thr, count, dist_old, shift, xnorm, ratio);
}

// one warp per data row: exact squared distances to the listed centroids
__global__ void assign_exact_kernel(const float* __restrict__ x, int64_t n, int dim, const float* __restrict__ cent,
                                    const uint64_t* __restrict__ keys, const int32_t* __restrict__ count,
                                    int32_t* __restrict__ assign, float* __restrict__ dist, int32_t* __restrict__ bad_rows,
                                    int32_t* bad_count, int parts) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n) return;
  const int lane = threadIdx.x & 31;
  // one 8-bit count per sub-list; the scan's column parts (2 or 4) each wrote one sub-list of kAssignCap / parts keys
  // parts == 0: one list of up to kAssignCap keys with a plain count (the stationary-block kernel)
  unsigned packed = (unsigned)count[row];
  int sub = kAssignCap;
  int total = 0;
  bool over = false;
  if (parts == 0) {
    total = (int)packed;
    over = total > kAssignCap;
    packed = (unsigned)min(total, 255);
    parts = 1;
  } else {
    sub = kAssignCap / parts;
    for (int p = 0; p < parts; ++p) {
      const int c = (int)((packed >> (8 * p)) & 0xffu);
      over |= c > sub;
      total += c;
    }
  }
  if (over || total <= 0) {
    if (lane == 0) bad_rows[atomicAdd(bad_count, 1)] = (int32_t)row;
    return;
  }
  const float* xr = x + row * dim;
  uint64_t bestk = kEmptyKey;
  for (int p = 0; p < parts; ++p)
  for (int c = 0; c < (int)((packed >> (8 * p)) & 0xffu); ++c) {
    const uint32_t id = (uint32_t)keys[row * kAssignCap + p * sub + c];
    const float* cr = cent + (int64_t)id * dim;
    float s = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float d = __ldg(xr + i) - __ldg(cr + i);
      s = fmaf(d, d, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    bestk = min(bestk, make_key(s, id));
  }
  if (lane == 0) {
    assign[row] = (int32_t)(uint32_t)bestk;
    if (dist) dist[row] = sqrtf(ordered_to_float((uint32_t)(bestk >> 32)));
  }
}

__global__ void scatter_best_kernel(const unsigned long long* __restrict__ best, const int32_t* __restrict__ rows,
                                    int64_t m, int32_t* __restrict__ assign, float* __restrict__ dist) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const unsigned long long b = best[i];
  assign[rows[i]] = (int32_t)(uint32_t)b;
  if (dist) dist[rows[i]] = sqrtf(ordered_to_float((uint32_t)(b >> 32)));
}

// Scale of the centroid operand and exponent of the folded term for one Lloyd iteration (device-side, nothing is
// read back).  With M = max |c|^2 / 2: the largest of the three fp16 pieces of s_c M 2^e / 16 should sit just below
// 2^14, and the constants on the data side, 4u and 2u with u = s_x 2^-e, must be normal fp16 numbers: u <= 2^13.  When u
// would be too large the centroid scale is lowered by the excess (the pieces shrink, e grows, u shrinks); the error
// bound is computed from the measured residuals of whatever scale is used, so it stays valid.
__global__ void assign_fold_setup_kernel(const unsigned* max_sq, float* scale_c, const float* scale_x, int* exp_out, float* u_out) {
  const float M = 0.5f * __uint_as_float(*max_sq);
  float sc = *scale_c;
  const float sx = *scale_x;
  int e = 0;
  if (M > 0.f && M < CUDART_INF_F) {
    int m2;
    frexpf(sc * M * 0.0625f, &m2);   // sc M / 16 = f 2^m2, f in [0.5, 1)
    e = 14 - m2;                     // brings it to [2^13, 2^14)
    int ex;
    frexpf(sx, &ex);                 // sx = 2^(ex-1)
    const int lu = (ex - 1) - e;     // log2 of u
    if (lu > 13) {
      const int shift = lu - 13;
      sc = ldexpf(sc, -shift);
      e += shift;
    } else if (lu < -14) {
      e -= (-14 - lu);               // u up to the smallest normal; the pieces only get smaller
    }
  }
  *scale_c = sc;
  *exp_out = e;
  *u_out = ldexpf(sx, -e);
}

// the data operand's fold columns hold the constant u (one 16-byte store of eight copies per thread)
// (u_done: the constant the columns hold already - a Lloyd iteration whose exponent has not changed writes nothing)
__global__ void assign_fill_fold_kernel(__half* __restrict__ rows16, int64_t n, int dim16, int col0, const float* __restrict__ u,
                                        const float* __restrict__ u_done) {
  if (*u == *u_done) return;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int chunks = kFoldCols / 8;
  if (i >= n * chunks) return;
  const int64_t row = i / chunks;
  const int c = (int)(i - row * chunks);
  const __half h = __float2half_rn(*u * (c == 0 ? 4.0f : 2.0f));   // columns 0-7: 4u, columns 8-15: 2u
  const __half2 h2 = __halves2half2(h, h);
  uint4 v;
  v.x = v.y = v.z = v.w = *reinterpret_cast<const unsigned*>(&h2);
  *reinterpret_cast<uint4*>(rows16 + row * dim16 + col0 + c * 8) = v;
}

template <int MODE>
int32_t launch_assign_scan(Ctx* ctx, const CUtensorMap& mx, const CUtensorMap& mc, const CUtensorMap& mxn, const CUtensorMap& mcn,
                           AsArgs a, unsigned* grid_out = nullptr, int64_t* log_cap_out = nullptr) {
  static bool attr_done = false;
  if (!attr_done) {
    VSK_CUDA(ctx, cudaFuncSetAttribute(assign_scan_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAsSmemBytes));
    attr_done = true;
  }
  const int sms = ctx->prop.multiProcessorCount;
  const int nb = (int)ceil_div(a.k, TN);
  const int64_t qtiles = ceil_div(a.n, TM);
  unsigned grid;
  if (nb <= sms) {
    a.groups = (int)std::max<int64_t>(1, std::min<int64_t>(sms / nb, qtiles));
    grid = (unsigned)(nb * a.groups);
  } else {
    a.groups = 1;
    grid = (unsigned)sms;
  }
  a.wait_limit = ctx->tuning.wait_limit_log2 > 0 ? (1u << std::min(ctx->tuning.wait_limit_log2, 30)) : 0u;
  a.log_cap = std::min<int64_t>(a.log_total / grid, 0x7fffffff);
  if (grid_out) *grid_out = grid;
  if (log_cap_out) *log_cap_out = a.log_cap;
  prof_begin(ctx);
  assign_scan_kernel<MODE><<<grid, AS_THREADS, kAsSmemBytes, ctx->stream>>>(mx, mc, mxn, mcn, a);
  prof_end(ctx);
  tl_mark(ctx, MODE == SCAN_ARGMIN ? "assign_argmin" : "assign_scan");
  ctx->stats.kernel_launches++;
  ctx->stats.tensor_tiles += (int64_t)nb * qtiles;
  VSK_CUDA(ctx, cudaGetLastError());
  return VSK_OK;
}

}  // namespace

void tensor_invalidate(Index* ix) { ix->n16 = -1; }
int32_t tensor_prepare_index(Index* ix) { return tensor_prepare(ix); }

// ---- query operands of a flat search ------------------------------------------------------------------
// fp16 operand rows of the queries, their error bound eps[q], the output coefficient alpha, and the small words a
// search needs (device error word, re-scored row counter), all in the current lane's scratch.
struct QueryOperands {
  __half* q16 = nullptr;
  float* eps = nullptr;
  float* alpha = nullptr;
  int32_t* err = nullptr;
  unsigned long long* rr_total = nullptr;
};

int32_t prepare_query_operands(Index* ix, const float* q, int64_t nq, QueryOperands* out) {
  VSK_TRACE("vsk:query_operands");
  Ctx* ctx = ix->ctx;
  static bool carveout_done = false;
  if (!carveout_done) {
    prefer_shared_carveout(absmax_kernel);
    prefer_shared_carveout(choose_scale_kernel);
    prefer_shared_carveout(scale_queries_kernel);
    prefer_shared_carveout(prep_rows_kernel<VSK_METRIC_EUCLIDEAN>);
    prefer_shared_carveout(prep_rows_kernel<VSK_METRIC_COSINE>);
    prefer_shared_carveout(prep_rows_kernel<VSK_METRIC_DOT_PRODUCT>);
    prefer_shared_carveout(bound_kernel<VSK_METRIC_EUCLIDEAN>);
    prefer_shared_carveout(bound_kernel<VSK_METRIC_COSINE>);
    prefer_shared_carveout(bound_kernel<VSK_METRIC_DOT_PRODUCT>);
    prefer_shared_carveout(bound_i8_kernel<VSK_METRIC_EUCLIDEAN>);
    prefer_shared_carveout(bound_i8_kernel<VSK_METRIC_DOT_PRODUCT>);
    prefer_shared_carveout(rerank_kernel<VSK_METRIC_EUCLIDEAN>);
    prefer_shared_carveout(rerank_kernel<VSK_METRIC_COSINE>);
    prefer_shared_carveout(rerank_kernel<VSK_METRIC_DOT_PRODUCT>);
    prefer_shared_carveout(rerank_i8_kernel<VSK_METRIC_EUCLIDEAN>);
    prefer_shared_carveout(rerank_i8_kernel<VSK_METRIC_DOT_PRODUCT>);
    carveout_done = true;
  }
  const int metric = ix->metric;
  const int dim = ix->dim, dim16 = ix->dim16;
  void* p;
  VSK_TRY(scratch(ctx, SLOT_Q16, (size_t)nq * dim16 * sizeof(__half), &p));
  __half* q16 = (__half*)p;
  VSK_TRY(scratch(ctx, SLOT_QAUX, (size_t)nq * 4 * sizeof(float) + 64, &p));
  float* qn16 = (float*)p;
  float* qe16 = qn16 + nq;
  float* eps = qe16 + nq;
  float* qn_tmp = eps + nq;
  VSK_TRY(scratch(ctx, SLOT_TC_B, 64, &p));
  unsigned* q_absmax = (unsigned*)p;
  float* q_scale = (float*)p + 1;
  float* alpha = (float*)p + 2;
  int32_t* err = (int32_t*)p + 3;
  unsigned long long* rr_total = (unsigned long long*)((char*)p + 16);
  VSK_CUDA(ctx, cudaMemsetAsync(p, 0, 64, ctx->stream));
  const bool cosine = metric == VSK_METRIC_COSINE;
  const bool i8 = ix->kind == INDEX_FLAT_I8;
  if (i8 && metric != VSK_METRIC_EUCLIDEAN && metric != VSK_METRIC_DOT_PRODUCT)
    return fail(ctx, VSK_ERR_UNSUPPORTED_OPERATION, "the tensor path over int8 codes covers euclidean and dotProduct");
  const float* qsrc = q;   // what the query operand is made from
  float* q_true_norm = nullptr;
  if (i8) {
    VSK_TRY(scratch(ctx, SLOT_TC_C, (size_t)nq * dim * sizeof(float), &p));
    float* qt = (float*)p;
    scale_queries_kernel<<<(unsigned)ceil_div(nq * (int64_t)dim, 256), 256, 0, ctx->stream>>>(q, nq * (int64_t)dim, dim, ix->sq_scale, qt);
    ctx->stats.kernel_launches++;
    qsrc = qt;
    VSK_TRY(scratch(ctx, SLOT_TC_D, (size_t)nq * sizeof(float), &p));
    q_true_norm = (float*)p;
    VSK_TRY(launch_row_norms(ctx, q, nq, dim, 0, q_true_norm));
  }
  if (!cosine) {
    absmax_kernel<<<296, 256, 0, ctx->stream>>>(qsrc, nq * (int64_t)dim, q_absmax);
    ctx->stats.kernel_launches++;
  }
  const bool fold = ix->fold16;
  const FoldArgs qfold{fold ? 2 : 0, fold_col0(ix->dim), ix->fold_exp};
  choose_scale_kernel<<<1, 1, 0, ctx->stream>>>(q_absmax, cosine ? 1 : 0, q_scale, fold ? 1 : 0, ix->fold_exp);
  ctx->stats.kernel_launches++;
  BoundConsts bc{ix->scale16, ix->max_xnorm16, ix->max_xerr16, ix->max_xnorm, ix->min_xnorm_nz, dim16, fold ? ix->fold_bmax : 0.f};
  const unsigned bgrid = (unsigned)ceil_div(nq, 256);
  if (i8) {
    launch_prep<VSK_METRIC_DOT_PRODUCT>(ctx, qsrc, nq, dim, dim16, q_scale, q16, nullptr, qn16, qe16, qn_tmp, nullptr);
    if (metric == VSK_METRIC_EUCLIDEAN)
      bound_i8_kernel<VSK_METRIC_EUCLIDEAN><<<bgrid, 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, q_true_norm, nq, q_scale, bc, eps, alpha);
    else
      bound_i8_kernel<VSK_METRIC_DOT_PRODUCT><<<bgrid, 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, q_true_norm, nq, q_scale, bc, eps, alpha);
  } else
  switch (metric) {
    case VSK_METRIC_EUCLIDEAN:
      launch_prep<VSK_METRIC_EUCLIDEAN>(ctx, q, nq, dim, dim16, q_scale, q16, nullptr, qn16, qe16, qn_tmp, nullptr, qfold);
      bound_kernel<VSK_METRIC_EUCLIDEAN><<<bgrid, 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, nq, q_scale, bc, eps, alpha);
      break;
    case VSK_METRIC_COSINE:
      launch_prep<VSK_METRIC_COSINE>(ctx, q, nq, dim, dim16, q_scale, q16, nullptr, qn16, qe16, qn_tmp, nullptr);
      bound_kernel<VSK_METRIC_COSINE><<<bgrid, 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, nq, q_scale, bc, eps, alpha);
      break;
    default:
      launch_prep<VSK_METRIC_DOT_PRODUCT>(ctx, q, nq, dim, dim16, q_scale, q16, nullptr, qn16, qe16, qn_tmp, nullptr);
      bound_kernel<VSK_METRIC_DOT_PRODUCT><<<bgrid, 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, nq, q_scale, bc, eps, alpha);
      break;
  }
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  tl_mark(ctx, "query_operands");
  out->q16 = q16;
  out->eps = eps;
  out->alpha = alpha;
  out->err = err;
  out->rr_total = rr_total;
  return VSK_OK;
}

int32_t cand_lists(Ctx* ctx, int64_t nq, CandLists* cand) {
  void* p;
  VSK_TRY(scratch(ctx, SLOT_CAND_KEYS, (size_t)nq * kCandCap * sizeof(uint64_t), &p));
  cand->keys = (uint64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_COUNT, (size_t)nq * 4, &p));
  cand->count = (int32_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_THR, (size_t)nq * 4, &p));
  cand->thr = (float*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_FLAGS, (size_t)nq * 4, &p));
  cand->flags = (int32_t*)p;
  cand->nq = nq;
  return VSK_OK;
}

// The search in two halves.  `begin` runs the scan and its compactions; `finish` certifies, re-scores and orders.
// A plain search calls them back to back.  A shard of a row-sharded search passes `bound_out` (and the number of
// shards): the last compaction is then left to `finish`, and bound_out[q] gets a value that this shard's
// ceil(k / shards) best rows do not exceed; the host takes the maximum over the shards (at least k rows overall lie
// below it) and hands it to `finish`, which keeps only rows that can still reach the overall top-k.
// qmasks (or null): per-query filter masks; rows are then filtered in the contraction's epilogue.
int32_t tensor_search_begin(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm, const uint64_t* qmasks,
                            int32_t shards, float* bound_out) {
  VSK_TRACE("vsk:scan");
  Ctx* ctx = ix->ctx;
  ctx->pending[ctx->lane] = ShardPending{};
  VSK_TRY(tensor_prepare(ix));
  const int metric = ix->metric;
  const int dim16 = ix->dim16;
  const int32_t keep = std::min<int32_t>(kCandCap / 2, k + std::max(8, k / 8));
  QueryOperands qo;
  VSK_TRY(prepare_query_operands(ix, q, nq, &qo));
  const bool fold = ix->fold16;

  CUtensorMap mq, mx;
  VSK_TRY(make_map(ctx, qo.q16, nq, dim16, TM, &mq));
  VSK_TRY(make_map(ctx, ix->rows16, ix->n, dim16, TN, &mx));

  // ---- candidate lists and the chunk schedule ----
  CandLists cand;
  VSK_TRY(cand_lists(ctx, nq, &cand));
  VSK_TRY(launch_init_cand(ctx, cand, nq));

  TcArgs a{};
  a.nq = nq;
  a.kblocks = dim16 / TK;
  a.k16_last = k16_last_of(fold ? fold_col0(ix->dim) + kFoldCols : ix->dim, dim16);
  a.alpha = qo.alpha;
  a.beta = (metric == VSK_METRIC_EUCLIDEAN && !fold) ? ix->row_aux : nullptr;
  a.cand = cand;
  a.cap = kCandCap;
  a.err = qo.err;
  if (qmasks && ix->has_masks) {
    a.row_masks = ix->masks;
    a.q_masks = qmasks;
  }
  const bool has_beta = a.beta != nullptr;
  SelectArgs sel{};
  sel.cand = cand;
  sel.nq = nq;
  sel.keep = keep;
  const int64_t n = ix->n;
  const int64_t room = kCandCap - keep;
  int64_t seen = std::min<int64_t>(n, schedule_dense_rows(ctx, keep));
  a.mode = SCAN_DENSE;
  a.row_begin = 0;
  a.row_end = seen;
  VSK_TRY(launch_tc<SCAN_DENSE>(ctx, mq, mx, a, has_beta));
  sel.dense_count = (int32_t)seen;
  sel.max_count = (int32_t)seen;
  sel.k = k;
  // the compaction after the last chunk keeps what the exact re-scoring needs and certifies the query; a shard
  // only measures its bound there and leaves that compaction to the second half
  auto last_select = [&]() {
    if (bound_out == nullptr) {
      sel.cert_eps = qo.eps;
    } else {
      sel.bound_out = bound_out;
      sel.bound_rank = (k + std::max(1, shards) - 1) / std::max(1, shards);
      sel.bound_eps = qo.eps;
    }
  };
  if (seen == n) last_select();
  VSK_TRY(launch_select(ctx, sel));
  sel.dense_count = -1;
  a.mode = SCAN_THRESHOLD;
  // A small batch is bound by its launches, not by its hits: fewer, faster-growing chunks (each still within what a
  // list can take, schedule_chunk) save a contraction and a compaction launch per step they skip.
  const int64_t growth = nq <= 2048 ? std::max(16, ctx->tuning.chunk_growth) : std::max(1, ctx->tuning.chunk_growth);
  while (seen < n) {
    // schedule_chunk bounds the chunk so that a list cannot plausibly overflow; below that bound chunks
    // grow geometrically (each no larger than three times the rows seen so far), which keeps the share of
    // rows scanned under a loose threshold small: the epilogue's append path costs far more than its filter.
    int64_t chunk = schedule_chunk(seen, keep, 0);
    chunk = std::min<int64_t>(chunk, std::max<int64_t>(growth >= 100 ? room : 1024, growth * seen));
    chunk = std::max<int64_t>(TN, chunk / TN * TN);   // whole row tiles
    chunk = std::min(chunk, n - seen);
    a.row_begin = seen;
    a.row_end = seen + chunk;
    VSK_TRY(launch_tc<SCAN_THRESHOLD>(ctx, mq, mx, a, has_beta));
    sel.max_count = schedule_max_count(seen, chunk, keep);
    seen += chunk;
    if (seen == n) last_select();
    VSK_TRY(launch_select(ctx, sel));
  }
  ShardPending& pd = ctx->pending[ctx->lane];
  pd.active = true;
  pd.tensor = true;
  pd.ix = ix;
  pd.q = q;
  pd.nq = nq;
  pd.k = k;
  pd.qnorm = qnorm;
  pd.qmasks = a.q_masks;
  pd.cand = cand;
  pd.eps = qo.eps;
  pd.err = qo.err;
  pd.rr_total = qo.rr_total;
  pd.keep = keep;
  pd.max_count = sel.max_count;
  pd.need_cert = bound_out != nullptr;
  return VSK_OK;
}

// Second half, part one: everything that can be enqueued without looking at results - the certifying compaction
// (a shard's), the exact re-scoring, the final order, and the copy of the flag words to pinned host memory.
int32_t tensor_search_finish_issue(Index* ix, const float* ext_bound, float* out_dist, int64_t* out_ids) {
  VSK_TRACE("vsk:finish");
  Ctx* ctx = ix->ctx;
  ShardPending& pd = ctx->pending[ctx->lane];
  if (!pd.active || !pd.tensor || pd.ix != ix || pd.issued)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "no search is waiting for its second half on this index");
  const float* q = pd.q;
  const float* qnorm = pd.qnorm;
  const int64_t nq = pd.nq;
  const int32_t k = pd.k, keep = pd.keep;
  const CandLists cand = pd.cand;
  const int metric = ix->metric;
  const int dim = ix->dim;
  const bool i8 = ix->kind == INDEX_FLAT_I8;
  if (pd.need_cert) {
    SelectArgs sel{};
    sel.cand = cand;
    sel.nq = nq;
    sel.keep = keep;
    sel.dense_count = -1;
    sel.k = k;
    sel.cert_eps = pd.eps;
    sel.ext_bound = ext_bound;
    sel.max_count = pd.max_count;
    VSK_TRY(launch_select(ctx, sel));
  }

  // ---- exact rerank + final order ----
  const size_t qsm = (size_t)dim * sizeof(float);
  if (qsm > 200 * 1024) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "dimension %d is too large for the rerank kernel", dim);
#define VSK_RERANK(M_)                                                                                          \
  do {                                                                                                          \
    if (qsm > 48 * 1024)                                                                                        \
      VSK_CUDA(ctx, cudaFuncSetAttribute(rerank_kernel<M_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)qsm)); \
    rerank_kernel<M_><<<(unsigned)nq, 256, qsm, ctx->stream>>>(q, ix->rows, dim, qnorm, ix->row_norm, cand, pd.rr_total); \
  } while (0)
  if (i8) {
    if (qsm > 48 * 1024) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "dimension %d is too large for the int8 rerank kernel", dim);
    if (metric == VSK_METRIC_EUCLIDEAN)
      rerank_i8_kernel<VSK_METRIC_EUCLIDEAN><<<(unsigned)nq, 256, qsm, ctx->stream>>>(q, ix->codes, dim, ix->sq_scale, ix->sq_offset, cand, pd.rr_total);
    else
      rerank_i8_kernel<VSK_METRIC_DOT_PRODUCT><<<(unsigned)nq, 256, qsm, ctx->stream>>>(q, ix->codes, dim, ix->sq_scale, ix->sq_offset, cand, pd.rr_total);
  } else
  switch (metric) {
    case VSK_METRIC_EUCLIDEAN: VSK_RERANK(VSK_METRIC_EUCLIDEAN); break;
    case VSK_METRIC_COSINE: VSK_RERANK(VSK_METRIC_COSINE); break;
    default: VSK_RERANK(VSK_METRIC_DOT_PRODUCT); break;
  }
#undef VSK_RERANK
  tl_mark(ctx, "rerank");
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  SelectArgs fin{};
  fin.cand = cand;
  fin.nq = nq;
  fin.dense_count = -1;
  fin.keep = k;
  fin.out_dist = out_dist;
  fin.out_ids = out_ids;
  fin.k = k;
  fin.metric = metric;
  fin.id_base = ix->id_base;
  fin.final_sqrt = metric == VSK_METRIC_EUCLIDEAN;
  fin.max_count = keep;
  VSK_TRY(launch_select(ctx, fin));

  // ---- flag words to the host: bounded-wait expiry, overflowed lists, failed certificates ----
  PinnedBuf& hb = ctx->host_flags[ctx->lane];
  VSK_TRY(pinned_reserve(ctx, &hb, (size_t)nq * 4 + 16));
  char* h = (char*)hb.p;
  VSK_CUDA(ctx, cudaMemcpyAsync(h, pd.err, 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(h + 8, pd.rr_total, 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(h + 16, cand.flags, (size_t)nq * 4, cudaMemcpyDeviceToHost, ctx->stream));
  pd.issued = true;
  pd.out_dist = out_dist;
  pd.out_ids = out_ids;
  return VSK_OK;
}

// Second half, part two, after the stream of lane `from_lane` has drained: reads that lane's flag words and re-runs
// on the fp32 scan (on the CURRENT lane) the queries whose candidate list overflowed or whose result could not be
// certified.
int32_t tensor_search_finish_collect(Index* ix, int from_lane) {
  Ctx* ctx = ix->ctx;
  if (from_lane < 0) from_lane = ctx->lane;
  const ShardPending pd = ctx->pending[from_lane];
  ctx->pending[from_lane] = ShardPending{};
  if (!pd.active || !pd.issued || pd.ix != ix)
    return fail(ctx, VSK_ERR_INVALID_INPUT, "no search is waiting to be collected on this index");
  const char* h = (const char*)ctx->host_flags[from_lane].p;
  int32_t herr;
  unsigned long long hrr;
  memcpy(&herr, h, 4);
  memcpy(&hrr, h + 8, 8);
  const int32_t* flags = (const int32_t*)(h + 16);
  ctx->stats.reranked_rows += (int64_t)hrr;
  if (herr != 0)
    return fail(ctx, VSK_ERR_TIMEOUT, "tensor-core scan: a bounded pipeline wait ran out (role %d)", herr);
  std::vector<int32_t> bad;
  for (int64_t i = 0; i < pd.nq; ++i)
    if (flags[i]) bad.push_back((int32_t)i);
  if (!bad.empty()) VSK_TRY(fp32_search_subset(ix, pd.q, bad, pd.k, pd.qnorm, pd.qmasks, pd.out_dist, pd.out_ids));
  return VSK_OK;
}

int32_t tensor_search_finish(Index* ix, const float* ext_bound, float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  VSK_TRY(tensor_search_finish_issue(ix, ext_bound, out_dist, out_ids));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return tensor_search_finish_collect(ix, -1);
}

// How a batch of nq queries is split over the two lanes: the first half's size (a whole number of query tiles), or 0
// for one lane.  Two lanes need enough queries that each half still fills the machine, and timing the scan kernels
// with events (vsk_profile) needs them alone on the device.
int64_t tensor_lane_split(const Ctx* ctx, int64_t nq) {
  const int64_t min_q = ctx->tuning.overlap_min_queries;
  if (min_q <= 0 || nq < min_q || nq < 4 * TM || ctx->profile) return 0;
  return ceil_div(ceil_div(nq, 2), TM) * TM;
}

int32_t tensor_search(Index* ix, const float* q, int64_t nq, int32_t k, const float* qnorm, const uint64_t* qmasks,
                      float* out_dist, int64_t* out_ids) {
  Ctx* ctx = ix->ctx;
  const int64_t na = ctx->lane == 0 ? tensor_lane_split(ctx, nq) : 0;
  if (na == 0) {
    VSK_TRY(tensor_search_begin(ix, q, nq, k, qnorm, qmasks, 1, nullptr));
    return tensor_search_finish(ix, nullptr, out_dist, out_ids);
  }
  // Two halves on two streams.  Each half is a complete search of its own queries (own candidate lists, own
  // operands); the device runs one half's compactions, re-scoring and final order while the other half's
  // contraction holds the tensor cores.
  VSK_TRY(tensor_prepare(ix));   // the shared operand copy is made before the lanes part
  const int64_t nb = nq - na;
  const float* qb = q + na * ix->dim;
  const float* qnb = qnorm ? qnorm + na : nullptr;
  const uint64_t* qmb = qmasks ? qmasks + na : nullptr;
  VSK_TRY(lanes_fork(ctx));
  int32_t st = VSK_OK;
  auto on_lane = [&](int lane, auto&& fn) {
    if (st != VSK_OK) return;
    LaneGuard g(ctx, lane);
    st = fn();
  };
  on_lane(0, [&] { return tensor_search_begin(ix, q, na, k, qnorm, qmasks, 1, nullptr); });
  on_lane(1, [&] { return tensor_search_begin(ix, qb, nb, k, qnb, qmb, 1, nullptr); });
  on_lane(0, [&] { return tensor_search_finish_issue(ix, nullptr, out_dist, out_ids); });
  on_lane(1, [&] { return tensor_search_finish_issue(ix, nullptr, out_dist + na * k, out_ids + na * k); });
  const int32_t jst = lanes_join(ctx);
  cudaStreamSynchronize(ctx->stream_main);   // lane 1 has joined: both halves are complete (or failed)
  if (st != VSK_OK || jst != VSK_OK) {
    cudaStreamSynchronize(ctx->stream_aux);
    ctx->pending[0] = ShardPending{};
    ctx->pending[1] = ShardPending{};
    return st != VSK_OK ? st : jst;
  }
  // flagged queries of either half are re-run on lane 0, whose own work is over
  const int32_t sa = tensor_search_finish_collect(ix, 0);
  const int32_t sb = tensor_search_finish_collect(ix, 1);
  return sa != VSK_OK ? sa : sb;
}

// keys of a dense chunk -> their values, row-major [nq][rows]
__global__ void keys_to_values_kernel(const uint64_t* __restrict__ keys, int64_t nq, int64_t rows, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq * rows) return;
  const int64_t q = i / rows, r = i - q * rows;
  out[i] = ordered_to_float((uint32_t)(keys[q * kCandCap + r] >> 32));
}

// The coarse values of the first `rows` rows (one dense chunk of the scan) and the bound the certificate assumes.
int32_t tensor_coarse_values(Index* ix, const float* q, int64_t nq, int64_t rows, float* coarse, float* eps_out) {
  Ctx* ctx = ix->ctx;
  if (rows <= 0 || rows > kCandCap || rows > ix->n)
    return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "rows must be in [1, min(%d, index size)]", kCandCap);
  VSK_TRY(tensor_prepare(ix));
  QueryOperands qo;
  VSK_TRY(prepare_query_operands(ix, q, nq, &qo));
  CUtensorMap mq, mx;
  VSK_TRY(make_map(ctx, qo.q16, nq, ix->dim16, TM, &mq));
  VSK_TRY(make_map(ctx, ix->rows16, ix->n, ix->dim16, TN, &mx));
  CandLists cand;
  VSK_TRY(cand_lists(ctx, nq, &cand));
  VSK_TRY(launch_init_cand(ctx, cand, nq));
  TcArgs a{};
  a.nq = nq;
  a.kblocks = ix->dim16 / TK;
  a.k16_last = k16_last_of(ix->fold16 ? fold_col0(ix->dim) + kFoldCols : ix->dim, ix->dim16);
  a.alpha = qo.alpha;
  a.beta = (ix->metric == VSK_METRIC_EUCLIDEAN && !ix->fold16) ? ix->row_aux : nullptr;
  a.cand = cand;
  a.cap = kCandCap;
  a.err = qo.err;
  a.mode = SCAN_DENSE;
  a.row_begin = 0;
  a.row_end = rows;
  VSK_TRY(launch_tc<SCAN_DENSE>(ctx, mq, mx, a, a.beta != nullptr));
  keys_to_values_kernel<<<(unsigned)ceil_div(nq * rows, 256), 256, 0, ctx->stream>>>(cand.keys, nq, rows, coarse);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  if (eps_out) VSK_CUDA(ctx, cudaMemcpyAsync(eps_out, qo.eps, (size_t)nq * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  int32_t herr = 0;
  VSK_CUDA(ctx, cudaMemcpyAsync(&herr, qo.err, 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (herr != 0) return fail(ctx, VSK_ERR_TIMEOUT, "tensor-core scan: a bounded pipeline wait ran out (role %d)", herr);
  return VSK_OK;
}


// ---- IVF list scan on the tensor cores --------------------------------------------------------------
// The probed lists of a batch, scanned with the same contraction kernel as the flat search.  Every (query, probed
// list) pair is an item; items are grouped by (stage, list), and the fp16 query operand is gathered in that order,
// so the queries that probe a list are consecutive rows of the "query" operand and a tile is 128 of them against
// 256 rows of the list.  The tiles of a launch are listed list by list (a list's rows are read from HBM once).
// Three launches: a pilot over the first rows of every query's nearest list with no threshold, then the remaining
// probe ranks in two groups (the rest of the nearest list is an item of the first group).  The kernel filters on
// the flat path's coarse values (|x|^2 - 2 q.x from fp16 operands); after every launch all listed rows are
// re-scored exactly and the k best exact values are kept, so thresholds are exact and the filter only has to be
// loose by the coarse values' error bound: no certificate is needed and the only queries handed back are those
// whose list overflowed.
constexpr int kIvfPilotTiles = 4;   // 1 024 rows of the nearest list set the first threshold

// key of item (query, slot): stage * nlist + list, or null_key.  Slot p < nprobe is probe rank p (stage 0 for the
// nearest list, 1 for ranks below r1, 2 above); slot nprobe is the rest of the nearest list beyond the pilot window.
__global__ void ivf_item_keys_kernel(const int64_t* __restrict__ probes, int64_t nq, int nprobe, int nlist, int r1,
                                     const int64_t* __restrict__ list_off, int64_t pilot_rows, int null_key,
                                     int32_t* __restrict__ keys) {
  const int slots = nprobe + 1;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq * slots) return;
  const int64_t pos = i / slots;
  const int p = (int)(i - pos * slots);
  int key = null_key;
  if (p < nprobe) {
    const int64_t l = probes[pos * nprobe + p];
    if (l >= 0 && l < nlist) key = (p == 0 ? 0 : (p < r1 ? 1 : 2)) * nlist + (int)l;
  } else {
    const int64_t l = probes[pos * nprobe];
    if (l >= 0 && l < nlist && list_off[l + 1] - list_off[l] > pilot_rows) key = nlist + (int)l;
  }
  keys[i] = key;
}

// per grouped item: its query and whether it is a remainder item; and the item's row of the gathered fp16 operand
__global__ void ivf_gather_items_kernel(const int32_t* __restrict__ order, int64_t nitems, int slots,
                                        const __half* __restrict__ q16, int dim16, uint32_t* __restrict__ pair_info,
                                        __half* __restrict__ g16) {
  const int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nitems) return;
  const int item = order[i];
  const int pos = item / slots;
  const int lane = threadIdx.x & 31;
  if (lane == 0) pair_info[i] = (uint32_t)pos | ((item - pos * slots) == slots - 1 ? 0x80000000u : 0u);
  const uint4* src = reinterpret_cast<const uint4*>(q16 + (int64_t)pos * dim16);
  uint4* dst = reinterpret_cast<uint4*>(g16 + i * dim16);
  for (int c = lane; c < dim16 / 8; c += 32) dst[c] = __ldg(src + c);
}

// tiles of (stage, list): ceil(pairs / 128) x row tiles (the pilot takes only the window)
__device__ __forceinline__ int ivf_row_tiles(int64_t len, int stage, int pilot_tiles) {
  const int t = (int)((len + TN - 1) / TN);
  return stage == 0 ? min(pilot_tiles, t) : t;
}

__global__ void ivf_tile_count_kernel(const int64_t* __restrict__ pair_off, int stage, int nlist,
                                      const int64_t* __restrict__ list_off, int64_t* __restrict__ counts,
                                      int pilot_tiles) {
  const int l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= nlist) return;
  const int64_t pairs = pair_off[(int64_t)stage * nlist + l + 1] - pair_off[(int64_t)stage * nlist + l];
  counts[l] = ((pairs + TM - 1) / TM) * ivf_row_tiles(list_off[l + 1] - list_off[l], stage, pilot_tiles);
}

__global__ void ivf_tile_fill_kernel(const int64_t* __restrict__ pair_off, int stage, int nlist,
                                     const int64_t* __restrict__ list_off, const int64_t* __restrict__ offsets,
                                     int4* __restrict__ tiles, int pilot_tiles) {
  const int l = blockIdx.x;
  const int64_t pbeg = pair_off[(int64_t)stage * nlist + l], pairs = pair_off[(int64_t)stage * nlist + l + 1] - pbeg;
  const int64_t beg = list_off[l], len = list_off[l + 1] - beg;
  const int ptiles = (int)((pairs + TM - 1) / TM), rtiles = ivf_row_tiles(len, stage, pilot_tiles);
  int4* out = tiles + offsets[l];
  for (int i = threadIdx.x; i < ptiles * rtiles; i += blockDim.x) {
    const int rt = i / ptiles, pt = i - rt * ptiles;
    const int64_t r0 = (int64_t)rt * TN;
    out[i] = make_int4((int)(pbeg + (int64_t)pt * TM), (int)(beg + r0),
                       (int)min((int64_t)TN, len - r0) | ((rt < pilot_tiles ? 1 : 0) << 30),
                       (int)min((int64_t)TM, pairs - (int64_t)pt * TM));
  }
}

// after the exact rerank: a key's row field goes from its storage position to the row's insertion index, so that
// the final order breaks ties the way the fp32 list scan does
__global__ void ivf_remap_keys_kernel(CandLists cand, int64_t nq, const int32_t* __restrict__ list_rows) {
  const int64_t qi = blockIdx.x;
  const int cnt = min(cand.count[qi], kCandCap);
  uint64_t* keys = cand.keys + qi * kCandCap;
  for (int c = threadIdx.x; c < cnt; c += blockDim.x) {
    const uint64_t key = keys[c];
    if (key != kEmptyKey) keys[c] = (key & 0xffffffff00000000ull) | (uint32_t)list_rows[(uint32_t)key];
  }
}

// Coarse-domain threshold of a query from its exact one.  A row's exact squared distance is |q|^2 + c with
// c = |x|^2 - 2 q.x, and its coarse value differs from c by at most eps, so every row with exact value <= T has
// coarse value <= T - |q|^2 + eps; the last term covers fp32 rounding of the quantities being compared.
// `dropped` (or null): the smallest coarse value the pilot's coarse pre-selection dropped for the query.  The pilot
// keeps only its best rows by coarse value before the exact re-scoring; that is safe iff everything it dropped lies
// above the coarse threshold, otherwise the query is flagged for the fp32 list scan.
__global__ void ivf_coarse_threshold_kernel(const float* __restrict__ thr_exact, const float* __restrict__ qnorm,
                                            const float* __restrict__ eps, float max_xnorm, int64_t nq,
                                            float* __restrict__ thr_coarse, const float* __restrict__ dropped,
                                            int32_t* __restrict__ flags) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq) return;
  const float t = thr_exact[i];
  float tc = CUDART_INF_F;
  if (t < CUDART_INF_F) {
    const float qn2 = qnorm[i] * qnorm[i];
    tc = (t - qn2) + eps[i] + 2e-6f * (qn2 + max_xnorm * max_xnorm + t);
  }
  thr_coarse[i] = tc;
  if (dropped && dropped[i] <= tc) atomicOr(&flags[i], 2);
}

// saved[i] = thr[i]; thr[i] = +inf (the next compaction works on exact values and must not inherit a coarse one)
__global__ void ivf_save_threshold_kernel(float* __restrict__ thr, float* __restrict__ saved, int64_t nq) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nq) return;
  saved[i] = thr[i];
  thr[i] = CUDART_INF_F;
}

// threshold of every item's query, so that the scan reads it with the item's index
__global__ void ivf_pair_threshold_kernel(const uint32_t* __restrict__ pair_info, int64_t nitems,
                                          const float* __restrict__ thr_coarse, float* __restrict__ pair_thr) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nitems) pair_thr[i] = thr_coarse[pair_info[i] & 0x7fffffffu];
}

bool ivf_tensor_applicable(const Index* ix, int64_t nq, int32_t nprobe, int32_t k) {
  return ix->kind == INDEX_IVF && nq >= 2 * TM && k <= kCandCap / 4 && ix->n >= 8 * TN &&
         (int64_t)nq * (nprobe + 1) < ((int64_t)1 << 30);
}

int32_t ivf_tensor_search(Index* ix, const float* q, int64_t nq, const int64_t* probes, int32_t nprobe, int32_t k,
                          const uint64_t* qmasks, float* out_dist, int64_t* out_ids, std::vector<int32_t>* flagged) {
  VSK_TRACE("vsk:ivf_list_scan");
  Ctx* ctx = ix->ctx;
  flagged->clear();
  VSK_TRY(tensor_prepare(ix));
  const int dim = ix->dim, dim16 = ix->dim16, nlist = ix->nlist;
  const int32_t keep = k;   // every compaction works on exact values, so no margin is needed
  void* p;

  // ---- query operands, bound, alpha (euclidean) ----
  VSK_TRY(scratch(ctx, SLOT_Q16, (size_t)nq * dim16 * sizeof(__half), &p));
  __half* q16 = (__half*)p;
  VSK_TRY(scratch(ctx, SLOT_QAUX, (size_t)nq * 4 * sizeof(float) + 64, &p));
  float* qn16 = (float*)p;
  float* qe16 = qn16 + nq;
  float* eps = qe16 + nq;
  float* qn_tmp = eps + nq;
  VSK_TRY(scratch(ctx, SLOT_TC_B, 64, &p));
  unsigned* q_absmax = (unsigned*)p;
  float* q_scale = (float*)p + 1;
  float* alpha = (float*)p + 2;
  int32_t* err = (int32_t*)p + 3;
  unsigned long long* rr_total = (unsigned long long*)((char*)p + 16);
  VSK_CUDA(ctx, cudaMemsetAsync(p, 0, 64, ctx->stream));
  absmax_kernel<<<296, 256, 0, ctx->stream>>>(q, nq * (int64_t)dim, q_absmax);
  const bool fold = ix->fold16;
  const FoldArgs qfold{fold ? 2 : 0, fold_col0(ix->dim), ix->fold_exp};
  choose_scale_kernel<<<1, 1, 0, ctx->stream>>>(q_absmax, 0, q_scale, fold ? 1 : 0, ix->fold_exp);
  ctx->stats.kernel_launches += 2;
  BoundConsts bc{ix->scale16, ix->max_xnorm16, ix->max_xerr16, ix->max_xnorm, ix->min_xnorm_nz, dim16, fold ? ix->fold_bmax : 0.f};
  launch_prep<VSK_METRIC_EUCLIDEAN>(ctx, q, nq, dim, dim16, q_scale, q16, nullptr, qn16, qe16, qn_tmp, nullptr, qfold);
  bound_kernel<VSK_METRIC_EUCLIDEAN><<<(unsigned)ceil_div(nq, 256), 256, 0, ctx->stream>>>(qn16, qe16, qn_tmp, nq, q_scale, bc, eps, alpha);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());

  // ---- stage plan: which probe ranks go with the remainder of the nearest list ----
  const double mean_len = std::max(1.0, (double)ix->n / (double)nlist);
  const int pilot_tiles = ctx->tuning.ivf_pilot_tiles > 0 ? ctx->tuning.ivf_pilot_tiles : kIvfPilotTiles;
  const int64_t pilot_rows = (int64_t)pilot_tiles * TN;
  // rows one launch may add after the pilot's rows without (plausibly) overflowing a list: the flat schedule's rule.
  // When all probed lists fit, one launch takes every remaining rank; otherwise the ranks are split in two groups.
  const double chunk = (double)schedule_chunk(pilot_rows, keep, 0);
  int r1 = mean_len * nprobe <= chunk ? (int)nprobe : (int)(chunk / 4.0 / mean_len);
  r1 = std::max(1, std::min(r1, (int)nprobe));
  const int nstages = r1 < nprobe ? 3 : 2;

  // ---- items grouped by (stage, list); the query operand gathered in that order ----
  const int slots = nprobe + 1;
  const int64_t nitems = nq * slots;
  const int nkeys = 3 * nlist + 1;
  VSK_TRY(scratch(ctx, SLOT_IVF_KEYS, (size_t)nitems * 4, &p));
  int32_t* keys = (int32_t*)p;
  VSK_TRY(scratch(ctx, SLOT_IVF_ORDER, (size_t)nitems * 4, &p));
  int32_t* order = (int32_t*)p;
  VSK_TRY(scratch(ctx, SLOT_IVF_PAIR_OFF, (size_t)(nkeys + 1) * 8, &p));
  int64_t* pair_off = (int64_t*)p;
  ivf_item_keys_kernel<<<(unsigned)ceil_div(nitems, 256), 256, 0, ctx->stream>>>(probes, nq, nprobe, nlist, r1, ix->list_offsets,
                                                                              pilot_rows, nkeys - 1, keys);
  ctx->stats.kernel_launches++;
  VSK_TRY(launch_stable_group(ctx, keys, nitems, nkeys, order, pair_off));
  VSK_TRY(scratch(ctx, SLOT_IVF_SUBSET, (size_t)(nitems + TM) * 8, &p));   // one tile of padding behind each array
  uint32_t* pair_info = (uint32_t*)p;
  float* pair_thr = (float*)(pair_info + nitems + TM);
  VSK_CUDA(ctx, cudaMemsetAsync(pair_info, 0, (size_t)(nitems + TM) * 8, ctx->stream));
  VSK_TRY(scratch(ctx, SLOT_IVF_STAGES, (size_t)(nitems + TM) * dim16 * sizeof(__half), &p));
  __half* g16 = (__half*)p;
  ivf_gather_items_kernel<<<(unsigned)ceil_div(nitems, 8), 256, 0, ctx->stream>>>(order, nitems, slots, q16, dim16, pair_info, g16);
  ctx->stats.kernel_launches++;

  CUtensorMap mq, mx;
  VSK_TRY(make_map(ctx, g16, nitems, dim16, TM, &mq));
  VSK_TRY(make_map(ctx, ix->rows16, ix->n, dim16, TN, &mx));

  CandLists cand;
  VSK_TRY(scratch(ctx, SLOT_CAND_KEYS, (size_t)nq * kCandCap * sizeof(uint64_t), &p));
  cand.keys = (uint64_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_COUNT, (size_t)nq * 4, &p));
  cand.count = (int32_t*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_THR, (size_t)nq * 4, &p));
  cand.thr = (float*)p;
  VSK_TRY(scratch(ctx, SLOT_CAND_FLAGS, (size_t)nq * 4, &p));
  cand.flags = (int32_t*)p;
  cand.nq = nq;
  VSK_TRY(launch_init_cand(ctx, cand, nq));

  // the kernel filters on coarse values: it sees the lists with a coarse threshold derived from the exact one
  VSK_TRY(scratch(ctx, SLOT_TC_D, (size_t)nq * sizeof(float), &p));
  float* thr_coarse = (float*)p;
  CandLists cand_coarse = cand;
  cand_coarse.thr = thr_coarse;
  VSK_TRY(scratch(ctx, SLOT_TC_C, (size_t)nq * sizeof(float), &p));
  float* pilot_dropped = (float*)p;
  const int32_t pilot_keep = std::min<int32_t>(1024, std::max(8 * k, 256));
  TcArgs a{};
  a.nq = nq;
  a.kblocks = dim16 / TK;
  a.k16_last = k16_last_of(fold ? fold_col0(ix->dim) + kFoldCols : ix->dim, dim16);
  a.mode = SCAN_THRESHOLD;
  a.alpha = alpha;
  a.beta = fold ? nullptr : ix->row_aux;
  a.cand = cand_coarse;
  a.cap = kCandCap;
  a.err = err;
  a.pair_info = pair_info;
  if (qmasks && ix->has_masks) {   // masks are kept in storage order, the order of the row operand
    a.row_masks = ix->masks;
    a.q_masks = qmasks;
  }
  SelectArgs sel{};
  sel.cand = cand;
  sel.nq = nq;
  sel.keep = keep;
  sel.dense_count = -1;
  sel.k = k;
  const size_t qsm = (size_t)dim * sizeof(float);
  if (qsm > 48 * 1024) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "dimension %d is too large for the rerank kernel", dim);
  const unsigned qgrid = (unsigned)ceil_div(nq, 256);

  void *cnt_p, *off_p;
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_CNT, (size_t)(nlist + 1) * 8, &cnt_p));
  VSK_TRY(scratch(ctx, SLOT_IVF_ITEM_OFF, (size_t)(nlist + 1) * 8, &off_p));
  for (int stage = 0; stage < nstages; ++stage) {
    ivf_tile_count_kernel<<<(unsigned)ceil_div(nlist, 256), 256, 0, ctx->stream>>>(pair_off, stage, nlist, ix->list_offsets, (int64_t*)cnt_p, pilot_tiles);
    VSK_TRY(launch_scan_i64(ctx, (const int64_t*)cnt_p, nlist, (int64_t*)off_p));
    int64_t total = 0;
    VSK_CUDA(ctx, cudaMemcpyAsync(&total, (int64_t*)off_p + nlist, 8, cudaMemcpyDeviceToHost, ctx->stream));
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->stats.kernel_launches += 2;
    if (total <= 0) continue;
    if (total > 0x7fffffffLL) return fail(ctx, VSK_ERR_INVALID_BUFFER_SIZE, "too many list tiles in one launch");
    VSK_TRY(scratch(ctx, SLOT_X_TMP, (size_t)total * sizeof(int4), &p));
    ivf_tile_fill_kernel<<<(unsigned)nlist, 128, 0, ctx->stream>>>(pair_off, stage, nlist, ix->list_offsets, (const int64_t*)off_p, (int4*)p, pilot_tiles);
    ivf_coarse_threshold_kernel<<<qgrid, 256, 0, ctx->stream>>>(cand.thr, qn_tmp, eps, ix->max_xnorm, nq, thr_coarse,
                                                                nullptr, cand.flags);
    ivf_pair_threshold_kernel<<<(unsigned)ceil_div(nitems, 256), 256, 0, ctx->stream>>>(pair_info, nitems, thr_coarse, pair_thr);
    ctx->stats.kernel_launches += 3;
    a.tiles = (const int4*)p;
    a.num_tiles = total;
    a.pair_thr = pair_thr;
    VSK_TRY(launch_tc<SCAN_THRESHOLD>(ctx, mq, mx, a, !fold));
    if (stage == 0) {
      // the pilot appended up to 1 024 rows per query: keep the best few by coarse value and re-score only those
      SelectArgs pre = sel;
      pre.keep = pilot_keep;
      pre.max_count = (int32_t)pilot_rows;
      VSK_TRY(launch_select(ctx, pre));
      ivf_save_threshold_kernel<<<qgrid, 256, 0, ctx->stream>>>(cand.thr, pilot_dropped, nq);
      ctx->stats.kernel_launches++;
    }
    // exact values for everything in the lists (the keys kept so far are re-scored too: at most k of them),
    // then the k best exact values stay and the k-th becomes the query's exact threshold
    rerank_kernel<VSK_METRIC_EUCLIDEAN><<<(unsigned)nq, 256, qsm, ctx->stream>>>(q, ix->rows, dim, nullptr, nullptr, cand, rr_total);
    ctx->stats.kernel_launches++;
    sel.max_count = stage == 0 ? pilot_keep : kCandCap;
    VSK_TRY(launch_select(ctx, sel));
    if (stage == 0) {
      // was the coarse pre-selection safe?  (also refreshes the coarse thresholds, which the next launch recomputes)
      ivf_coarse_threshold_kernel<<<qgrid, 256, 0, ctx->stream>>>(cand.thr, qn_tmp, eps, ix->max_xnorm, nq, thr_coarse,
                                                                  pilot_dropped, cand.flags);
      ctx->stats.kernel_launches++;
    }
  }

  // ---- ids back to insertion order, final order ----
  ivf_remap_keys_kernel<<<(unsigned)nq, 128, 0, ctx->stream>>>(cand, nq, ix->list_rows);
  ctx->stats.kernel_launches++;
  VSK_CUDA(ctx, cudaGetLastError());
  SelectArgs fin{};
  fin.cand = cand;
  fin.nq = nq;
  fin.dense_count = -1;
  fin.keep = k;
  fin.out_dist = out_dist;
  fin.out_ids = out_ids;
  fin.k = k;
  fin.metric = VSK_METRIC_EUCLIDEAN;
  fin.id_base = ix->id_base;
  fin.final_sqrt = 1;
  fin.max_count = keep;
  VSK_TRY(launch_select(ctx, fin));

  std::vector<int32_t> flags((size_t)nq);
  int32_t herr = 0;
  unsigned long long hrr = 0;
  VSK_CUDA(ctx, cudaMemcpyAsync(flags.data(), cand.flags, nq * 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(&herr, err, 4, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaMemcpyAsync(&hrr, rr_total, 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  ctx->stats.reranked_rows += (int64_t)hrr;
  if (herr != 0)
    return fail(ctx, VSK_ERR_TIMEOUT, "tensor-core scan: a bounded pipeline wait ran out (role %d)", herr);
  for (int64_t i = 0; i < nq; ++i)
    if (flags[i]) flagged->push_back((int32_t)i);
  return VSK_OK;
}

// ---- public: tensor-core nearest-centroid assignment (used by kmeans.cu) ---------------------------
int32_t tensor_assign_prepare(Ctx* ctx, const float* rows, int64_t n, int32_t dim, TensorAssign* ta) {
  ta->n = n;
  ta->dim = dim;
  // Short contractions keep a block of centroids resident (assign_scan_kernel): the operands then carry 16 more
  // columns for the folded |c|^2 / 2 term.  Longer ones (more than four k-blocks with those columns) take the general kernel.
  ta->stationary = fold_col0(dim) + kFoldCols <= AS_MAX_KB * TK;
  ta->dim16 = (int32_t)(ceil_div(ta->stationary ? fold_col0(dim) + kFoldCols : dim, TK) * TK);
  VSK_TRY(dev_alloc(ctx, (void**)&ta->rows16, (size_t)n * ta->dim16 * sizeof(__half)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->stats, (size_t)n * 4 * sizeof(float)));
  // stationary kernel: `keys` is the hit log (a hit or two per row as a rule; six entries per row of room)
  VSK_TRY(dev_alloc(ctx, (void**)&ta->keys, (size_t)n * (ta->stationary ? kAssignLogPerRow : kAssignCap) * sizeof(uint64_t)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->best, (size_t)n * sizeof(unsigned long long)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->count, (size_t)n * sizeof(int32_t)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->thr, (size_t)n * sizeof(float)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->bad_rows, (size_t)n * sizeof(int32_t)));
  VSK_TRY(dev_alloc(ctx, (void**)&ta->small, 256));
  VSK_CUDA(ctx, cudaMemsetAsync(ta->small, 0, 256, ctx->stream));
  // small: [0] absmax(rows) [1] scale_x [2] absmax(cent) [3] scale_c [4] alpha [5] err [6] bad_count, then PrepStats at +64
  unsigned* sm = (unsigned*)ta->small;
  absmax_kernel<<<1184, 256, 0, ctx->stream>>>(rows, n * (int64_t)dim, sm + 0);
  choose_scale_kernel<<<1, 1, 0, ctx->stream>>>(sm + 0, 0, (float*)sm + 1);
  float* st = (float*)ta->stats;
  launch_prep<VSK_METRIC_DOT_PRODUCT>(ctx, rows, n, dim, ta->dim16, (float*)sm + 1, ta->rows16, nullptr, st, st + n, st + 2 * n, nullptr);
  ctx->stats.kernel_launches += 2;
  VSK_CUDA(ctx, cudaGetLastError());
  VSK_TRY(make_map(ctx, ta->rows16, n, ta->dim16, TM, (CUtensorMap*)ta->map_rows));
  VSK_TRY(make_map_narrow(ctx, ta->rows16, n, ta->dim16, TM, (CUtensorMap*)ta->map_rows_narrow));
  return VSK_OK;
}

void tensor_assign_release(TensorAssign* ta) {
  dev_free(ta->rows16); dev_free(ta->stats); dev_free(ta->keys); dev_free(ta->best); dev_free(ta->count);
  dev_free(ta->thr); dev_free(ta->bad_rows); dev_free(ta->small); dev_free(ta->prev_cent); dev_free(ta->shift);
  *ta = TensorAssign{};
}

int32_t tensor_assign(Ctx* ctx, TensorAssign* ta, const float* rows, const float* centroids, int32_t k,
                      int32_t* assign, float* dist, bool assign_holds_previous) {
  VSK_TRACE("vsk:assign");
  static_assert(sizeof(CUtensorMap) <= sizeof(ta->map_rows), "tensor map storage too small");
  const int64_t n = ta->n;
  const int dim = ta->dim, dim16 = ta->dim16;
  unsigned* sm = (unsigned*)ta->small;
  float* fsm = (float*)ta->small;
  PrepStats* cs = (PrepStats*)((char*)ta->small + 64);
  float* st = (float*)ta->stats;
  float* eps = st + 3 * n;
  // centroid operand: fp16 rows, |c|^2, stats
  void* p;
  VSK_TRY(scratch(ctx, SLOT_TC_C, (size_t)k * dim16 * sizeof(__half), &p));
  __half* c16 = (__half*)p;
  VSK_TRY(scratch(ctx, SLOT_TC_D, (size_t)k * sizeof(float), &p));
  float* caux = (float*)p;
  PrepStats init{0u, 0u, 0u, 0u, 0x7f800000u};
  VSK_CUDA(ctx, cudaMemcpyAsync(cs, &init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
  VSK_CUDA(ctx, cudaMemsetAsync(sm + 2, 0, 4, ctx->stream));
  VSK_CUDA(ctx, cudaMemsetAsync(sm + 5, 0, 8, ctx->stream));
  absmax_kernel<<<64, 256, 0, ctx->stream>>>(centroids, (int64_t)k * dim, sm + 2);
  choose_scale_kernel<<<1, 1, 0, ctx->stream>>>(sm + 2, 0, fsm + 3);
  FoldArgs cfold{0, 0, 0};
  if (ta->stationary) {
    // words 24..27 of `small`: max |c|^2, the fold exponent, (unused), the data side's constant
    VSK_CUDA(ctx, cudaMemsetAsync(sm + 24, 0, 16, ctx->stream));
    max_sq_kernel<<<(unsigned)ceil_div(k, 8), 256, 0, ctx->stream>>>(centroids, k, dim, sm + 24);
    assign_fold_setup_kernel<<<1, 1, 0, ctx->stream>>>(sm + 24, fsm + 3, fsm + 1, (int*)sm + 25, fsm + 27);
    // word 30: the constant the data operand's fold columns hold (0 = none yet; a real constant is a power of two)
    assign_fill_fold_kernel<<<(unsigned)ceil_div(n * (kFoldCols / 8), 256), 256, 0, ctx->stream>>>(ta->rows16, n, dim16, fold_col0(dim), fsm + 27, fsm + 30);
    VSK_CUDA(ctx, cudaMemcpyAsync(fsm + 30, fsm + 27, sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    ctx->stats.kernel_launches += 3;
    cfold = FoldArgs{1, fold_col0(dim), 0, (const int*)sm + 25};
  }
  launch_prep<VSK_METRIC_EUCLIDEAN>(ctx, centroids, k, dim, dim16, fsm + 3, c16, caux, nullptr, nullptr, nullptr, cs, cfold);
  assign_bound_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(st, st + n, st + 2 * n, n, fsm + 1, fsm + 3, cs, dim16, eps, fsm + 4,
                                                                         ta->stationary ? 1 : 0);
  ctx->stats.kernel_launches += 3;
  VSK_CUDA(ctx, cudaGetLastError());
  CUtensorMap mc;
  VSK_TRY(make_map(ctx, c16, k, dim16, TN, &mc));
  const CUtensorMap& mr = *(const CUtensorMap*)ta->map_rows;
  CUtensorMap mcn;
  VSK_TRY(make_map_narrow(ctx, c16, k, dim16, TN, &mcn));
  const CUtensorMap& mrn = *(const CUtensorMap*)ta->map_rows_narrow;
  if (ta->stationary) {
    AsArgs sa{};
    sa.n = n;
    sa.k = k;
    sa.kblocks = dim16 / TK;
    sa.k16_last = k16_last_of(fold_col0(dim) + kFoldCols, dim16);
    sa.max_stages = ctx->tuning.assign_stages;
    sa.narrow_ok = 1;
    sa.alpha = fsm + 4;
    sa.thr = ta->thr;
    // the hit log lives in the rows' key lists (n x kAssignCap words of 8 bytes), its per-CTA counts in `count`
    sa.log = reinterpret_cast<uint2*>(ta->keys);
    sa.log_total = n * (int64_t)kAssignLogPerRow;
    sa.log_count = ta->count;
    sa.best = ta->best;
    sa.err = (int32_t*)(sm + 5);
    // The centroids of the previous call and how far each has moved since: rows whose centroid has hardly moved take
    // their threshold from the triangle inequality instead of a read of the row (assign_prev_threshold_kernel).
    if (ta->prev_k != k) {
      dev_free(ta->prev_cent);
      dev_free(ta->shift);
      ta->prev_cent = nullptr;
      ta->shift = nullptr;
      ta->prev_k = 0;
      VSK_TRY(dev_alloc(ctx, (void**)&ta->prev_cent, (size_t)k * dim * sizeof(float)));
      VSK_TRY(dev_alloc(ctx, (void**)&ta->shift, (size_t)k * sizeof(float)));
      ta->prev_k = k;
      ta->have_prev = false;
    }
    const bool bound_ok = assign_holds_previous && ta->have_prev && ta->bound_allowed && dist != nullptr;
    if (bound_ok) {
      assign_shift_kernel<<<(unsigned)ceil_div(k, 8), 256, 0, ctx->stream>>>(centroids, ta->prev_cent, k, dim, ta->shift);
      ctx->stats.kernel_launches++;
    }
    unsigned sgrid = 0;
    int64_t log_cap = 0;
    // one pass: thresholds (or the coarse arg-min of a first iteration), threshold scan, exact decisions
    auto pass = [&](bool with_bound) -> int32_t {
      VSK_CUDA(ctx, cudaMemsetAsync(sm + 5, 0, 8, ctx->stream));
      if (assign_holds_previous) {
        launch_prev_threshold(ctx, rows, n, dim, centroids, assign, eps, ta->thr, ta->count, with_bound ? dist : nullptr,
                              ta->shift, st + 2 * n, 0.02f);
      } else {
        VSK_CUDA(ctx, cudaMemsetAsync(ta->best, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
        VSK_TRY(launch_assign_scan<SCAN_ARGMIN>(ctx, mr, mc, mrn, mcn, sa));
        assign_threshold_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(ta->best, eps, n, ta->thr, ta->count);
      }
      VSK_CUDA(ctx, cudaMemsetAsync(ta->best, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
      tl_mark(ctx, "assign_thresholds");
      VSK_TRY(launch_assign_scan<SCAN_THRESHOLD>(ctx, mr, mc, mrn, mcn, sa, &sgrid, &log_cap));
      if (dim % 4 == 0 && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)centroids & 15) == 0)
        assign_log_exact_kernel<true><<<dim3(64, sgrid), 256, 0, ctx->stream>>>(rows, dim, centroids, sa.log, sa.log_count, log_cap, ta->best);
      else
        assign_log_exact_kernel<false><<<dim3(64, sgrid), 256, 0, ctx->stream>>>(rows, dim, centroids, sa.log, sa.log_count, log_cap, ta->best);
      tl_mark(ctx, "assign_exact");
      // writes nothing when the scan raised an error: the previous assignment survives for a repeat
      assign_log_decode_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(ta->best, n, assign, dist, ta->bad_rows, (int32_t*)(sm + 6),
                                                                                (const int32_t*)(sm + 5));
      ctx->stats.kernel_launches += 4;
      VSK_CUDA(ctx, cudaGetLastError());
      return VSK_OK;
    };
    VSK_TRY(pass(bound_ok));
    if (bound_ok) {
      // The looser thresholds list more centroids per row; data without gaps between its clusters can fill the hit
      // log.  Then the pass is repeated once with exact thresholds, and the bound is not tried again on this data.
      int32_t e0 = 0;
      VSK_CUDA(ctx, cudaMemcpyAsync(&e0, sm + 5, 4, cudaMemcpyDeviceToHost, ctx->stream));
      VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      if (e0 == 9) {
        ta->bound_allowed = false;
        VSK_TRY(pass(false));
      }
    }
    // remember these centroids for the next call's shifts
    VSK_CUDA(ctx, cudaMemcpyAsync(ta->prev_cent, centroids, (size_t)k * dim * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    ta->have_prev = true;
  } else {

  TcArgs a{};
  a.nq = n;
  a.row_begin = 0;
  a.row_end = k;
  a.kblocks = dim16 / TK;
  a.k16_last = k16_last_of(dim, dim16);
  a.alpha = fsm + 4;
  a.beta = caux;
  a.row_tile_fastest = 1;
  a.err = (int32_t*)(sm + 5);
  a.best = ta->best;
  a.cap = kAssignCap;
  a.cand.keys = ta->keys;
  a.cand.count = ta->count;
  a.cand.thr = ta->thr;
  a.cand.flags = nullptr;
  a.cand.nq = n;
  if (assign_holds_previous) {
    launch_prev_threshold(ctx, rows, n, dim, centroids, assign, eps, ta->thr, ta->count, nullptr, nullptr, nullptr, 0.f);
  } else {
    VSK_CUDA(ctx, cudaMemsetAsync(ta->best, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
    a.mode = SCAN_ARGMIN;
    VSK_TRY(launch_tc<SCAN_ARGMIN>(ctx, mr, mc, a, true));
    assign_threshold_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(ta->best, eps, n, ta->thr, ta->count);
  }
  a.mode = SCAN_THRESHOLD;
  VSK_TRY(launch_tc<SCAN_THRESHOLD>(ctx, mr, mc, a, true));
  assign_exact_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, ctx->stream>>>(rows, n, dim, centroids, ta->keys, ta->count, assign, dist,
                                                                         ta->bad_rows, (int32_t*)(sm + 6), tc_epilogue_warps(a.kblocks) / 4);
  ctx->stats.kernel_launches += 2;
  VSK_CUDA(ctx, cudaGetLastError());
  }
  int32_t h[2] = {0, 0};
  VSK_CUDA(ctx, cudaMemcpyAsync(h, sm + 5, 8, cudaMemcpyDeviceToHost, ctx->stream));
  VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (h[0] == 9) {
    // a CTA's hit log ran full (rows with very many near-ties): the fp32 tile decides for every row
    ctx->stats.fallback_queries += n;
    ExactScanArgs e{};
    e.metric = VSK_METRIC_EUCLIDEAN;
    e.mode = SCAN_ARGMIN;
    e.q = rows;
    e.nq = n;
    e.x = centroids;
    e.dim = dim;
    e.row_begin = 0;
    e.row_end = k;
    e.best = ta->best;
    VSK_CUDA(ctx, cudaMemsetAsync(ta->best, 0xff, (size_t)n * sizeof(unsigned long long), ctx->stream));
    VSK_TRY(launch_exact_scan(ctx, e));
    VSK_CUDA(ctx, cudaMemsetAsync(sm + 6, 0, 4, ctx->stream));
    assign_log_decode_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, ctx->stream>>>(ta->best, n, assign, dist, ta->bad_rows, (int32_t*)(sm + 6),
                                                                              nullptr);
    ctx->stats.kernel_launches++;
    VSK_CUDA(ctx, cudaGetLastError());
    VSK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return VSK_OK;
  }
  if (h[0] != 0) return fail(ctx, VSK_ERR_TIMEOUT, "tensor-core assignment: a bounded pipeline wait ran out (role %d)", h[0]);
  if (h[1] > 0) {
    // rows with too many near-ties (or none listed): the fp32 tile decides
    const int64_t m = h[1];
    ctx->stats.fallback_queries += m;
    VSK_CUDA(ctx, cudaMemsetAsync(ta->best, 0xff, (size_t)m * sizeof(unsigned long long), ctx->stream));
    ExactScanArgs e{};
    e.metric = VSK_METRIC_EUCLIDEAN;
    e.mode = SCAN_ARGMIN;
    e.q = rows;
    e.nq = m;
    e.q_subset = ta->bad_rows;
    e.x = centroids;
    e.dim = dim;
    e.row_begin = 0;
    e.row_end = k;
    e.best = ta->best;
    VSK_TRY(launch_exact_scan(ctx, e));
    scatter_best_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, ctx->stream>>>(ta->best, ta->bad_rows, m, assign, dist);
    ctx->stats.kernel_launches++;
    VSK_CUDA(ctx, cudaGetLastError());
  }
  return VSK_OK;
}

}  // namespace vsk
