// The streaming sampler kernel: one thread-block cluster (1, 2, 4 or 8 CTAs) per logit row.
//
// Reference behaviour reproduced (qpack src/sampler.cpp): penalty set over the history window (32-38), the exact
// M = K + |penalty set| largest raw logits under (value desc, index asc) (top_m, 12-27, with the scan of
// kernels_x86.cpp:505-513), candidate penalty, ordering and truncation to K (42-44), greedy exit (45), softmax
// numerators with the C library's expf and ordered double sums (46-47), min-p / top-p cut (48-53),
// renormalisation (54-55) and the seeded inverse-CDF draw (58-63).
//
// How it maps to the B200: every f32 logit is read from HBM exactly once.  Each CTA streams its contiguous
// slice of the row through a ring of shared-memory stages filled by bulk-async copies (cp.async.bulk +
// mbarrier, no multicast), compares each float against a running threshold (one predicate per element) and
// appends the few survivors to a shared-memory candidate list; when the list fills, a radix select over the
// 64-bit (key, ~index) composites keeps the best M and raises the threshold.  With more than one CTA per row
// the per-CTA winners are pushed into the leader CTA's shared memory over DSMEM and selected once more.  The
// leader then finishes the row on at most a few hundred candidates: penalty, top-K select, rank sort, softmax,
// cut, draw.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace qpb {
namespace cg = cooperative_groups;

constexpr int kThreads = 256;                // threads per CTA
constexpr int kTile = 4096;                  // floats per ring stage (16 KB)
constexpr int kStages = 2;                   // ring depth: 32 KB in flight per CTA, 4 CTAs per SM
constexpr int kChunk = kThreads * 4;         // careful mode scans a tile in chunks of one float4 per thread
constexpr int kCandCap = 2048;               // candidate entries of the streaming phase (16 KB)
constexpr int kCandHigh = kCandCap - kChunk; // careful mode: select when the list grows beyond this (a chunk adds <= kChunk)
constexpr int kCandHighFast = 1280;          // fast mode: select after a tile that left more than this
constexpr int kRingEntries = kStages * kTile * 4 / 8;
constexpr int kMergeCap = kCandCap + kRingEntries;  // entries available to the cluster merge (ring reused)
// Rows with top_k + window above this take the whole-row kernel instead.  It also bounds the "whole row" case of
// top_m (M >= V/4 implies V <= 4 * 500 + 3 = 2003 <= kCandCap).
constexpr int kSmallMaxM = 500;
constexpr int kPenBloomBits = 4096;          // one-probe negative test in front of the penalty hash table
constexpr int kPenEmpty = -1;
static_assert(kSmallMaxM <= kCandHigh && 4 * kSmallMaxM + 3 <= kCandCap, "candidate list sizing");
static_assert(8 * kSmallMaxM <= kMergeCap, "cluster merge sizing");
static_assert(kTile % kChunk == 0, "chunking");

enum : int { MODE_SAMPLE = 0, MODE_LOCAL_TOPM = 1, MODE_MERGE = 2 };

struct StreamArgs {
  const float *logits;     // [n_rows][row_stride] this GPU's columns of every row
  long long row_stride;    // elements
  int vocab;               // columns held here
  int vocab_total;         // full vocabulary (== vocab unless vocab-sharded)
  int id_offset;           // global id of local column 0
  int n_rows;              // rows in this launch
  const int *row_list;     // row indices to process, or nullptr for 0..n_rows-1
  const RowParams *params; // [1] or [rows]
  int params_per_row;      // 0: params[0] for every row
  const int *history;      // [rows][hist_stride] or nullptr
  long long hist_stride;
  const int *hist_len;     // [rows] visible history length, or nullptr = hist_len_all
  int hist_len_all;
  unsigned long long *rng_state;  // [rows][312]
  unsigned int *rng_drawn;        // [rows]
  int *out_ids;            // [rows] (may be nullptr when draw == 0)
  int draw;                // 1: make the draw (takes a random word unless one entry survives); 0: distribution only
  int *dist_ids;           // optional [rows][max_out]
  float *dist_p;           // optional [rows][max_out]
  int *dist_count;         // optional [rows]
  int max_out;
  unsigned long long *cand_io;  // MODE_LOCAL_TOPM: out [rows][cand_slots]; MODE_MERGE: in [n_shards][rows][cand_slots]
  int cand_slots;
  int n_shards;
  int cand_rows;           // row dimension of cand_io
  int pen_slots;           // penalty hash slots (power of two)
  // Row pieces (one CTA per cluster only).  units_per_cta > 0: the rows of this launch, cut into tiles of kTile
  // columns and laid end to end, are dealt out in equal runs of units_per_cta tiles to the CTAs of the grid; a row
  // that straddles CTAs is sampled in pieces, each piece leaves its best candidates in piece_cand, and the CTA
  // that delivers the last piece of a row merges them and finishes the row.
  int units_per_cta;
  int tiles_per_row;
  int max_pieces;                   // pieces a row can have
  unsigned long long *piece_cand;   // [rows][max_pieces][kSmallMaxM]
  int *piece_cnt;                   // [rows][max_pieces]
  int *piece_done;                  // [rows], zero between launches (the finishing CTA resets it)
  int *status;
  long long *phase_clk;    // optional [rows][16]: SM clock stamps of the leader CTA's phases (latency breakdown)
};

struct __align__(16) StreamSmem {
  unsigned long long cand[kCandCap];  // candidates; the ring follows directly so that the merge can use both
  float ring[kStages][kTile];
  uint64_t full[kStages];
  unsigned long long exp_tab[32];
  uint32_t hist[256];
  uint32_t pen_bloom[kPenBloomBits / 32];
  uint32_t sel[4];
  int cand_count;
  int pen_unique;
  int misc[2];
  // followed by the penalty hash table: pen_slots ints
};

// ---- penalty set: open-addressing hash set of the distinct in-range ids of the window (sampler.cpp:32-38) ------
__device__ __forceinline__ uint32_t pen_hash(int id, int slots) { return ((uint32_t)id * 2654435761u) & (uint32_t)(slots - 1); }

__device__ __forceinline__ uint32_t pen_bloom_bit(int id) { return ((uint32_t)id * 0x9E3779B1u) >> (32 - 12); }
static_assert(kPenBloomBits == 1 << 12, "pen_bloom_bit takes 12 hash bits");

__device__ __forceinline__ bool pen_contains(const int *tab, int slots, int id) {
  uint32_t h = pen_hash(id, slots);
#pragma unroll 1
  for (int probe = 0; probe < slots; ++probe) {
    const int t = tab[h];
    if (t == id) return true;
    if (t == kPenEmpty) return false;
    h = (h + 1) & (uint32_t)(slots - 1);
  }
  return false;
}

// Part 1 (no barrier): clears the table, the filter and the counter.  The caller fetches each thread's first id
// of the window early, so that the global load is in flight while other work goes on.
__device__ __forceinline__ void pen_clear(int *tab, int slots, int *unique_ctr, uint32_t *bloom) {
  for (int i = threadIdx.x; i < slots; i += kThreads) tab[i] = kPenEmpty;
  if (threadIdx.x < kPenBloomBits / 32) bloom[threadIdx.x] = 0u;
  if (threadIdx.x == 0) *unique_ctr = 0;
}
__device__ __forceinline__ int pen_insert(int *tab, int slots, int t, int vocab_total, int *status,
                                          uint32_t *bloom = nullptr) {
  if (t < 0 || t >= vocab_total) return 0;  // out-of-range ids are skipped (sampler.cpp:36)
  if (bloom) { const uint32_t b = pen_bloom_bit(t); atomicOr(&bloom[b >> 5], 1u << (b & 31)); }
  uint32_t h = pen_hash(t, slots);
#pragma unroll 1
  for (int probe = 0; probe < slots; ++probe) {
    const int old = atomicCAS(&tab[h], kPenEmpty, t);
    if (old == kPenEmpty) return 1;
    if (old == t) return 0;
    h = (h + 1) & (uint32_t)(slots - 1);
  }
  atomicOr(status, ST_PEN_TABLE_FULL);
  return 0;
}
// Part 2 (a barrier must separate it from part 1): inserts the window, returns the number of distinct ids.
__device__ int pen_build(int *tab, int slots, int *unique_ctr, const int *hist, long long from, long long hn,
                         int first_id, int vocab_total, int *status, uint32_t *bloom) {
  int mine = pen_insert(tab, slots, first_id, vocab_total, status, bloom);
  for (long long i = from + kThreads + threadIdx.x; i < hn; i += kThreads)
    mine += pen_insert(tab, slots, hist[i], vocab_total, status, bloom);
  if (mine) atomicAdd(unique_ctr, mine);
  __syncthreads();
  return *unique_ctr;
}

// (The block-wide helpers below are called from many places and kept out of line: the cold phases of the kernel are
// limited by instruction fetch, so code size matters more than call overhead.)
// ---- radix select over composites ------------------------------------------------------------------------
// Returns a pivot such that exactly `want` of c[0..n) are >= pivot (composites are distinct).  0 < want < n.
// 8-bit digits from the top; stops as soon as the chosen bucket is taken whole.  All threads call it.
__device__ unsigned long long block_select_pivot(const unsigned long long *c, int n, int want, uint32_t *hist,
                                                 uint32_t *sel) {
  unsigned long long prefix = 0, mask = 0;
  uint32_t need = (uint32_t)want;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  hist[threadIdx.x] = 0;  // kThreads == 256
  __syncthreads();
  for (int shift = 56; shift >= 0; shift -= 8) {
#pragma unroll 1
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const unsigned long long v = c[i];
      if ((v & mask) == prefix) atomicAdd(&hist[(uint32_t)(v >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (warp == 0) {  // lane l owns bins 8l .. 8l+7: reads them, clears them for the next pass
      uint32_t loc[8], s = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) { loc[k] = hist[8 * lane + k]; s += loc[k]; hist[8 * lane + k] = 0; }
      uint32_t suf = s;  // inclusive suffix sum over lanes >= lane
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += t;
      }
      const uint32_t above = suf - s;
      if (above < need && need <= suf) {
        uint32_t acc = above;
#pragma unroll
        for (int k = 7; k >= 0; --k) {
          if (acc + loc[k] >= need) { sel[0] = 8 * lane + k; sel[1] = need - acc; sel[2] = loc[k]; break; }
          acc += loc[k];
        }
      }
    }
    __syncthreads();
    const uint32_t d = sel[0], bucket = sel[2];
    need = sel[1];
    prefix |= (unsigned long long)d << shift;
    mask |= 0xffULL << shift;
    if (need == bucket) break;
  }
  return prefix;
}

// In-place compaction: keeps the entries >= pivot at the front (order not preserved).  Returns the new count.
__device__ int block_compact(unsigned long long *c, int n, unsigned long long pivot, int *counter) {
  constexpr int PER = 4;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) *counter = 0;
  __syncthreads();
#pragma unroll 1
  for (int base = 0; base < n; base += PER * kThreads) {
    unsigned long long r[PER];
    int mine = 0;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = base + k * kThreads + threadIdx.x;
      r[k] = (i < n) ? c[i] : 0ULL;
      if (r[k] < pivot) r[k] = 0ULL;  // composites are never 0
      mine += r[k] != 0ULL;
    }
    int incl = mine;  // warp scan of the per-lane keep counts, then one reservation per warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    __syncthreads();  // every entry of this chunk is in registers before any slot below its end is rewritten
    int pos = 0;
    if (lane == 31 && total > 0) pos = atomicAdd(counter, total);
    pos = __shfl_sync(0xffffffffu, pos, 31) + incl - mine;
#pragma unroll
    for (int k = 0; k < PER; ++k)
      if (r[k] != 0ULL) c[pos++] = r[k];
  }
  __syncthreads();
  return *counter;
}

// keep the `want` largest of c[0..n) at the front (no-op when n <= want); returns the new count
__device__ __forceinline__ int block_keep_top(unsigned long long *c, int n, int want, uint32_t *hist, uint32_t *sel,
                                              int *counter) {
  if (n <= want) return n;
  const unsigned long long pivot = block_select_pivot(c, n, want, hist, sel);
  return block_compact(c, n, pivot, counter);
}

// ---- the finish: penalty, order, softmax, cut, draw (leader CTA) ----------------------------------------------
// cand[0..n): a superset of the candidates the reference would hold, unordered (exactly its M largest raw
// entries when the caller had to cut to M).  `sorted` (kCandCap composites) must not overlap cand; ev / pv
// (kCandCap floats each) may alias cand, which is dead once `sorted` is written.
// candidate penalty (sampler.cpp:42): positive logits are divided, the others multiplied.  All threads call it.
__device__ __forceinline__ void penalise_candidates(unsigned long long *cand, int n, const int *pen_tab, int pen_slots,
                                                    const uint32_t *bloom, float rp) {
#pragma unroll 1
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const unsigned long long c = cand[i];
    const int id = comp_id(c);
    const uint32_t b = pen_bloom_bit(id);
    if (((bloom[b >> 5] >> (b & 31)) & 1u) && pen_contains(pen_tab, pen_slots, id)) {
      float v = key2f(comp_key(c));
      v = v > 0.f ? __fdiv_rn(v, rp) : __fmul_rn(v, rp);
      cand[i] = make_comp(f2key(v), (uint32_t)id);
    }
  }
  __syncthreads();
}

__device__ void finish_row(const StreamArgs &a, int row, const RowParams &p, unsigned long long *cand, int n, int K,
                           const int *pen_tab, int npen, unsigned long long *sorted, float *ev, float *pv,
                           StreamSmem &S, long long *clk, bool penalised = false) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the RNG words of a possible draw: requested now, used after the ordering and the softmax
  MtFetch rng = {};
  if (threadIdx.x == 0 && a.draw && p.temperature > 0.f) rng = mt_fetch(a.rng_state + (size_t)row * MT_N, a.rng_drawn + row);
  if (npen > 0 && !penalised) penalise_candidates(cand, n, pen_tab, a.pen_slots, S.pen_bloom, p.repeat_penalty);
  if (clk) clk[11] = clock64();
  // the K best by (value desc, id asc) (sampler.cpp:43-44): select, then rank = number of larger composites
  n = block_keep_top(cand, n, K, S.hist, S.sel, &S.cand_count);
  if (clk) clk[12] = clock64();
  const int nK = n;
  {
    // P lanes share one entry (P = 32, 16, 8, 4, 2 or 1, as many as the CTA can spare), each counting over a
    // strided part of the list; partial ranks are summed with shuffles
    int P = 32;
    while (P > 1 && nK * P > kThreads) P >>= 1;
    const int sub = threadIdx.x & (P - 1);
    for (int i0 = 0; i0 < nK; i0 += kThreads / P) {
      const int i = i0 + threadIdx.x / P;
      const unsigned long long c = i < nK ? cand[i] : 0ULL;
      int rank = 0;
#pragma unroll 2
      for (int j = sub; j < nK; j += P) rank += (cand[j] > c) ? 1 : 0;
      for (int o = P >> 1; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
      if (i < nK && sub == 0) sorted[rank] = c;
    }
  }
  __syncthreads();
  if (clk) clk[5] = clock64();

  const bool greedy = p.temperature <= 0.f;
  if (greedy) {  // sampler.cpp:45; draw() of a one-entry distribution takes no random word (sampler.cpp:59)
    if (threadIdx.x == 0) {
      const int id = comp_id(sorted[0]);
      if (a.out_ids) a.out_ids[row] = id;
      if (a.dist_count) a.dist_count[row] = 1;
      if (a.dist_ids && a.max_out > 0) { a.dist_ids[(size_t)row * a.max_out] = id; a.dist_p[(size_t)row * a.max_out] = 1.f; }
    }
    return;
  }
  // softmax numerators (sampler.cpp:46-47): float subtract, float divide, the library's expf
  const float mx = key2f(comp_key(sorted[0]));
  for (int i = threadIdx.x; i < nK; i += kThreads) {
    const float v = key2f(comp_key(sorted[i]));
    ev[i] = expf_libm(__fdiv_rn(__fsub_rn(v, mx), p.temperature), S.exp_tab);
  }
  __syncthreads();
  if (clk) clk[6] = clock64();
  if (warp != 0) return;

  // Ordered double arithmetic, replayed exactly: every lane of warp 0 carries the same running values.
  double sum = 0.0;
#pragma unroll 4
  for (int j = 0; j < nK; ++j) sum += (double)ev[j];
  if (clk) clk[13] = clock64();
  const float minp_thr = __fmul_rn(p.min_p, ev[0]);
  const bool use_minp = p.min_p > 0.f;
  const double top_p = (double)p.top_p;
  int keep = nK;
  double cum = 0.0;
  bool done = false;
  double *qs = reinterpret_cast<double *>(S.hist);  // 32 quotients of the current chunk (the histogram is idle)
  for (int base = 0; base < nK && !done; base += 32) {  // sampler.cpp:48-52, 32 positions at a time
    const int i = base + lane;
    const float e = i < nK ? ev[i] : 0.f;
    qs[lane] = __ddiv_rn((double)e, sum);
    const bool fail = use_minp && i < nK && e < minp_thr;
    const uint32_t failmask = __ballot_sync(0xffffffffu, fail);
    const int cnt = nK - base < 32 ? nK - base : 32;
    __syncwarp();
    // the running sum is a dependent chain of double adds; without branches inside, its loads and compares overlap
    int first_top = 32;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const double next = cum + qs[j];
      const bool valid = j < cnt;
      cum = valid ? next : cum;
      first_top = (valid && first_top == 32 && next >= top_p) ? j : first_top;
    }
    const int first_fail = failmask ? __ffs(failmask) - 1 : 32;
    // position i: the min-p test comes first, then the sum test (sampler.cpp:50-51)
    if (first_fail <= first_top && first_fail < 32) { keep = base + first_fail > 1 ? base + first_fail : 1; done = true; }
    else if (first_top < 32) { keep = base + first_top + 1; done = true; }
    __syncwarp();
  }
  if (clk) clk[15] = clock64();
  double tot = 0.0;
#pragma unroll 4
  for (int j = 0; j < keep; ++j) tot += (double)ev[j];  // sampler.cpp:54
  for (int j = lane; j < keep; j += 32) pv[j] = __double2float_rn(__ddiv_rn((double)ev[j], tot));  // :55
  __syncwarp();
  if (clk) clk[3] = clock64();
  // draw (sampler.cpp:58-63)
  int pick = 0;
  if (keep > 1 && a.draw) {
    unsigned long long w = 0;
    if (lane == 0) w = mt_commit(rng, a.rng_state + (size_t)row * MT_N, a.rng_drawn + row);
    w = __shfl_sync(0xffffffffu, w, 0);
    double r = word_to_uniform(w);
    pick = keep - 1;
#pragma unroll 1
    for (int j = 0; j < keep; ++j) {
      r -= (double)pv[j];
      if (r <= 0.0) { pick = j; break; }
    }
  }
  if (lane == 0) {
    if (a.draw && a.out_ids) a.out_ids[row] = comp_id(sorted[pick]);
    if (a.dist_count) a.dist_count[row] = keep;
  }
  if (a.dist_ids) {
    const int m = keep < a.max_out ? keep : a.max_out;
    for (int j = lane; j < m; j += 32) {
      a.dist_ids[(size_t)row * a.max_out + j] = comp_id(sorted[j]);
      a.dist_p[(size_t)row * a.max_out + j] = pv[j];
    }
  }
}

}  // namespace qpb
