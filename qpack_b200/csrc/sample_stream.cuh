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
  for (int probe = 0; probe < slots; ++probe) {
    const int t = tab[h];
    if (t == id) return true;
    if (t == kPenEmpty) return false;
    h = (h + 1) & (uint32_t)(slots - 1);
  }
  return false;
}

// Part 1 (no barrier): clears the table and fetches this thread's first id of the window, so that the global
// load is in flight while other work goes on.  window = [from, hn) of hist.
__device__ __forceinline__ int pen_prefetch(int *tab, int slots, int *unique_ctr, const int *hist, long long from,
                                            long long hn, uint32_t *bloom) {
  for (int i = threadIdx.x; i < slots; i += kThreads) tab[i] = kPenEmpty;
  if (threadIdx.x < kPenBloomBits / 32) bloom[threadIdx.x] = 0u;
  if (threadIdx.x == 0) *unique_ctr = 0;
  return (from + threadIdx.x < hn) ? hist[from + threadIdx.x] : -1;
}
__device__ __forceinline__ int pen_insert(int *tab, int slots, int t, int vocab_total, int *status,
                                          uint32_t *bloom = nullptr) {
  if (t < 0 || t >= vocab_total) return 0;  // out-of-range ids are skipped (sampler.cpp:36)
  if (bloom) { const uint32_t b = pen_bloom_bit(t); atomicOr(&bloom[b >> 5], 1u << (b & 31)); }
  uint32_t h = pen_hash(t, slots);
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
#pragma unroll 4
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
__device__ void finish_row(const StreamArgs &a, int row, const RowParams &p, unsigned long long *cand, int n, int K,
                           const int *pen_tab, int npen, unsigned long long *sorted, float *ev, float *pv,
                           StreamSmem &S, const MtFetch &rng, long long *clk) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // candidate penalty (sampler.cpp:42): positive logits are divided, the others multiplied
  if (npen > 0) {
    const float rp = p.repeat_penalty;
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const unsigned long long c = cand[i];
      const int id = comp_id(c);
      const uint32_t b = pen_bloom_bit(id);
      if (((S.pen_bloom[b >> 5] >> (b & 31)) & 1u) && pen_contains(pen_tab, a.pen_slots, id)) {
        float v = key2f(comp_key(c));
        v = v > 0.f ? __fdiv_rn(v, rp) : __fmul_rn(v, rp);
        cand[i] = make_comp(f2key(v), (uint32_t)id);
      }
    }
    __syncthreads();
  }
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
#pragma unroll 4
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
#pragma unroll 8
  for (int j = 0; j < nK; ++j) sum += (double)ev[j];
  const float minp_thr = __fmul_rn(p.min_p, ev[0]);
  const bool use_minp = p.min_p > 0.f;
  const double top_p = (double)p.top_p;
  int keep = nK;
  double cum = 0.0;
  bool done = false;
  for (int base = 0; base < nK && !done; base += 32) {  // sampler.cpp:48-52
    const int i = base + lane;
    const float e = i < nK ? ev[i] : 0.f;
    const double q = __ddiv_rn((double)e, sum);
    const bool fail = use_minp && i < nK && e < minp_thr;
    const uint32_t failmask = __ballot_sync(0xffffffffu, fail);
    const int cnt = nK - base < 32 ? nK - base : 32;
    for (int j = 0; j < cnt; ++j) {
      if ((failmask >> j) & 1u) { keep = base + j > 1 ? base + j : 1; done = true; break; }
      cum += __shfl_sync(0xffffffffu, q, j);
      if (cum >= top_p) { keep = base + j + 1; done = true; break; }
    }
  }
  double tot = 0.0;
#pragma unroll 8
  for (int j = 0; j < keep; ++j) tot += (double)ev[j];  // sampler.cpp:54
  for (int j = lane; j < keep; j += 32) pv[j] = __double2float_rn(__ddiv_rn((double)ev[j], tot));  // :55
  __syncwarp();
  // draw (sampler.cpp:58-63)
  int pick = 0;
  if (keep > 1 && a.draw) {
    unsigned long long w = 0;
    if (lane == 0) w = mt_commit(rng, a.rng_state + (size_t)row * MT_N, a.rng_drawn + row);
    w = __shfl_sync(0xffffffffu, w, 0);
    double r = word_to_uniform(w);
    pick = keep - 1;
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

// ---- the kernel ----------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kThreads, 4) stream_rows_kernel(const __grid_constant__ StreamArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  StreamSmem &S = *reinterpret_cast<StreamSmem *>(smem_raw);
  int *pen_tab = reinterpret_cast<int *>(smem_raw + sizeof(StreamSmem));

  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();
  const int crank = (int)cluster.block_rank();
  const int slot = blockIdx.x / csize;
  const int row = a.row_list ? a.row_list[slot] : slot;
  const int tid = threadIdx.x, lane = tid & 31;

  // independent global loads first, so that their latencies overlap
  const RowParams p = a.params[a.params_per_row ? row : 0];
  long long hn = (a.history == nullptr) ? 0 : (a.hist_len ? a.hist_len[row] : a.hist_len_all);
  const bool want_rng = MODE != MODE_LOCAL_TOPM && crank == 0 && tid == 0 && a.draw;
  const int Vt = a.vocab_total;
  long long *clk = (a.phase_clk && crank == 0 && tid == 0) ? a.phase_clk + (size_t)row * 16 : nullptr;
  long long select_clk = 0;
  int n_selects = 0;
#define QPB_STAMP(k) do { if (clk) clk[k] = clock64(); } while (0)
  QPB_STAMP(0);
  if (clk) { clk[11] = 0; clk[12] = 0; clk[13] = 0; clk[14] = 0; }

  // this CTA's slice [s0, s1) of the local columns, cut at multiples of 4 floats to keep 16-byte alignment
  int per = (a.vocab + csize - 1) / csize;
  per = (per + 3) & ~3;
  const int s0 = min(a.vocab, crank * per), s1 = min(a.vocab, s0 + per);
  const float *rowp = a.logits + (size_t)row * a.row_stride;
  const int n_tiles = (MODE == MODE_MERGE) ? 0 : (s1 - s0 + kTile - 1) / kTile;
  const bool base_aligned = ((reinterpret_cast<uintptr_t>(rowp + s0) & 15u) == 0);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&S.full[s], 1);
    mbar_fence_init();
    S.cand_count = 0;
  }
  if (tid < 32) S.exp_tab[tid] = kExp2Tab[tid];
  __syncthreads();

  auto tile_len = [&](int t) { return min(kTile, s1 - s0 - t * kTile); };
  auto tile_bulk = [&](int t) { return base_aligned && ((tile_len(t) & 3) == 0); };
  // Ring slots are handed out by a running counter g: slot g uses stage g % kStages on phase (g / kStages) & 1.
  auto issue = [&](int t, int g) {  // thread 0 only: tile t of the slice into ring slot g
    if (t < n_tiles && tile_bulk(t)) {
      const uint32_t bytes = (uint32_t)tile_len(t) * 4u;
      uint64_t *bar = &S.full[g % kStages];
      mbar_expect_tx(bar, bytes);
      bulk_g2s(S.ring[g % kStages], rowp + s0 + (size_t)t * kTile, bytes, bar);
    }
  };
  // Threshold bootstrap (long slices only): the first kStages copies fetch tiles spread over the slice as a
  // sample; a value that a chosen number of sampled columns reach becomes the first threshold, so that the stream
  // itself only picks up about twice the M columns it needs instead of filling the list several times.  It is a
  // guess: if fewer than M columns pass, the slice is streamed again without it.
  const bool can_boot = MODE != MODE_MERGE && base_aligned && n_tiles > 2 * kStages;
  if (tid == 0)
    for (int j = 0; j < kStages; ++j) issue(can_boot ? (int)((long long)j * n_tiles / kStages) : j, j);

  // the three RNG state words this row's draw may need: loaded now, used at the very end
  MtFetch rng = {};
  if (want_rng) rng = mt_fetch(a.rng_state + (size_t)row * MT_N, a.rng_drawn + row);

  // history window (sampler.cpp:32-35): "hn > (size_t)repeat_last_n ? hn - repeat_last_n : 0", so a negative
  // repeat_last_n means the whole history.  The ids are fetched now and inserted after the sample scan.
  const bool use_pen = p.repeat_penalty != 1.f && a.history != nullptr;
  hn = hn < 0 ? 0 : (hn > a.hist_stride ? a.hist_stride : hn);
  long long hfrom = 0;
  if (p.repeat_last_n >= 0 && hn > (long long)p.repeat_last_n) hfrom = hn - p.repeat_last_n;
  const int *hrow = a.history + (size_t)row * a.hist_stride;
  int first_id = -1;
  if (use_pen) first_id = pen_prefetch(pen_tab, a.pen_slots, &S.pen_unique, hrow, hfrom, hn, S.pen_bloom);

  // A column is a candidate unless it is <= thr: while thr is NaN every column is taken; afterwards thr is the
  // weakest kept value, and an equal value at a higher index loses (strict compare, sampler.cpp:16 and
  // kernels_x86.cpp:509).  A NaN logit passes the test and is ordered below -inf by its key later.
  float thr = __int_as_float(0x7fc00000);
  bool failed = false;
  int g0 = 0;  // ring slot of the slice's tile 0
  float m1 = __int_as_float(0xff800000), m2 = m1;  // this thread's two largest sampled values
  if (can_boot) {
    for (int j = 0; j < kStages; ++j) {
      if (!mbar_wait_bounded(&S.full[j], 0u)) failed = true;
#pragma unroll
      for (int h = 0; h < kTile / (kThreads * 4); ++h) {
        const float4 v = *reinterpret_cast<const float4 *>(&S.ring[j][h * kThreads * 4 + tid * 4]);
        const float f4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float x = f4[e];  // NaN is ignored by fmaxf / fminf
          m2 = fmaxf(m2, fminf(m1, x));
          m1 = fmaxf(m1, x);
        }
      }
    }
  }
  __syncthreads();  // the sample has been read by every thread; the penalty table is cleared
  if (can_boot) {   // start the stream proper while the threshold is worked out (tile 0 is fetched again)
    g0 = kStages;
    if (tid == 0)
      for (int j = 0; j < kStages; ++j) issue(j, g0 + j);
  }
  const int npen = use_pen ? pen_build(pen_tab, a.pen_slots, &S.pen_unique, hrow, hfrom, hn, first_id, Vt, a.status, S.pen_bloom) : 0;
  QPB_STAMP(1);
  const bool greedy = p.temperature <= 0.f;
  const int K = greedy ? 1 : (p.top_k > 0 ? min(p.top_k, Vt) : Vt);  // sampler.cpp:39-40
  int M = min(Vt, K + npen);
  if (M >= Vt / 4) M = Vt;  // top_m returns the whole row in this case (sampler.cpp:14)
  const int need = min(M, s1 - s0);  // columns this CTA must deliver
  bool booted = false;
  if (can_boot) {
    // rank of the threshold within the sample: 2.25 x the share of the needed columns expected in the sample
    const long long sample = (long long)kStages * kTile;
    long long r = (9LL * M * sample + 4LL * (s1 - s0) - 1) / (4LL * (s1 - s0));
    r = r < 16 ? 16 : r;
    booted = M < Vt && r <= 128;  // two maxima per thread hold the sample's best 128 well enough
    if (booted) {
      S.cand[2 * tid] = make_comp(f2key(m1), (uint32_t)(2 * tid));
      S.cand[2 * tid + 1] = make_comp(f2key(m2), (uint32_t)(2 * tid + 1));
      __syncthreads();
      const unsigned long long pivot = block_select_pivot(S.cand, 2 * kThreads, (int)r, S.hist, S.sel);
      thr = key2f((uint32_t)(pivot >> 32));  // a lower bound of the r-th largest; key 0 gives NaN = no threshold
      __syncthreads();  // the list is free again
    }
    if (clk) clk[15] = clock64() - clk[1];
  }

  // keep the M best of the list and raise the threshold to the weakest of them; all threads call it
  auto shrink = [&]() {
    const long long c0 = clk ? clock64() : 0;
    block_keep_top(S.cand, min(S.cand_count, kCandCap), M, S.hist, S.sel, &S.cand_count);
    // later columns must beat the weakest kept key: an equal key at a higher index loses.  The select may stop
    // on a key prefix, so take the minimum over the kept entries.
    uint32_t mk = 0xffffffffu;
    for (int i = tid; i < M; i += kThreads) mk = min(mk, comp_key(S.cand[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mk = min(mk, __shfl_xor_sync(0xffffffffu, mk, o));
    if (tid == 0) S.sel[3] = 0xffffffffu;
    __syncthreads();
    if (lane == 0) atomicMin(&S.sel[3], mk);
    __syncthreads();
    thr = key2f(S.sel[3]);  // key 1 (a NaN is among the kept) maps back to NaN: keep taking everything
    if (clk) { select_clk += clock64() - c0; ++n_selects; }
  };

  // ---- streaming phase ----
  // Fast mode scans a whole tile between two barriers and expects a handful of survivors.  Careful mode (no
  // threshold yet, or a tile that overflowed the list in fast mode) scans half a tile at a time and selects
  // whenever another half might not fit, so the list can never overflow whatever the data.
  const uint32_t ring_s = smem_u32(&S.ring[0][0]), full_s = smem_u32(&S.full[0]);
  for (int attempt = 0; attempt < 2; ++attempt) {
    bool careful = false;
    for (int t = 0; t < n_tiles;) {
      const int g = g0 + t;
      const int st = g % kStages;
      const int len = tile_len(t);
      const int tbase = s0 + t * kTile;
      if (!careful && thr == thr && len == kTile && base_aligned) {
        // ---- fast tile: full, bulk-copied, threshold known.  Kept to a minimum of instructions: the scan is
        // issue-latency bound with 8 warps per CTA. ----
        const uint32_t bar = full_s + (uint32_t)st * 8u;
        const uint32_t par = (uint32_t)(g / kStages) & 1u;
        for (int polls = 0; !mbar_try_wait_addr(bar, par);)
          if (++polls > (1 << 22)) { failed = true; break; }
        const int cnt_before = S.cand_count;
        const uint32_t stage_s = ring_s + (uint32_t)st * (kTile * 4u);
        const uint32_t lane_s = stage_s + (uint32_t)tid * 16u;
        uint32_t mask = 0;  // bit 4c + j: column c * 1024 + tid * 4 + j of the tile survives
        mask_not_le<0>(lds_f4(lane_s), thr, mask);
        mask_not_le<4>(lds_f4(lane_s + 4096u), thr, mask);
        mask_not_le<8>(lds_f4(lane_s + 8192u), thr, mask);
        mask_not_le<12>(lds_f4(lane_s + 12288u), thr, mask);
        const uint32_t lanes = __ballot_sync(0xffffffffu, mask != 0u);
        if (lanes != 0u) {
          // Same-address shared-memory atomics serialise and a warp scan is not free either: a warp with few
          // survivors lets each of those lanes reserve its own slots, a warp with many reserves once for all of
          // them.  Survivors are re-read from the stage by position so that only they cost instructions.
          const int nacc = __popc(mask);
          int pos;
          if (__popc(lanes) <= 6) {
            pos = nacc ? smem_atomic_add(&S.cand_count, nacc) : 0;
          } else {
            int incl = nacc;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const int v = __shfl_up_sync(0xffffffffu, incl, o);
              if (lane >= o) incl += v;
            }
            int wbase = 0;
            if (lane == 31) wbase = smem_atomic_add(&S.cand_count, incl);
            pos = __shfl_sync(0xffffffffu, wbase, 31) + incl - nacc;
          }
          while (mask) {
            const int e = __ffs(mask) - 1;
            mask &= mask - 1u;
            const int off = (e >> 2) * (kThreads * 4) + tid * 4 + (e & 3);
            if (pos < kCandCap)
              smem_store_u64(&S.cand[pos], make_comp(f2key(lds_f32(stage_s + (uint32_t)off * 4u)), (uint32_t)(a.id_offset + tbase + off)));
            ++pos;
          }
        }
        __syncthreads();  // stage consumed by every thread; candidate count settled
        const int cnt = S.cand_count;
        if (cnt > kCandCap) {
          // more survivors than the list holds: forget this tile's, scan it again half by half
          __syncthreads();
          if (tid == 0) S.cand_count = cnt_before;
          careful = true;
          if (cnt_before > kCandHigh && cnt_before > M) { __syncthreads(); shrink(); }
          __syncthreads();
          continue;
        }
        if (tid == 0) issue(t + kStages, g + kStages);
        if (cnt > kCandHighFast && cnt > M) shrink();
        ++t;
        continue;
      }
      if (tile_bulk(t)) {
        if (!mbar_wait_bounded(&S.full[st], (uint32_t)(g / kStages) & 1u)) failed = true;
      } else {  // unaligned row or ragged tail: plain loads into the same stage
        for (int i = tid; i < len; i += kThreads) S.ring[st][i] = rowp[tbase + i];
        __syncthreads();
      }
      const int cnt_before = S.cand_count;  // settled: the previous tile ended with a barrier
      const bool slow = careful || thr != thr;
      for (int q = 0; q < kTile / kChunk; ++q) {
        const int qlen = min(kChunk, len - q * kChunk);  // columns of this chunk (uniform)
        if (qlen <= 0) break;
        const float *src = &S.ring[st][q * kChunk];
        const float4 v = smem_load_f4(src + tid * 4);
        const float f[4] = {v.x, v.y, v.z, v.w};
        const int qbase = a.id_offset + tbase + q * kChunk;  // global id of the chunk's first column
        if (thr != thr) {
          // no threshold yet: the whole chunk is taken, every column has its own slot, no atomics
          const int cbase = S.cand_count;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int off = tid * 4 + e;
            if (off < qlen && cbase + off < kCandCap) S.cand[cbase + off] = make_comp(f2key(f[e]), (uint32_t)(qbase + off));
          }
          __syncthreads();
          if (tid == 0) S.cand_count = cbase + qlen;
        } else {
          // one predicate per column; the bits of a ragged last chunk are masked by position
          uint32_t accmask = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) accmask |= !(f[e] <= thr) ? (1u << e) : 0u;
          if (qlen != kChunk) accmask &= (1u << min(4, max(0, qlen - tid * 4))) - 1u;
          const uint32_t lanes = __ballot_sync(0xffffffffu, accmask != 0u);
          if (lanes != 0u) {  // same slot reservation as on the fast path
            const int nacc = __popc(accmask);
            int pos;
            if (__popc(lanes) <= 6) {
              pos = nacc ? smem_atomic_add(&S.cand_count, nacc) : 0;
            } else {
              int incl = nacc;
#pragma unroll
              for (int o = 1; o < 32; o <<= 1) {
                const int t2 = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t2;
              }
              int wbase = 0;
              if (lane == 31) wbase = smem_atomic_add(&S.cand_count, incl);
              pos = __shfl_sync(0xffffffffu, wbase, 31) + incl - nacc;
            }
            while (accmask) {
              const int e = __ffs(accmask) - 1;
              accmask &= accmask - 1u;
              const int off = tid * 4 + e;
              if (pos < kCandCap) smem_store_u64(&S.cand[pos], make_comp(f2key(src[off]), (uint32_t)(qbase + off)));
              ++pos;
            }
          }
        }
        if (slow) {
          __syncthreads();
          const int c = S.cand_count;
          if (c > kCandCap && tid == 0) atomicOr(a.status, ST_CAPACITY);  // cannot happen: c <= kCandHigh + kChunk
          if (c > kCandHigh && c > M) shrink();
        }
      }
      __syncthreads();  // stage consumed by every thread; candidate count settled
      const int cnt = S.cand_count;
      if (!slow && cnt > kCandCap) {
        // more survivors than the list holds: forget this tile's, scan it again chunk by chunk
        __syncthreads();
        if (tid == 0) S.cand_count = cnt_before;
        careful = true;
        if (cnt_before > kCandHigh && cnt_before > M) { __syncthreads(); shrink(); }
        __syncthreads();
        continue;
      }
      if (tid == 0) issue(t + kStages, g + kStages);
      if (!slow && cnt > kCandHighFast && cnt > M) shrink();
      ++t;
    }
    // every column above the bootstrap threshold was collected; with at least `need` of them the needed ones
    // are all in the list.  Otherwise the guess was too high: stream the slice once more from "no threshold".
    if (!booted || S.cand_count >= need) break;
    __syncthreads();
    booted = false;
    thr = __int_as_float(0x7fc00000);
    g0 += n_tiles;
    if (tid == 0) {
      S.cand_count = 0;
      for (int j = 0; j < kStages; ++j) issue(j, g0 + j);
    }
    if (clk) clk[14] += 1;
    __syncthreads();
  }
  QPB_STAMP(2);
  if (clk) { clk[8] = select_clk; clk[9] = n_selects; clk[10] = S.cand_count; }
  if (failed && tid == 0) atomicOr(a.status, ST_COPY_TIMEOUT);

  // MODE_MERGE: candidates come from the gathered per-shard lists instead of a stream
  if (MODE == MODE_MERGE) {
    const int total = a.n_shards * a.cand_slots;
    for (int i0 = 0; i0 < total; i0 += kThreads) {  // uniform trip count: every lane votes
      const int i = i0 + tid;
      unsigned long long c = 0ULL;
      if (i < total) {
        const int sh = i / a.cand_slots, s = i - sh * a.cand_slots;
        c = a.cand_io[((size_t)sh * a.cand_rows + row) * a.cand_slots + s];
      }
      const uint32_t m = __ballot_sync(0xffffffffu, c != 0ULL);
      int wbase = 0;
      if (lane == 0 && m) wbase = atomicAdd(&S.cand_count, __popc(m));
      wbase = __shfl_sync(0xffffffffu, wbase, 0);
      const int pos = wbase + __popc(m & ((1u << lane) - 1u));
      if (c != 0ULL && pos < kMergeCap) S.cand[pos] = c;
    }
    __syncthreads();
    if (S.cand_count > kMergeCap && tid == 0) atomicOr(a.status, ST_CAPACITY);
  }

  int n = min(S.cand_count, MODE == MODE_MERGE ? kMergeCap : kCandCap);
  // The reference penalises exactly its M largest raw entries.  When the penalty only lowers values
  // (repeat_penalty >= 1) the K best after the penalty are the same over any superset of those M, so the exact
  // raw cut can be skipped; a penalty below 1 raises values and needs it.  Lists that travel (cluster merge,
  // all-gather) are always cut to M to bound their size.
  const bool exact_m = (npen > 0 && !(p.repeat_penalty >= 1.f)) || csize > 1 || MODE != MODE_SAMPLE;
  if (exact_m) n = block_keep_top(S.cand, n, M, S.hist, S.sel, &S.cand_count);
  QPB_STAMP(3);

  // ---- cluster merge: every CTA pushes its winners into the leader's list over DSMEM ----
  if (csize > 1) {
    cluster.sync();  // the leader's ring is idle and its own list is final
    if (crank != 0) {
      StreamSmem *L = cluster.map_shared_rank(&S, 0);
      if (tid == 0) S.misc[0] = atomicAdd(&L->cand_count, n);
      __syncthreads();
      const int base = S.misc[0];
      for (int i = tid; i < n; i += kThreads)
        if (base + i < kMergeCap) L->cand[base + i] = S.cand[i];
      if (base + n > kMergeCap && tid == 0) atomicOr(a.status, ST_CAPACITY);
    }
    cluster.sync();
    if (crank != 0) return;
    n = min(S.cand_count, kMergeCap);
    n = block_keep_top(S.cand, n, M, S.hist, S.sel, &S.cand_count);
  }
  QPB_STAMP(4);

  if (MODE == MODE_LOCAL_TOPM) {  // hand this GPU's winners to the all-gather
    unsigned long long *out = a.cand_io + (size_t)row * a.cand_slots;
    for (int i = tid; i < a.cand_slots; i += kThreads) out[i] = i < n ? S.cand[i] : 0ULL;
    if (n > a.cand_slots && tid == 0) atomicOr(a.status, ST_CAPACITY);
    return;
  }

  unsigned long long *sorted = reinterpret_cast<unsigned long long *>(&S.ring[0][0]);
  float *ev = reinterpret_cast<float *>(&S.cand[0]);
  float *pv = ev + kCandCap;
  finish_row(a, row, p, S.cand, n, K, pen_tab, npen, sorted, ev, pv, S, rng, clk);
  QPB_STAMP(7);
#undef QPB_STAMP
}

}  // namespace qpb
