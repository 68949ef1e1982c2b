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
// mbarrier, no multicast), compares order-preserving keys against a running threshold and appends the few
// survivors to a shared-memory candidate list; when the list fills, a radix select over the 64-bit
// (key, ~index) composites keeps the best M and raises the threshold.  With more than one CTA per row the
// per-CTA winners are pushed into the leader CTA's shared memory over DSMEM and selected once more.  The leader
// then finishes the row on at most a few hundred candidates: penalty, rank sort, softmax, cut, draw.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace qpb {
namespace cg = cooperative_groups;

constexpr int kThreads = 256;        // threads per CTA
constexpr int kTile = 2048;          // floats per ring stage (8 KB)
constexpr int kStages = 4;           // ring depth: 32 KB in flight per CTA
constexpr int kCandCap = 4096;       // candidate entries of the streaming phase (32 KB)
constexpr int kCandHigh = kCandCap - kTile;  // select when the list grows beyond this
constexpr int kMergeCap = kCandCap + kStages * kTile * 4 / 8;  // entries available to the cluster merge (ring reused)
constexpr int kSmallMaxM = 768;      // rows with top_k + window above this take the whole-row kernel instead
constexpr int kPenEmpty = -1;

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
};

struct __align__(16) StreamSmem {
  unsigned long long cand[kCandCap];        // candidates; the ring follows directly so that the merge can use both
  float ring[kStages][kTile];
  uint64_t full[kStages];
  uint32_t hist[256];
  uint32_t sel[4];
  int cand_count;
  int pen_unique;
  int misc[2];
  // followed by the penalty hash table: pen_slots ints
};

// ---- penalty set: open-addressing hash set of the distinct in-range ids of the window (sampler.cpp:32-38) ------
__device__ __forceinline__ uint32_t pen_hash(int id, int slots) { return ((uint32_t)id * 2654435761u) & (uint32_t)(slots - 1); }

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

// returns the number of distinct ids; all threads of the CTA call it
__device__ int build_pen_set(int *tab, int slots, int *unique_ctr, const int *hist, long long hn, int last_n,
                             int vocab_total, int *status) {
  for (int i = threadIdx.x; i < slots; i += kThreads) tab[i] = kPenEmpty;
  if (threadIdx.x == 0) *unique_ctr = 0;
  __syncthreads();
  // "hn > (size_t)repeat_last_n ? hn - repeat_last_n : 0": a negative repeat_last_n means the whole history
  long long from = 0;
  if (last_n >= 0 && hn > (long long)last_n) from = hn - last_n;
  int mine = 0;
  for (long long i = from + threadIdx.x; i < hn; i += kThreads) {
    const int t = hist[i];
    if (t < 0 || t >= vocab_total) continue;
    uint32_t h = pen_hash(t, slots);
    int probe = 0;
    for (; probe < slots; ++probe) {
      const int old = atomicCAS(&tab[h], kPenEmpty, t);
      if (old == kPenEmpty) { ++mine; break; }
      if (old == t) break;
      h = (h + 1) & (uint32_t)(slots - 1);
    }
    if (probe == slots) atomicOr(status, ST_PEN_TABLE_FULL);
  }
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
  for (int shift = 56; shift >= 0; shift -= 8) {
    hist[threadIdx.x] = 0;  // kThreads == 256
    __syncthreads();
    for (int base = 0; base < n; base += kThreads) {  // uniform trip count: every lane takes part in the votes
      const int i = base + threadIdx.x;
      const unsigned long long v = i < n ? c[i] : 0ULL;
      const bool in = i < n && (v & mask) == prefix;
      // warp-aggregated histogram: lanes with the same digit elect one to add their count (tie-heavy rows
      // would otherwise serialise on one shared-memory word)
      const uint32_t digit = (uint32_t)(v >> shift) & 255u;
      const uint32_t active = __ballot_sync(0xffffffffu, in);
      if (in) {
        const uint32_t peers = __match_any_sync(active, digit);
        if ((peers & ((1u << lane) - 1u)) == 0) atomicAdd(&hist[digit], __popc(peers));
      }
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t loc[8], s = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) { loc[k] = hist[8 * lane + k]; s += loc[k]; }
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
  __syncthreads();
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
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = base + k * kThreads + threadIdx.x;
      r[k] = (i < n) ? c[i] : 0ULL;
    }
    __syncthreads();  // every entry of this chunk is in registers before any slot below its end is rewritten
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const bool keep = r[k] >= pivot && r[k] != 0ULL;
      const uint32_t m = __ballot_sync(0xffffffffu, keep);
      if (m) {
        int basepos = 0;
        if (lane == __ffs(m) - 1) basepos = atomicAdd(counter, __popc(m));
        basepos = __shfl_sync(0xffffffffu, basepos, __ffs(m) - 1);
        if (keep) c[basepos + __popc(m & ((1u << lane) - 1u))] = r[k];
      }
    }
  }
  __syncthreads();
  return *counter;
}

// ---- the finish: penalty, order, softmax, cut, draw on n <= 4096 candidates (leader CTA) ------------------------
// cand[0..n): exact M largest raw (key, id) composites, unordered.  `sorted` and `ev`/`pv` are shared-memory
// areas that do not overlap cand[0..n) resp. each other: sorted: 4096 composites; ev, pv: 4096 floats each.
__device__ void finish_row(const StreamArgs &a, int row, const RowParams &p, unsigned long long *cand, int n, int K,
                           const int *pen_tab, int npen, unsigned long long *sorted, float *ev, float *pv) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // candidate penalty (sampler.cpp:42): positive logits are divided, the others multiplied
  if (npen > 0) {
    const float rp = p.repeat_penalty;
    for (int i = threadIdx.x; i < n; i += kThreads) {
      const unsigned long long c = cand[i];
      const int id = comp_id(c);
      if (pen_contains(pen_tab, a.pen_slots, id)) {
        float v = key2f(comp_key(c));
        v = v > 0.f ? __fdiv_rn(v, rp) : __fmul_rn(v, rp);
        cand[i] = make_comp(f2key(v), (uint32_t)id);
      }
    }
    __syncthreads();
  }
  // order by (value desc, id asc) and keep the first K (sampler.cpp:43-44): rank = number of larger composites
  const int nK = n < K ? n : K;
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const unsigned long long c = cand[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += (cand[j] > c) ? 1 : 0;
    if (rank < nK) sorted[rank] = c;
  }
  __syncthreads();

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
    ev[i] = expf_libm(__fdiv_rn(__fsub_rn(v, mx), p.temperature));
  }
  __syncthreads();
  if (warp != 0) return;

  // Ordered double arithmetic, replayed exactly: every lane of warp 0 carries the same running values.
  double sum = 0.0;
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
  for (int j = 0; j < keep; ++j) tot += (double)ev[j];  // sampler.cpp:54
  for (int j = lane; j < keep; j += 32) pv[j] = __double2float_rn(__ddiv_rn((double)ev[j], tot));  // :55
  __syncwarp();
  // draw (sampler.cpp:58-63)
  int pick = 0;
  if (keep > 1 && a.draw) {
    unsigned long long w = 0;
    if (lane == 0) w = mt_next(a.rng_state + (size_t)row * MT_N, a.rng_drawn + row);
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
__global__ void __launch_bounds__(kThreads, 3) stream_rows_kernel(const __grid_constant__ StreamArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  StreamSmem &S = *reinterpret_cast<StreamSmem *>(smem_raw);
  int *pen_tab = reinterpret_cast<int *>(smem_raw + sizeof(StreamSmem));

  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();
  const int crank = (int)cluster.block_rank();
  const int slot = blockIdx.x / csize;
  const int row = a.row_list ? a.row_list[slot] : slot;
  const int tid = threadIdx.x, lane = tid & 31;

  const RowParams p = a.params[a.params_per_row ? row : 0];
  const int Vt = a.vocab_total;

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
  __syncthreads();

  auto tile_len = [&](int t) { return min(kTile, s1 - s0 - t * kTile); };
  auto tile_bulk = [&](int t) { return base_aligned && ((tile_len(t) & 3) == 0); };
  auto issue = [&](int t) {  // thread 0 only
    if (t < n_tiles && tile_bulk(t)) {
      const uint32_t bytes = (uint32_t)tile_len(t) * 4u;
      uint64_t *bar = &S.full[t % kStages];
      mbar_expect_tx(bar, bytes);
      bulk_g2s(S.ring[t % kStages], rowp + s0 + (size_t)t * kTile, bytes, bar);
    }
  };
  if (tid == 0)
    for (int t = 0; t < kStages; ++t) issue(t);

  // penalty set and the candidate budget, while the first copies are in flight
  int npen = 0;
  if (p.repeat_penalty != 1.f && a.history != nullptr) {
    long long hn = a.hist_len ? a.hist_len[row] : a.hist_len_all;
    hn = hn < 0 ? 0 : (hn > a.hist_stride ? a.hist_stride : hn);
    npen = build_pen_set(pen_tab, a.pen_slots, &S.pen_unique, a.history + (size_t)row * a.hist_stride, hn,
                         p.repeat_last_n, Vt, a.status);
  }
  const bool greedy = p.temperature <= 0.f;
  const int K = greedy ? 1 : (p.top_k > 0 ? min(p.top_k, Vt) : Vt);  // sampler.cpp:39-40
  int M = min(Vt, K + npen);
  if (M >= Vt / 4) M = Vt;  // top_m returns the whole row in this case (sampler.cpp:14)

  // ---- streaming phase ----
  uint32_t thr = 0;  // accept keys strictly above; 0 accepts everything
  bool failed = false;
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t % kStages;
    const int len = tile_len(t);
    const int tbase = s0 + t * kTile;
    if (tile_bulk(t)) {
      if (!mbar_wait_bounded(&S.full[st], (uint32_t)(t / kStages) & 1u)) failed = true;
    } else {  // unaligned row or ragged tail: plain loads into the same stage
      for (int i = tid; i < len; i += kThreads) S.ring[st][i] = rowp[tbase + i];
      __syncthreads();
    }
    uint32_t keys[8];
    int nacc = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int off = h * (kThreads * 4) + tid * 4;
      const float4 v = *reinterpret_cast<const float4 *>(&S.ring[st][off]);
      const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t k = f2key(f[j]);
        const bool acc = (off + j < len) && (k > thr);
        keys[h * 4 + j] = acc ? k : 0u;
        nacc += acc ? 1 : 0;
      }
    }
    if (__any_sync(0xffffffffu, nacc > 0)) {
      int incl = nacc;  // warp inclusive scan of the per-lane accept counts
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      int wbase = 0;
      if (lane == 0) wbase = atomicAdd(&S.cand_count, total);
      wbase = __shfl_sync(0xffffffffu, wbase, 0);
      int pos = wbase + incl - nacc;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (keys[e] != 0u) {
          const int off = (e >> 2) * (kThreads * 4) + tid * 4 + (e & 3);
          if (pos < kCandCap) S.cand[pos] = make_comp(keys[e], (uint32_t)(a.id_offset + tbase + off));
          ++pos;
        }
      }
    }
    __syncthreads();  // stage consumed by every thread; candidate count settled
    if (tid == 0) issue(t + kStages);
    const int cnt = S.cand_count;
    if (cnt > kCandCap) { if (tid == 0) atomicOr(a.status, ST_CAPACITY); }
    if (cnt > kCandHigh && cnt > M) {
      const int nn = min(cnt, kCandCap);
      const unsigned long long pivot = block_select_pivot(S.cand, nn, M, S.hist, S.sel);
      block_compact(S.cand, nn, pivot, &S.cand_count);
      // later columns must beat the weakest kept key: an equal key at a higher index loses (sampler.cpp:16).
      // The select may stop on a key prefix, so take the minimum over the kept entries.
      uint32_t mk = 0xffffffffu;
      for (int i = tid; i < M; i += kThreads) mk = min(mk, comp_key(S.cand[i]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mk = min(mk, __shfl_xor_sync(0xffffffffu, mk, o));
      if (tid == 0) S.sel[3] = 0xffffffffu;
      __syncthreads();
      if (lane == 0) atomicMin(&S.sel[3], mk);
      __syncthreads();
      thr = S.sel[3];
    }
  }
  if (failed && tid == 0) atomicOr(a.status, ST_COPY_TIMEOUT);

  // MODE_MERGE: candidates come from the gathered per-shard lists instead of a stream
  if (MODE == MODE_MERGE) {
    const int total = a.n_shards * a.cand_slots;
    for (int i = tid; i < total; i += kThreads) {
      const int sh = i / a.cand_slots, s = i - sh * a.cand_slots;
      const unsigned long long c = a.cand_io[((size_t)sh * a.cand_rows + row) * a.cand_slots + s];
      if (c != 0ULL) {
        const int pos = atomicAdd(&S.cand_count, 1);
        if (pos < kMergeCap) S.cand[pos] = c;
      }
    }
    __syncthreads();
    if (S.cand_count > kMergeCap && tid == 0) atomicOr(a.status, ST_CAPACITY);
  }

  // ---- exact top-M of this CTA ----
  int n = min(S.cand_count, MODE == MODE_MERGE ? kMergeCap : kCandCap);
  if (n > M) {
    const unsigned long long pivot = block_select_pivot(S.cand, n, M, S.hist, S.sel);
    n = block_compact(S.cand, n, pivot, &S.cand_count);
  }

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
    if (n > M) {
      const unsigned long long pivot = block_select_pivot(S.cand, n, M, S.hist, S.sel);
      n = block_compact(S.cand, n, pivot, &S.cand_count);
    }
  }

  if (MODE == MODE_LOCAL_TOPM) {  // hand this GPU's winners to the all-gather
    unsigned long long *out = a.cand_io + (size_t)row * a.cand_slots;
    for (int i = tid; i < a.cand_slots; i += kThreads) out[i] = i < n ? S.cand[i] : 0ULL;
    if (n > a.cand_slots && tid == 0) atomicOr(a.status, ST_CAPACITY);
    return;
  }

  unsigned long long *sorted = reinterpret_cast<unsigned long long *>(&S.ring[0][0]);
  float *ev = reinterpret_cast<float *>(&S.cand[0]);
  float *pv = ev + kCandCap;
  // finish_row reads cand[0..n) until the rank sort is done, then overwrites it with ev / pv (n <= 4096)
  finish_row(a, row, p, S.cand, n, K, pen_tab, npen, sorted, ev, pv);
}

}  // namespace qpb
