// Speculative verification on the device: the accept / resample rule of qp::Sampler::accept (src/sampler.cpp:65-73)
// and the draw of qp::Sampler::draw (58-63), applied to CHAINS of rows the way Session::generate does
// (src/chat.cpp:236-251): the rows of a chain are the distributions after each proposed token, they are verified in
// order with ONE random stream (the sampler of the request), verification stops at the first rejected proposal with
// the replacement token, and a chain whose proposals all pass takes its next token from the row after the last one.
//
// Random words are taken exactly as the reference takes them.  For a proposal of probability p in its row: none for
// the acceptance test if p >= 1 or p == 0, else one; after a rejection one more for the replacement draw unless at
// most one other entry is left.  For the final draw one, unless that distribution has a single entry.
//
// One warp per chain.  The distributions are the (id, probability) rows written by the sampling kernels.
#pragma once
#include "common.cuh"

namespace qpb {

struct VerifyArgs {
  const int *dist_ids;      // [n_chains * chain_rows][max_out]
  const float *dist_p;      // same shape
  const int *dist_count;    // [n_chains * chain_rows]
  int max_out;
  int n_chains;
  int chain_rows;           // rows per chain: one per proposal, plus the row after the last proposal
  const int *proposals;     // [n_chains][chain_rows - 1]
  const int *n_proposals;   // [n_chains] (each 0 .. chain_rows - 1) or nullptr = chain_rows - 1 everywhere
  unsigned long long *rng_state;  // [rows][312]: chain c draws from the state of its first row, c * chain_rows
  unsigned int *rng_drawn;        // [rows]
  int *accepted;            // [n_chains] proposals accepted
  int *next;                // [n_chains] the token that follows them: the replacement, or the draw of the next row
  int *status;
  int debug_flags;          // bit 0: take the sequential walk always (tests)
};

constexpr int kVerifyWarps = 4;  // chains per CTA

// one uniform variate of the chain's stream, on every lane
__device__ __forceinline__ double verify_uniform(unsigned long long *mt, unsigned int *drawn, int lane) {
  unsigned long long w = 0;
  if (lane == 0) {
    const MtFetch f = mt_fetch(mt, drawn);
    w = mt_commit(f, mt, drawn);
  }
  w = __shfl_sync(0xffffffffu, w, 0);
  return word_to_uniform(w);
}

// Sampler::draw over the entries of a row whose id differs from `skip` (skip < 0: every entry), each probability
// divided by `denom` in float first when `divide` is set (the `rest` list of accept, sampler.cpp:70-71).  `m` is the
// number of such entries (>= 2) and `r` the variate.  The reference subtracts entry by entry in double and returns
// the first entry at which the remainder is <= 0, else the last entry.  Here 32 entries at a time are compared
// through a warp prefix sum; a comparison within 1e-9 of equality (the two orders of addition differ by far less)
// sends the whole walk down the sequential path instead.
__device__ int verify_walk(const int *ids, const float *p, int n, int skip, bool divide, float denom, double r, int lane,
                           bool force_sequential) {
  constexpr double kEps = 1e-9;
  double carry = 0.0;
  int last_id = -1;
  bool ambiguous = force_sequential;
  for (int base = 0; base < n && !ambiguous; base += 32) {
    const int j = base + lane;
    int id = -1;
    double q = 0.0;
    bool live = false;
    if (j < n) {
      id = ids[j];
      live = id != skip;
      if (live) q = (double)(divide ? __fdiv_rn(p[j], denom) : p[j]);
    }
    double incl = q;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const double c = carry + incl;
    const uint32_t livemask = __ballot_sync(0xffffffffu, live);
    const uint32_t hit = __ballot_sync(0xffffffffu, live && c >= r);
    const uint32_t amb = __ballot_sync(0xffffffffu, live && fabs(c - r) <= kEps);
    // an ambiguous compare only matters up to the first clear hit, and never at the very last live entry
    const uint32_t upto = hit ? ((2u << (__ffs(hit) - 1)) - 1u) : 0xffffffffu;
    uint32_t amb_rel = amb & upto;
    if (amb_rel && base + 32 >= n) amb_rel &= ~(1u << (31 - __clz(livemask)));  // livemask != 0 when amb != 0
    if (amb_rel) { ambiguous = true; break; }
    if (hit) return __shfl_sync(0xffffffffu, id, __ffs(hit) - 1);
    if (livemask) last_id = __shfl_sync(0xffffffffu, id, 31 - __clz(livemask));
    carry = __shfl_sync(0xffffffffu, c, 31);
  }
  if (!ambiguous) return last_id;
  // sequential walk (every lane the same)
  double rr = r;
  int pick = -1;
#pragma unroll 1
  for (int j = 0; j < n; ++j) {
    const int id = ids[j];
    if (id == skip) continue;
    pick = id;
    rr -= (double)(divide ? __fdiv_rn(p[j], denom) : p[j]);
    if (rr <= 0.0) break;
  }
  return pick;
}

__global__ void __launch_bounds__(32 * kVerifyWarps) verify_chains_kernel(const VerifyArgs a) {
  const int lane = threadIdx.x & 31;
  const int chain = blockIdx.x * kVerifyWarps + (threadIdx.x >> 5);
  if (chain >= a.n_chains) return;
  const int row0 = chain * a.chain_rows;
  unsigned long long *mt = a.rng_state + (size_t)row0 * MT_N;
  unsigned int *drawn = a.rng_drawn + row0;
  int k = a.n_proposals ? a.n_proposals[chain] : a.chain_rows - 1;
  k = k < 0 ? 0 : (k > a.chain_rows - 1 ? a.chain_rows - 1 : k);
  int acc = 0, next = -1;
  for (int i = 0; i < k; ++i) {
    const int row = row0 + i;
    const int *ids = a.dist_ids + (size_t)row * a.max_out;
    const float *pr = a.dist_p + (size_t)row * a.max_out;
    int n = a.dist_count[row];
    if (n > a.max_out) { if (lane == 0) atomicOr(a.status, ST_CAPACITY); n = a.max_out; }
    const int token = a.proposals[(size_t)chain * (a.chain_rows - 1) + i];
    // probability of the proposal: the first entry with its id (sampler.cpp:66); entries with its id in all
    float p = 0.f;
    int matches = 0;
    bool found = false;
    for (int base = 0; base < n; base += 32) {
      const int j = base + lane;
      const bool m = j < n && ids[j] == token;
      const uint32_t mm = __ballot_sync(0xffffffffu, m);
      if (mm && !found) {
        found = true;
        p = pr[base + __ffs(mm) - 1];
      }
      matches += __popc(mm);
    }
    bool ok = p >= 1.f;                                                        // sampler.cpp:67
    if (!ok && p > 0.f) ok = verify_uniform(mt, drawn, lane) < (double)p;      // :68
    if (ok) { ++acc; continue; }
    const int m = n - matches;  // entries of `rest` (:69-70)
    if (m <= 0) {
      next = token;             // :71, nothing else to offer
    } else if (m == 1) {
      int other = -1;           // a one-entry draw takes no random word (:59)
      for (int base = 0; base < n; base += 32) {
        const int j = base + lane;
        const uint32_t mm = __ballot_sync(0xffffffffu, j < n && ids[j] != token);
        if (mm) other = ids[base + __ffs(mm) - 1];
      }
      next = other;
    } else {
      const double r = verify_uniform(mt, drawn, lane);
      next = verify_walk(ids, pr, n, token, true, __fsub_rn(1.f, p), r, lane, a.debug_flags & 1);
    }
    break;
  }
  if (next < 0) {
    // every proposal passed: the token after the last one is drawn from the next row (chat.cpp:250)
    const int row = row0 + acc;
    const int *ids = a.dist_ids + (size_t)row * a.max_out;
    const float *pr = a.dist_p + (size_t)row * a.max_out;
    int n = a.dist_count[row];
    if (n > a.max_out) { if (lane == 0) atomicOr(a.status, ST_CAPACITY); n = a.max_out; }
    if (n <= 1) next = n == 1 ? ids[0] : -1;
    else next = verify_walk(ids, pr, n, -1, false, 1.f, verify_uniform(mt, drawn, lane), lane, a.debug_flags & 1);
  }
  if (lane == 0) {
    a.accepted[chain] = acc;
    a.next[chain] = next;
  }
}

}  // namespace qpb
