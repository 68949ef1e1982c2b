/*
 * CPU oracle for the token sampler: TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of the reference sampler chain (qpack src/sampler.cpp:8-73 with the
 * parameter block of include/qpack/engine.h:17-25).  Only the tests, the smoke check and the CPU
 * leg of the benchmark may load it; the CUDA library never links or calls it.
 *
 * Parity status: the reference ships no test, golden vector or known answer for its sampler, so this
 * restatement is pinned against outputs of the reference itself (the reference sources compiled by
 * oracle/Makefile into oracle/_ref/, and the fixtures under tests/golden/ generated from that build).
 *
 * Third-party pieces the reference takes from its toolchain, restated here:
 *   - std::mt19937_64 (ISO C++ [rand.predef]; libstdc++ 13.3): 64-bit Mersenne twister,
 *     w=64 n=312 m=156 r=31 a=0xb5026f5aa96619e9 u=29 d=0x5555555555555555 s=17 b=0x71d67fffeda60000
 *     t=37 c=0xfff7eee000000000 l=43 f=6364136223846793005; call sites sampler.cpp:8,60,68.
 *   - std::uniform_real_distribution<double>(0,1) on that engine (libstdc++ generate_canonical):
 *     one 64-bit word w per variate, u = (double)w * 2^-64, clamped to the largest double below 1.
 *   - expf: the C library's own (glibc 2.39), called, not restated, because the reference calls it too
 *     (sampler.cpp:47).
 *   - std::nth_element / std::sort: any exact selection / sort gives the same result because the
 *     comparator (value descending, index ascending) is a strict total order on distinct pairs.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MT_N 312
#define ORC_MT_M 156

typedef struct {
  float temperature;
  int32_t top_k;
  float top_p;
  float min_p;
  float repeat_penalty;
  int32_t repeat_last_n;
  uint64_t seed;
} orc_params; /* same field order and 32-byte layout as qp::SamplerParams, engine.h:17-25 */

typedef struct {
  int32_t id;
  float v;
} orc_pair;

typedef struct orc_sampler {
  orc_params p;
  uint64_t mt[ORC_MT_N];
  int mti;
  uint64_t words_drawn;
  orc_pair *buf; /* candidate scratch */
  size_t buf_cap;
  int32_t *pen;
  size_t pen_cap;
} orc_sampler;

/* ---- mt19937_64, seeding as std::mersenne_twister_engine::seed(value) ------------------------------ */
static void mt_seed(orc_sampler *s, uint64_t seed) {
  s->mt[0] = seed;
  for (int i = 1; i < ORC_MT_N; i++)
    s->mt[i] = 6364136223846793005ULL * (s->mt[i - 1] ^ (s->mt[i - 1] >> 62)) + (uint64_t)i;
  s->mti = ORC_MT_N;
  s->words_drawn = 0;
}

static uint64_t mt_next(orc_sampler *s) {
  if (s->mti >= ORC_MT_N) {
    const uint64_t UM = 0xFFFFFFFF80000000ULL, LM = 0x7FFFFFFFULL, A = 0xB5026F5AA96619E9ULL;
    for (int k = 0; k < ORC_MT_N; k++) {
      uint64_t y = (s->mt[k] & UM) | (s->mt[(k + 1) % ORC_MT_N] & LM);
      s->mt[k] = s->mt[(k + ORC_MT_M) % ORC_MT_N] ^ (y >> 1) ^ ((y & 1) ? A : 0);
    }
    s->mti = 0;
  }
  uint64_t x = s->mt[s->mti++];
  x ^= (x >> 29) & 0x5555555555555555ULL;
  x ^= (x << 17) & 0x71D67FFFEDA60000ULL;
  x ^= (x << 37) & 0xFFF7EEE000000000ULL;
  x ^= x >> 43;
  s->words_drawn++;
  return x;
}

static double mt_uniform(orc_sampler *s) {
  double u = (double)mt_next(s) * 0x1p-64;
  if (u >= 1.0) u = nextafter(1.0, 0.0);
  return u;
}

/* ---- construction -------------------------------------------------------------------------------- */
orc_sampler *orc_create(const orc_params *p) {
  orc_sampler *s = (orc_sampler *)calloc(1, sizeof(orc_sampler));
  if (!s) return NULL;
  s->p = *p;
  /* seed 0 means "non-deterministic" in the reference (sampler.cpp:8); the oracle has no use for that and
     seeds with 0 literally, callers never pass 0 */
  mt_seed(s, p->seed);
  return s;
}

void orc_destroy(orc_sampler *s) {
  if (!s) return;
  free(s->buf);
  free(s->pen);
  free(s);
}

void orc_reseed(orc_sampler *s, uint64_t seed) { mt_seed(s, seed); }
uint64_t orc_words_drawn(const orc_sampler *s) { return s->words_drawn; }
uint64_t orc_next_word(orc_sampler *s) { return mt_next(s); }
double orc_next_uniform(orc_sampler *s) { return mt_uniform(s); }

/* (value descending, index ascending): the one order used everywhere, sampler.cpp:16,43 */
static int pair_before(const orc_pair *a, const orc_pair *b) {
  return a->v > b->v || (a->v == b->v && a->id < b->id);
}
static int pair_cmp(const void *a, const void *b) {
  const orc_pair *x = (const orc_pair *)a, *y = (const orc_pair *)b;
  if (pair_before(x, y)) return -1;
  if (pair_before(y, x)) return 1;
  return 0;
}

/* min-heap on the order above: heap[0] is the weakest kept pair */
static void heap_sift_down(orc_pair *h, int n, int i) {
  for (;;) {
    int l = 2 * i + 1, r = l + 1, w = i;
    if (l < n && pair_before(&h[w], &h[l])) w = l;
    if (r < n && pair_before(&h[w], &h[r])) w = r;
    if (w == i) return;
    orc_pair t = h[i];
    h[i] = h[w];
    h[w] = t;
    i = w;
  }
}

/* the M largest (index, value) pairs of x, unordered; all V when M >= V/4 (sampler.cpp:12-27) */
static int top_m(const float *x, int V, int M, orc_pair *out) {
  if (M >= V / 4) {
    for (int v = 0; v < V; v++) {
      out[v].id = v;
      out[v].v = x[v];
    }
    return V;
  }
  int n = 0;
  for (int v = 0; v < V; v++) {
    if (n < M) {
      out[n].id = v;
      out[n].v = x[v];
      n++;
      if (n == M)
        for (int i = M / 2 - 1; i >= 0; i--) heap_sift_down(out, M, i);
    } else if (x[v] > out[0].v) { /* an equal value at a higher index never displaces a kept pair */
      out[0].id = v;
      out[0].v = x[v];
      heap_sift_down(out, M, 0);
    }
  }
  return n;
}

/*
 * Sampler::dist (sampler.cpp:29-56).  history[0..hist_n) with only its first hist_len entries visible
 * (hist_len < 0 = all).  Writes up to cap (id, p) pairs, most likely first; returns the full count.
 */
int orc_dist(orc_sampler *s, const float *logits, int V, const int32_t *history, int64_t hist_n, int64_t hist_len,
             int32_t *out_ids, float *out_p, int cap) {
  const orc_params *p = &s->p;
  const int64_t hn = (hist_len < 0 || hist_len > hist_n) ? hist_n : hist_len;
  int npen = 0;
  if (p->repeat_penalty != 1.f) { /* sampler.cpp:34-38 */
    /* hn > (size_t)repeat_last_n: a negative repeat_last_n converts to a huge size_t, i.e. "whole history" */
    int64_t from = 0;
    if (p->repeat_last_n >= 0 && hn > (int64_t)p->repeat_last_n) from = hn - p->repeat_last_n;
    if ((size_t)(hn - from) > s->pen_cap) {
      s->pen_cap = (size_t)(hn - from);
      s->pen = (int32_t *)realloc(s->pen, s->pen_cap * sizeof(int32_t));
    }
    for (int64_t i = from; i < hn; i++) {
      const int32_t t = history[i];
      if (t < 0 || t >= V) continue;
      int dup = 0;
      for (int j = 0; j < npen; j++)
        if (s->pen[j] == t) {
          dup = 1;
          break;
        }
      if (!dup) s->pen[npen++] = t;
    }
  }
  const int greedy = p->temperature <= 0;
  const int K = greedy ? 1 : (p->top_k > 0 ? (p->top_k < V ? p->top_k : V) : V); /* sampler.cpp:39-40 */
  int M = K + npen;
  if (M > V) M = V;
  if ((size_t)V > s->buf_cap) {
    s->buf_cap = (size_t)V;
    s->buf = (orc_pair *)realloc(s->buf, s->buf_cap * sizeof(orc_pair));
  }
  orc_pair *c = s->buf;
  int n = top_m(logits, V, M, c);
  if (npen) /* sampler.cpp:42 */
    for (int i = 0; i < n; i++)
      for (int j = 0; j < npen; j++)
        if (s->pen[j] == c[i].id) {
          c[i].v = c[i].v > 0 ? c[i].v / p->repeat_penalty : c[i].v * p->repeat_penalty;
          break;
        }
  qsort(c, (size_t)n, sizeof(orc_pair), pair_cmp); /* sampler.cpp:43 */
  if (n > K) n = K;
  if (greedy) { /* sampler.cpp:45 */
    if (cap > 0) {
      out_ids[0] = c[0].id;
      out_p[0] = 1.f;
    }
    return 1;
  }
  const float mx = c[0].v;
  double sum = 0;
  for (int i = 0; i < n; i++) { /* sampler.cpp:46-47 */
    c[i].v = expf((c[i].v - mx) / p->temperature);
    sum += c[i].v;
  }
  int keep = n;
  double cum = 0;
  for (int i = 0; i < n; i++) { /* sampler.cpp:48-52 */
    if (p->min_p > 0 && c[i].v < p->min_p * c[0].v) {
      keep = i > 1 ? i : 1;
      break;
    }
    cum += c[i].v / sum;
    if (cum >= p->top_p) {
      keep = i + 1;
      break;
    }
  }
  double tot = 0;
  for (int i = 0; i < keep; i++) tot += c[i].v; /* sampler.cpp:54 */
  for (int i = 0; i < keep && i < cap; i++) {
    out_ids[i] = c[i].id;
    out_p[i] = (float)(c[i].v / tot); /* sampler.cpp:55 */
  }
  return keep;
}

/* Sampler::draw (sampler.cpp:58-63) */
int orc_draw(orc_sampler *s, const int32_t *ids, const float *p, int n) {
  if (n == 1) return ids[0];
  double r = mt_uniform(s);
  for (int i = 0; i < n; i++) {
    r -= p[i];
    if (r <= 0) return ids[i];
  }
  return ids[n - 1];
}

/* Sampler::accept (sampler.cpp:65-73); returns 1 = accepted, 0 = rejected with *repl set */
int orc_accept(orc_sampler *s, const int32_t *ids, const float *p, int n, int32_t token, int32_t *repl) {
  float pt = 0;
  for (int i = 0; i < n; i++)
    if (ids[i] == token) {
      pt = p[i];
      break;
    }
  if (pt >= 1.f) return 1;
  if (pt > 0 && mt_uniform(s) < pt) return 1;
  int32_t *rid = (int32_t *)malloc((size_t)(n > 0 ? n : 1) * sizeof(int32_t));
  float *rp = (float *)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
  int m = 0;
  for (int i = 0; i < n; i++)
    if (ids[i] != token) {
      rid[m] = ids[i];
      rp[m] = p[i] / (1.f - pt);
      m++;
    }
  *repl = m == 0 ? token : orc_draw(s, rid, rp, m);
  free(rid);
  free(rp);
  return 0;
}

/* Sampler::sample (engine.h:30): dist on the whole history, then draw.  count_out (optional) = survivors. */
int orc_sample(orc_sampler *s, const float *logits, int V, const int32_t *history, int64_t hist_n, int *count_out) {
  int32_t *ids = (int32_t *)malloc((size_t)V * sizeof(int32_t));
  float *pr = (float *)malloc((size_t)V * sizeof(float));
  int n = orc_dist(s, logits, V, history, hist_n, -1, ids, pr, V);
  int t = orc_draw(s, ids, pr, n);
  if (count_out) *count_out = n;
  free(ids);
  free(pr);
  return t;
}

/*
 * Convenience for the tests: one fresh sampler per row (params[row % n_params], its own seed), one sample()
 * per row.  Optionally returns each row's distribution (first max_out pairs) and survivor count, and whether
 * the draw consumed a random word.
 */
void orc_sample_rows(const orc_params *params, int n_params, const float *logits, int64_t row_stride, int n_rows,
                     int V, const int32_t *history, int64_t hist_stride, const int32_t *hist_len, int32_t *out_ids,
                     int32_t *out_count, int32_t *dist_ids, float *dist_p, int max_out, int32_t *consumed) {
  int32_t *ids = (int32_t *)malloc((size_t)V * sizeof(int32_t));
  float *pr = (float *)malloc((size_t)V * sizeof(float));
  for (int r = 0; r < n_rows; r++) {
    orc_sampler *s = orc_create(&params[n_params == 1 ? 0 : r]);
    const int32_t *h = history ? history + (size_t)r * hist_stride : NULL;
    const int64_t hn = (history && hist_len) ? hist_len[r] : 0;
    int n = orc_dist(s, logits + (size_t)r * row_stride, V, h, hn, -1, ids, pr, V);
    out_ids[r] = orc_draw(s, ids, pr, n);
    if (out_count) out_count[r] = n;
    if (consumed) consumed[r] = (int32_t)s->words_drawn;
    if (dist_ids)
      for (int i = 0; i < n && i < max_out; i++) {
        dist_ids[(size_t)r * max_out + i] = ids[i];
        dist_p[(size_t)r * max_out + i] = pr[i];
      }
    orc_destroy(s);
  }
  free(ids);
  free(pr);
}

/* the C library's expf over an array: what the device restatement is compared with */
void orc_expf_vec(const float *x, float *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = expf(x[i]);
}
