// C entry points around the UNMODIFIED reference sampler (qp::Sampler, include/qpack/engine.h:27-43,
// src/sampler.cpp) so that Python tests and the CPU-baseline leg of the benchmark can drive it.
// TEST INFRASTRUCTURE: compiled by oracle/Makefile together with the reference's own src/sampler.cpp and
// src/kernels_x86.cpp (read where they lie; never copied into this repository) into oracle/_ref/.
// Nothing in the CUDA library links or loads this.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "qpack/engine.h"

namespace {
struct Params {  // byte-compatible with qp::SamplerParams (engine.h:17-25)
  float temperature;
  int32_t top_k;
  float top_p;
  float min_p;
  float repeat_penalty;
  int32_t repeat_last_n;
  uint64_t seed;
};
static_assert(sizeof(Params) == sizeof(qp::SamplerParams), "parameter block layout");

qp::SamplerParams to_qp(const Params &p) {
  qp::SamplerParams q;
  q.temperature = p.temperature;
  q.top_k = p.top_k;
  q.top_p = p.top_p;
  q.min_p = p.min_p;
  q.repeat_penalty = p.repeat_penalty;
  q.repeat_last_n = p.repeat_last_n;
  q.seed = p.seed;
  return q;
}
}  // namespace

extern "C" {

void *ref_create(const Params *p) { return new qp::Sampler(to_qp(*p)); }
void ref_destroy(void *s) { delete static_cast<qp::Sampler *>(s); }

int ref_sample(void *s, const float *logits, int V, const int32_t *history, int64_t hist_n) {
  std::vector<int> h(history, history + hist_n);
  return static_cast<qp::Sampler *>(s)->sample(logits, V, h);
}

int ref_dist(void *s, const float *logits, int V, const int32_t *history, int64_t hist_n, int64_t hist_len,
             int32_t *out_ids, float *out_p, int cap) {
  std::vector<int> h(history, history + hist_n);
  std::vector<std::pair<int, float>> d;
  static_cast<qp::Sampler *>(s)->dist(logits, V, h, d, hist_len < 0 ? (size_t)-1 : (size_t)hist_len);
  for (size_t i = 0; i < d.size() && (int)i < cap; i++) {
    out_ids[i] = d[i].first;
    out_p[i] = d[i].second;
  }
  return (int)d.size();
}

int ref_draw(void *s, const int32_t *ids, const float *p, int n) {
  std::vector<std::pair<int, float>> d(n);
  for (int i = 0; i < n; i++) d[i] = {ids[i], p[i]};
  return static_cast<qp::Sampler *>(s)->draw(d);
}

int ref_accept(void *s, const int32_t *ids, const float *p, int n, int32_t token, int32_t *repl) {
  std::vector<std::pair<int, float>> d(n);
  for (int i = 0; i < n; i++) d[i] = {ids[i], p[i]};
  int r = -1;
  const bool ok = static_cast<qp::Sampler *>(s)->accept(d, token, &r);
  *repl = r;
  return ok ? 1 : 0;
}

// One fresh qp::Sampler per row (params[row] or params[0]); rows fanned over `threads` host threads.
// Returns the wall-clock seconds spent inside the sampling loop (thread start-up included).
double ref_sample_rows(const Params *params, int n_params, const float *logits, int64_t row_stride, int n_rows, int V,
                       const int32_t *history, int64_t hist_stride, const int32_t *hist_len, int32_t *out_ids,
                       int32_t *out_count, int32_t *dist_ids, float *dist_p, int max_out, int threads) {
  if (threads < 1) threads = 1;
  std::atomic<int> next{0};
  auto work = [&]() {
    std::vector<int> h;
    std::vector<std::pair<int, float>> d;
    for (;;) {
      const int r = next.fetch_add(1);
      if (r >= n_rows) break;
      qp::Sampler s(to_qp(params[n_params == 1 ? 0 : r]));
      h.clear();
      if (history && hist_len) h.assign(history + (size_t)r * hist_stride, history + (size_t)r * hist_stride + hist_len[r]);
      s.dist(logits + (size_t)r * row_stride, V, h, d);
      out_ids[r] = s.draw(d);
      if (out_count) out_count[r] = (int)d.size();
      if (dist_ids)
        for (size_t i = 0; i < d.size() && (int)i < max_out; i++) {
          dist_ids[(size_t)r * max_out + i] = d[i].first;
          dist_p[(size_t)r * max_out + i] = d[i].second;
        }
    }
  };
  const auto t0 = std::chrono::steady_clock::now();
  if (threads == 1) {
    work();
  } else {
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; t++) pool.emplace_back(work);
    for (auto &t : pool) t.join();
  }
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

int ref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
