// Port of the reference micro-benchmark (bench/sampler_bench.cpp) to the C++ mirror of qp::Sampler: same logits
// (1000 distinct values, ~152-way ties), same 300-entry history, the four temperature / penalty combinations, but
// with seed 42 so that the output is reproducible.  Prints, per combination, the size of the distribution, its
// first ids and eight successive draws; tests/test_gpu_cpp.py compares them with the fixtures generated from
// the reference.  Also times 200 sample() calls like the original.
#include <chrono>
#include <cstdio>
#include <vector>

#include "qpack_b200/sampler.hpp"

static double now() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

int main() {
  const int V = 151936;
  std::vector<float> lg(V);
  for (int i = 0; i < V; i++) lg[i] = (float)((i * 7919) % 1000) / 100.f;
  std::vector<int> hist(300);
  for (int i = 0; i < 300; i++) hist[i] = (i * 31) % V;
  for (float temp : {0.f, 0.7f})
    for (float rp : {1.f, 1.1f}) {
      qpb::SamplerParams p;
      p.temperature = temp;
      p.repeat_penalty = rp;
      p.seed = 42;
      qpb::Sampler s(p);
      std::vector<std::pair<int, float>> d;
      s.dist(lg.data(), V, hist, d);
      printf("temp %.1f rep %.1f: dist %zu first %d p0 %.9g draws", temp, rp, d.size(), d[0].first, d[0].second);
      for (int r = 0; r < 8; r++) printf(" %d", s.sample(lg.data(), V, hist));
      // draw() / accept() on host-side pairs share the sampler's stream
      int repl = -1;
      const bool acc = s.accept(d, d[0].first, &repl);
      printf(" accept %d repl %d draw %d", acc ? 1 : 0, repl, s.draw(d));
      double a = now();
      int x = 0;
      for (int r = 0; r < 200; r++) x += s.sample(lg.data(), V, hist);
      printf(" | %.1f us/token (%d)\n", (now() - a) / 200 * 1e6, x % 7);
    }
  return 0;
}
