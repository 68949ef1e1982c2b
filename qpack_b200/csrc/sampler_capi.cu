// Host side of the C ABI declared in include/qpack_b200_sampler.h: handle, parameter routing, launches.
// There is no CPU fallback: every entry point runs the sm_100a kernels or returns an error.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <random>
#include <string>
#include <vector>

#include "../../include/qpack_b200_sampler.h"
#include "sample_stream.cuh"
#include "sample_whole_kernel.cuh"

using namespace qpb;

static_assert(sizeof(qpb_sampler_params) == sizeof(RowParams), "C and device parameter blocks must match");

struct qpb_sampler {
  int device = 0;
  int max_rows = 0;
  int sm_count = 148;
  int n_params = 0;  // 0: not set, 1: shared, else per row
  std::vector<qpb_sampler_params> h_params;
  RowParams *d_params = nullptr;
  unsigned long long *d_rng = nullptr;  // [max_rows][312]
  unsigned int *d_drawn = nullptr;      // [max_rows]
  int *d_status = nullptr;
  int *d_rows_stream = nullptr;  // rows taking the streaming kernel
  int *d_rows_whole = nullptr;   // rows taking the whole-row kernel
  // routing cache: valid for (routed_rows, routed_vocab)
  int routed_rows = -1, routed_vocab = -1, n_stream = 0, n_whole = 0, max_window = 0;
  long long routed_hist_cap = -1;
  int cluster = 0;
  int stream_slots = 0;  // CTAs of the streaming kernel resident on the GPU at once (0: not queried yet)
  bool attr_done[4] = {false, false, false, false};
  int64_t launches = 0;
  // staging for the host-buffer entry point
  float *d_stage_logits = nullptr;
  size_t stage_logits_bytes = 0;
  int *d_stage_hist = nullptr;
  size_t stage_hist_bytes = 0;
  int *d_stage_hlen = nullptr;
  int *d_stage_ids = nullptr;
  cudaStream_t own_stream = nullptr;
  long long *d_phase_clk = nullptr;  // [max_rows][16] when phase stamps are enabled
  std::string err;
};

namespace {

int fail(qpb_sampler *s, int code, const std::string &msg) {
  if (s) s->err = msg;
  return code;
}
#define QPB_CUDA(s, call)                                                                                     \
  do {                                                                                                        \
    cudaError_t e_ = (call);                                                                                  \
    if (e_ != cudaSuccess) return fail((s), QPB_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// std::mersenne_twister_engine::seed(value) for mt19937_64 (the constructor the reference uses, sampler.cpp:8)
void mt_seed_host(uint64_t seed, uint64_t *mt) {
  mt[0] = seed;
  for (int i = 1; i < MT_N; i++) mt[i] = 6364136223846793005ULL * (mt[i - 1] ^ (mt[i - 1] >> 62)) + (uint64_t)i;
}

// candidate budget a row can need: top_k + window, or "whole row" (returned as a huge value)
long long row_budget(const qpb_sampler_params &p, int vocab_total) {
  const bool greedy = p.temperature <= 0.f;
  const long long K = greedy ? 1 : (p.top_k > 0 ? (p.top_k < vocab_total ? p.top_k : vocab_total) : vocab_total);
  long long window = 0;
  if (p.repeat_penalty != 1.f) window = p.repeat_last_n < 0 ? (long long)1 << 40 : p.repeat_last_n;
  return K + window;
}

int pen_slots_for(long long window) {
  int slots = 64;
  while (slots < 2 * window && slots < (1 << 20)) slots <<= 1;
  return slots;
}

// Splits rows [0, n_rows) between the two kernels and uploads the lists.  hist_cap bounds the window.
int route_rows(qpb_sampler *s, int n_rows, int vocab_total, long long hist_cap, cudaStream_t st) {
  if (s->routed_rows == n_rows && s->routed_vocab == vocab_total && s->routed_hist_cap == hist_cap) return QPB_OK;
  std::vector<int> a, b;
  long long maxw = 0;
  for (int r = 0; r < n_rows; r++) {
    const qpb_sampler_params &p = s->h_params[s->n_params == 1 ? 0 : r];
    long long w = 0;
    if (p.repeat_penalty != 1.f) w = p.repeat_last_n < 0 ? hist_cap : (p.repeat_last_n < hist_cap ? p.repeat_last_n : hist_cap);
    if (w > maxw) maxw = w;
    const bool greedy = p.temperature <= 0.f;
    const long long K = greedy ? 1 : (p.top_k > 0 ? (p.top_k < vocab_total ? p.top_k : vocab_total) : vocab_total);
    (K + w <= kSmallMaxM ? a : b).push_back(r);
  }
  s->n_stream = (int)a.size();
  s->n_whole = (int)b.size();
  s->max_window = (int)(maxw > (1 << 30) ? (1 << 30) : maxw);
  // pageable-source async copies return after the source has been staged, so the vectors may go out of scope
  if (!a.empty()) QPB_CUDA(s, cudaMemcpyAsync(s->d_rows_stream, a.data(), a.size() * sizeof(int), cudaMemcpyHostToDevice, st));
  if (!b.empty()) QPB_CUDA(s, cudaMemcpyAsync(s->d_rows_whole, b.data(), b.size() * sizeof(int), cudaMemcpyHostToDevice, st));
  s->routed_rows = n_rows;
  s->routed_vocab = vocab_total;
  s->routed_hist_cap = hist_cap;
  return QPB_OK;
}

int pick_cluster(const qpb_sampler *s, int rows) {
  if (s->cluster) return s->cluster;
  // one CTA per row as soon as a handful of rows are in flight; a cluster only pays for a few rows
  return rows <= 8 ? 8 : 1;
}

template <int MODE>
int launch_stream(qpb_sampler *s, const StreamArgs &args, int rows, int cluster, cudaStream_t st) {
  const size_t smem = sizeof(StreamSmem) + (size_t)args.pen_slots * sizeof(int);
  if (smem > 200 * 1024) return fail(s, QPB_ERR_UNSUPPORTED, "history window too large for the penalty table");
  if (!s->attr_done[MODE]) {  // once per handle (the attribute is per device)
    QPB_CUDA(s, cudaFuncSetAttribute(stream_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    s->attr_done[MODE] = true;
    if (MODE == MODE_SAMPLE) {
      int per_sm = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, stream_rows_kernel<MODE>, kThreads, smem) == cudaSuccess && per_sm > 0)
        s->stream_slots = per_sm * s->sm_count;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * cluster), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  QPB_CUDA(s, cudaLaunchKernelEx(&cfg, stream_rows_kernel<MODE>, args));
  s->launches++;
  return QPB_OK;
}

struct Inputs {
  const float *d_logits;
  int64_t row_stride;
  int n_rows;
  int vocab;
  int vocab_total;
  int id_offset;
  const int32_t *d_history;
  int64_t hist_stride;
  const int32_t *d_hist_len;
  int hist_len_all;
};

int check_inputs(qpb_sampler *s, const Inputs &in, bool need_logits) {
  if (!s) return QPB_ERR_INVALID;
  if (s->n_params == 0) return fail(s, QPB_ERR_INVALID, "qpb_sampler_set_params has not been called");
  if (need_logits && !in.d_logits) return fail(s, QPB_ERR_INVALID, "logits pointer is null");
  if (in.n_rows <= 0 || in.n_rows > s->max_rows) return fail(s, QPB_ERR_INVALID, "n_rows outside [1, max_rows]");
  if (s->n_params != 1 && in.n_rows > s->n_params) return fail(s, QPB_ERR_INVALID, "n_rows exceeds the number of parameter blocks");
  if (in.vocab <= 0 || in.vocab_total < in.vocab) return fail(s, QPB_ERR_INVALID, "vocab must be positive");
  if (need_logits && in.row_stride < in.vocab) return fail(s, QPB_ERR_INVALID, "row_stride smaller than vocab");
  if (in.d_history && (in.hist_stride < 0 || (!in.d_hist_len && (in.hist_len_all < 0 || in.hist_len_all > in.hist_stride))))
    return fail(s, QPB_ERR_INVALID, "history length outside [0, hist_stride]");
  return QPB_OK;
}

void fill_common(qpb_sampler *s, const Inputs &in, StreamArgs &a) {
  a.logits = in.d_logits;
  a.row_stride = in.row_stride;
  a.vocab = in.vocab;
  a.vocab_total = in.vocab_total;
  a.id_offset = in.id_offset;
  a.params = s->d_params;
  a.params_per_row = s->n_params == 1 ? 0 : 1;
  a.history = in.d_history;
  a.hist_stride = in.hist_stride;
  a.hist_len = in.d_hist_len;
  a.hist_len_all = in.d_history ? in.hist_len_all : 0;
  a.rng_state = s->d_rng;
  a.rng_drawn = s->d_drawn;
  a.status = s->d_status;
  a.pen_slots = pen_slots_for(s->max_window);
  a.phase_clk = s->d_phase_clk;
}

// Rows whose candidate budget exceeds the streaming kernel's take the whole-row kernel: one cluster per row,
// the row resident in the cluster's shared memory.
int launch_whole(qpb_sampler *s, const Inputs &in, int32_t *d_dist_ids, float *d_dist_p, int32_t *d_dist_count,
                 int max_out, int32_t *d_out_ids, bool draw, cudaStream_t st) {
  const int cluster = in.vocab >= 8192 ? kWMaxCluster : 1;
  int per = (in.vocab + cluster - 1) / cluster;
  per = (per + 3) & ~3;
  WholeArgs wa = {};
  fill_common(s, in, wa.s);
  wa.s.n_rows = s->n_whole;
  wa.s.row_list = s->d_rows_whole;
  wa.s.out_ids = d_out_ids;
  wa.s.draw = draw ? 1 : 0;
  wa.s.dist_ids = d_dist_ids;
  wa.s.dist_p = d_dist_p;
  wa.s.dist_count = d_dist_count;
  wa.s.max_out = max_out;
  wa.slice_cap = per;
  const size_t fixed = sizeof(WholeSmem) + (size_t)wa.s.pen_slots * sizeof(int);
  const size_t limit = 227 * 1024;
  if (fixed + (size_t)per * 4 > limit)
    return fail(s, QPB_ERR_UNSUPPORTED, "vocabulary too large for the whole-row kernel (about 440k columns)");
  wa.have_e = fixed + (size_t)per * 8 <= limit ? 1 : 0;
  const size_t smem = fixed + (size_t)per * (wa.have_e ? 8 : 4);
  if (!s->attr_done[3]) {
    QPB_CUDA(s, cudaFuncSetAttribute(whole_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit));
    s->attr_done[3] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(s->n_whole * cluster), 1, 1);
  cfg.blockDim = dim3(kWThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)cluster;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  QPB_CUDA(s, cudaLaunchKernelEx(&cfg, whole_rows_kernel, wa));
  s->launches++;
  return QPB_OK;
}
void whole_free(qpb_sampler *) {}

// sample / dist over whole (unsharded) rows
int run_rows(qpb_sampler *s, const Inputs &in, int32_t *d_dist_ids, float *d_dist_p, int32_t *d_dist_count, int max_out,
             int32_t *d_out_ids, bool draw, cudaStream_t st) {
  int rc = check_inputs(s, in, true);
  if (rc) return rc;
  DeviceGuard g(s->device);
  rc = route_rows(s, in.n_rows, in.vocab_total, in.d_history ? in.hist_stride : 0, st);
  if (rc) return rc;
  if (s->n_stream > 0) {
    StreamArgs a = {};
    fill_common(s, in, a);
    a.out_ids = d_out_ids;
    a.draw = draw ? 1 : 0;
    a.dist_ids = d_dist_ids;
    a.dist_p = d_dist_p;
    a.dist_count = d_dist_count;
    a.max_out = max_out;
    a.n_rows = s->n_stream;
    a.row_list = s->d_rows_stream;
    rc = launch_stream<MODE_SAMPLE>(s, a, s->n_stream, pick_cluster(s, s->n_stream), st);
    if (rc) return rc;
  }
  if (s->n_whole > 0) {
    rc = launch_whole(s, in, d_dist_ids, d_dist_p, d_dist_count, max_out, d_out_ids, draw, st);
    if (rc) return rc;
  }
  return QPB_OK;
}

}  // namespace


extern "C" {

int qpb_sampler_create(qpb_sampler **out, int device, int max_rows) {
  if (!out || max_rows <= 0) return QPB_ERR_INVALID;
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev) return QPB_ERR_CUDA;
  qpb_sampler *s = new (std::nothrow) qpb_sampler();
  if (!s) return QPB_ERR_INTERNAL;
  s->device = device;
  s->max_rows = max_rows;
  DeviceGuard g(device);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major < 10) {
    delete s;
    return QPB_ERR_UNSUPPORTED;  // sm_100a kernels only
  }
  s->sm_count = prop.multiProcessorCount;
  bool ok = cudaMalloc(&s->d_params, sizeof(RowParams) * max_rows) == cudaSuccess &&
            cudaMalloc(&s->d_rng, sizeof(unsigned long long) * MT_N * (size_t)max_rows) == cudaSuccess &&
            cudaMalloc(&s->d_drawn, sizeof(unsigned int) * max_rows) == cudaSuccess &&
            cudaMalloc(&s->d_status, sizeof(int)) == cudaSuccess &&
            cudaMalloc(&s->d_rows_stream, sizeof(int) * max_rows) == cudaSuccess &&
            cudaMalloc(&s->d_rows_whole, sizeof(int) * max_rows) == cudaSuccess &&
            cudaMemset(s->d_status, 0, sizeof(int)) == cudaSuccess &&
            cudaStreamCreateWithFlags(&s->own_stream, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    qpb_sampler_destroy(s);
    return QPB_ERR_CUDA;
  }
  *out = s;
  return QPB_OK;
}

int qpb_sampler_destroy(qpb_sampler *s) {
  if (!s) return QPB_OK;
  DeviceGuard g(s->device);
  cudaFree(s->d_params);
  cudaFree(s->d_rng);
  cudaFree(s->d_drawn);
  cudaFree(s->d_status);
  cudaFree(s->d_rows_stream);
  cudaFree(s->d_rows_whole);
  cudaFree(s->d_stage_logits);
  cudaFree(s->d_stage_hist);
  cudaFree(s->d_stage_hlen);
  cudaFree(s->d_stage_ids);
  cudaFree(s->d_phase_clk);
  whole_free(s);
  if (s->own_stream) cudaStreamDestroy(s->own_stream);
  delete s;
  return QPB_OK;
}

int qpb_sampler_set_params(qpb_sampler *s, const qpb_sampler_params *params, int n) {
  if (!s) return QPB_ERR_INVALID;
  if (!params || n < 1 || n > s->max_rows) return fail(s, QPB_ERR_INVALID, "params null or n outside [1, max_rows]");
  DeviceGuard g(s->device);
  s->h_params.assign(params, params + n);
  s->n_params = n;
  s->routed_rows = -1;
  std::vector<uint64_t> mt((size_t)s->max_rows * MT_N);
  std::random_device rd;
  for (int r = 0; r < s->max_rows; r++) {
    uint64_t seed = (n == 1) ? params[0].seed + (uint64_t)r : (r < n ? params[r].seed : 0);
    if ((n == 1 ? params[0].seed : (r < n ? params[r].seed : 1)) == 0)
      seed = ((uint64_t)rd() << 32) ^ rd();  // seed 0: non-deterministic, as std::random_device{}() in the reference
    mt_seed_host(seed, &mt[(size_t)r * MT_N]);
  }
  QPB_CUDA(s, cudaDeviceSynchronize());
  QPB_CUDA(s, cudaMemcpy(s->d_params, params, sizeof(RowParams) * n, cudaMemcpyHostToDevice));
  QPB_CUDA(s, cudaMemcpy(s->d_rng, mt.data(), mt.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
  QPB_CUDA(s, cudaMemset(s->d_drawn, 0, sizeof(unsigned int) * s->max_rows));
  return QPB_OK;
}

int qpb_sampler_sample_batch(qpb_sampler *s, const float *d_logits, int64_t row_stride, int n_rows, int vocab,
                             const int32_t *d_history, int64_t hist_stride, const int32_t *d_hist_len,
                             int hist_len_all, int32_t *d_out_ids, void *stream) {
  if (!s) return QPB_ERR_INVALID;
  if (!d_out_ids) return fail(s, QPB_ERR_INVALID, "output pointer is null");
  Inputs in{d_logits, row_stride, n_rows, vocab, vocab, 0, d_history, hist_stride, d_hist_len, hist_len_all};
  return run_rows(s, in, nullptr, nullptr, nullptr, 0, d_out_ids, true, (cudaStream_t)stream);
}

int qpb_sampler_dist_batch(qpb_sampler *s, const float *d_logits, int64_t row_stride, int n_rows, int vocab,
                           const int32_t *d_history, int64_t hist_stride, const int32_t *d_hist_len, int hist_len_all,
                           int32_t *d_dist_ids, float *d_dist_p, int32_t *d_dist_count, int max_out,
                           int32_t *d_out_ids, void *stream) {
  if (!s) return QPB_ERR_INVALID;
  if (!d_dist_count || max_out < 0 || (max_out > 0 && (!d_dist_ids || !d_dist_p)))
    return fail(s, QPB_ERR_INVALID, "distribution output pointers are null");
  Inputs in{d_logits, row_stride, n_rows, vocab, vocab, 0, d_history, hist_stride, d_hist_len, hist_len_all};
  return run_rows(s, in, max_out > 0 ? d_dist_ids : nullptr, d_dist_p, d_dist_count, max_out, d_out_ids,
                  d_out_ids != nullptr, (cudaStream_t)stream);
}

int qpb_sampler_check(qpb_sampler *s, void *stream) {
  if (!s) return QPB_ERR_INVALID;
  DeviceGuard g(s->device);
  int st = 0;
  QPB_CUDA(s, cudaMemcpyAsync(&st, s->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  QPB_CUDA(s, cudaStreamSynchronize((cudaStream_t)stream));
  if (st == 0) return QPB_OK;
  QPB_CUDA(s, cudaMemsetAsync(s->d_status, 0, sizeof(int), (cudaStream_t)stream));
  if (st & ST_COPY_TIMEOUT) return fail(s, QPB_ERR_DEVICE_TIMEOUT, "a device-side wait on a bulk copy gave up");
  char buf[96];
  snprintf(buf, sizeof buf, "device-side capacity check failed (status 0x%x)", st);
  return fail(s, QPB_ERR_INTERNAL, buf);
}

int qpb_sampler_sample_host(qpb_sampler *s, const float *h_logits, int64_t row_stride, int n_rows, int vocab,
                            const int32_t *h_history, int64_t hist_stride, const int32_t *h_hist_len,
                            int hist_len_all, int32_t *h_out_ids) {
  if (!s) return QPB_ERR_INVALID;
  if (!h_logits || !h_out_ids) return fail(s, QPB_ERR_INVALID, "host pointer is null");
  if (n_rows <= 0 || n_rows > s->max_rows || vocab <= 0 || row_stride < vocab)
    return fail(s, QPB_ERR_INVALID, "n_rows / vocab / row_stride out of range");
  DeviceGuard g(s->device);
  cudaStream_t st = s->own_stream;
  const size_t lbytes = ((size_t)(n_rows - 1) * row_stride + vocab) * sizeof(float);
  if (lbytes > s->stage_logits_bytes) {
    cudaFree(s->d_stage_logits);
    s->d_stage_logits = nullptr;
    s->stage_logits_bytes = 0;
    QPB_CUDA(s, cudaMalloc(&s->d_stage_logits, lbytes));
    s->stage_logits_bytes = lbytes;
  }
  if (!s->d_stage_ids) {
    QPB_CUDA(s, cudaMalloc(&s->d_stage_ids, sizeof(int) * s->max_rows));
    QPB_CUDA(s, cudaMalloc(&s->d_stage_hlen, sizeof(int) * s->max_rows));
  }
  const int *d_hist = nullptr, *d_hlen = nullptr;
  if (h_history && hist_stride > 0) {
    const size_t hbytes = (size_t)n_rows * hist_stride * sizeof(int);
    if (hbytes > s->stage_hist_bytes) {
      cudaFree(s->d_stage_hist);
      s->d_stage_hist = nullptr;
      s->stage_hist_bytes = 0;
      QPB_CUDA(s, cudaMalloc(&s->d_stage_hist, hbytes));
      s->stage_hist_bytes = hbytes;
    }
    QPB_CUDA(s, cudaMemcpyAsync(s->d_stage_hist, h_history, hbytes, cudaMemcpyHostToDevice, st));
    d_hist = s->d_stage_hist;
    if (h_hist_len) {
      QPB_CUDA(s, cudaMemcpyAsync(s->d_stage_hlen, h_hist_len, sizeof(int) * n_rows, cudaMemcpyHostToDevice, st));
      d_hlen = s->d_stage_hlen;
    }
  }
  QPB_CUDA(s, cudaMemcpyAsync(s->d_stage_logits, h_logits, lbytes, cudaMemcpyHostToDevice, st));
  Inputs in{s->d_stage_logits, row_stride, n_rows, vocab, vocab, 0, d_hist, hist_stride, d_hlen, hist_len_all};
  int rc = run_rows(s, in, nullptr, nullptr, nullptr, 0, s->d_stage_ids, true, st);
  if (rc) return rc;
  QPB_CUDA(s, cudaMemcpyAsync(h_out_ids, s->d_stage_ids, sizeof(int) * n_rows, cudaMemcpyDeviceToHost, st));
  return qpb_sampler_check(s, st);
}

int qpb_sampler_rng_get(qpb_sampler *s, int row, uint64_t *h_state313) {
  if (!s) return QPB_ERR_INVALID;
  if (!h_state313 || row < 0 || row >= s->max_rows) return fail(s, QPB_ERR_INVALID, "row out of range");
  DeviceGuard g(s->device);
  QPB_CUDA(s, cudaDeviceSynchronize());
  unsigned int drawn = 0;
  QPB_CUDA(s, cudaMemcpy(h_state313, s->d_rng + (size_t)row * MT_N, sizeof(uint64_t) * MT_N, cudaMemcpyDeviceToHost));
  QPB_CUDA(s, cudaMemcpy(&drawn, s->d_drawn + row, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  h_state313[MT_N] = drawn;
  return QPB_OK;
}

int qpb_sampler_rng_set(qpb_sampler *s, int row, const uint64_t *h_state313) {
  if (!s) return QPB_ERR_INVALID;
  if (!h_state313 || row < 0 || row >= s->max_rows) return fail(s, QPB_ERR_INVALID, "row out of range");
  DeviceGuard g(s->device);
  QPB_CUDA(s, cudaDeviceSynchronize());
  const unsigned int drawn = (unsigned int)h_state313[MT_N];
  QPB_CUDA(s, cudaMemcpy(s->d_rng + (size_t)row * MT_N, h_state313, sizeof(uint64_t) * MT_N, cudaMemcpyHostToDevice));
  QPB_CUDA(s, cudaMemcpy(s->d_drawn + row, &drawn, sizeof(unsigned int), cudaMemcpyHostToDevice));
  return QPB_OK;
}

int qpb_sampler_set_cluster(qpb_sampler *s, int cluster) {
  if (!s) return QPB_ERR_INVALID;
  if (cluster < 0 || cluster > 8) return fail(s, QPB_ERR_INVALID, "cluster must be 0 (automatic) or 1..8");
  s->cluster = cluster;
  return QPB_OK;
}

int qpb_sampler_phase_clocks(qpb_sampler *s, int enable, long long *h_clk, int n_rows) {
  if (!s) return QPB_ERR_INVALID;
  DeviceGuard g(s->device);
  if (enable && !s->d_phase_clk) {
    QPB_CUDA(s, cudaMalloc(&s->d_phase_clk, sizeof(long long) * 16 * (size_t)s->max_rows));
    QPB_CUDA(s, cudaMemset(s->d_phase_clk, 0, sizeof(long long) * 16 * (size_t)s->max_rows));
  }
  if (h_clk && s->d_phase_clk) {
    if (n_rows < 1 || n_rows > s->max_rows) return fail(s, QPB_ERR_INVALID, "n_rows outside [1, max_rows]");
    QPB_CUDA(s, cudaDeviceSynchronize());
    QPB_CUDA(s, cudaMemcpy(h_clk, s->d_phase_clk, sizeof(long long) * 16 * (size_t)n_rows, cudaMemcpyDeviceToHost));
  }
  if (!enable && s->d_phase_clk) {
    QPB_CUDA(s, cudaDeviceSynchronize());
    cudaFree(s->d_phase_clk);
    s->d_phase_clk = nullptr;
  }
  return QPB_OK;
}

int64_t qpb_sampler_launch_count(const qpb_sampler *s) { return s ? s->launches : 0; }

const char *qpb_sampler_last_error(const qpb_sampler *s) { return s ? s->err.c_str() : "null handle"; }

int qpb_sampler_cand_slots(qpb_sampler *s, int vocab_total, int vocab_local_max, int *slots) {
  if (!s || !slots) return QPB_ERR_INVALID;
  if (s->n_params == 0) return fail(s, QPB_ERR_INVALID, "qpb_sampler_set_params has not been called");
  long long m = 1;
  for (const auto &p : s->h_params) {
    long long b = row_budget(p, vocab_total);
    if (b > kSmallMaxM) return fail(s, QPB_ERR_UNSUPPORTED, "vocab-sharded rows need top_k + window <= 500");
    if (b >= vocab_total / 4) b = vocab_total;
    if (b > m) m = b;
  }
  if (m > vocab_local_max) m = vocab_local_max;
  *slots = (int)m;
  return QPB_OK;
}

int qpb_sampler_local_candidates(qpb_sampler *s, const float *d_logits, int64_t row_stride, int n_rows,
                                 int vocab_local, int vocab_total, int id_offset, const int32_t *d_history,
                                 int64_t hist_stride, const int32_t *d_hist_len, int hist_len_all, uint64_t *d_cand,
                                 int slots, void *stream) {
  if (!s) return QPB_ERR_INVALID;
  if (!d_cand || slots <= 0 || id_offset < 0 || id_offset + vocab_local > vocab_total)
    return fail(s, QPB_ERR_INVALID, "candidate buffer / shard range invalid");
  Inputs in{d_logits, row_stride, n_rows, vocab_local, vocab_total, id_offset, d_history, hist_stride, d_hist_len, hist_len_all};
  int rc = check_inputs(s, in, true);
  if (rc) return rc;
  DeviceGuard g(s->device);
  rc = route_rows(s, n_rows, vocab_total, d_history ? hist_stride : 0, (cudaStream_t)stream);
  if (rc) return rc;
  if (s->n_whole > 0) return fail(s, QPB_ERR_UNSUPPORTED, "vocab-sharded rows need top_k + window <= 500");
  StreamArgs a = {};
  fill_common(s, in, a);
  a.n_rows = n_rows;
  a.cand_io = reinterpret_cast<unsigned long long *>(d_cand);
  a.cand_slots = slots;
  a.cand_rows = n_rows;
  return launch_stream<MODE_LOCAL_TOPM>(s, a, n_rows, pick_cluster(s, n_rows), (cudaStream_t)stream);
}

int qpb_sampler_merge_sample(qpb_sampler *s, const uint64_t *d_cand_all, int n_shards, int n_rows, int slots,
                             int vocab_total, const int32_t *d_history, int64_t hist_stride,
                             const int32_t *d_hist_len, int hist_len_all, int32_t *d_dist_ids, float *d_dist_p,
                             int32_t *d_dist_count, int max_out, int32_t *d_out_ids, void *stream) {
  if (!s) return QPB_ERR_INVALID;
  if (!d_cand_all || n_shards <= 0 || slots <= 0) return fail(s, QPB_ERR_INVALID, "candidate buffer invalid");
  if ((long long)n_shards * slots > kMergeCap) return fail(s, QPB_ERR_UNSUPPORTED, "n_shards * slots exceeds 8192");
  if (!d_out_ids && !d_dist_count) return fail(s, QPB_ERR_INVALID, "no output requested");
  Inputs in{nullptr, 0, n_rows, vocab_total, vocab_total, 0, d_history, hist_stride, d_hist_len, hist_len_all};
  int rc = check_inputs(s, in, false);
  if (rc) return rc;
  DeviceGuard g(s->device);
  rc = route_rows(s, n_rows, vocab_total, d_history ? hist_stride : 0, (cudaStream_t)stream);
  if (rc) return rc;
  if (s->n_whole > 0) return fail(s, QPB_ERR_UNSUPPORTED, "vocab-sharded rows need top_k + window <= 500");
  StreamArgs a = {};
  fill_common(s, in, a);
  a.n_rows = n_rows;
  a.cand_io = const_cast<unsigned long long *>(reinterpret_cast<const unsigned long long *>(d_cand_all));
  a.cand_slots = slots;
  a.cand_rows = n_rows;
  a.n_shards = n_shards;
  a.out_ids = d_out_ids;
  a.draw = d_out_ids ? 1 : 0;
  a.dist_ids = max_out > 0 ? d_dist_ids : nullptr;
  a.dist_p = d_dist_p;
  a.dist_count = d_dist_count;
  a.max_out = max_out;
  return launch_stream<MODE_MERGE>(s, a, n_rows, 1, (cudaStream_t)stream);
}

__global__ void debug_expf_kernel(const float *x, float *out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = expf_libm(x[i]);
}

int qpb_debug_expf(const float *d_x, float *d_out, int n, void *stream) {
  if (!d_x || !d_out || n <= 0) return QPB_ERR_INVALID;
  debug_expf_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(d_x, d_out, n);
  return cudaGetLastError() == cudaSuccess ? QPB_OK : QPB_ERR_CUDA;
}

}  // extern "C"
