// Host-side helpers behind include/gptoss_engine.h: CUDA runtime wrappers for
// buffers, streams and events; the RoPE table builder; the seeded synthetic
// tensor generator.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/gptoss_engine.h"
#include "common.cuh"

namespace gptoss {

int cuda_status(cudaError_t e) {
  if (e == cudaSuccess)
    return GPTOSS_OK;
  note_cuda_error(e);
  (void)cudaGetLastError(); // clear the sticky "last error" so later launches are judged on their own
  return GPTOSS_ERR_CUDA;
}

int host_threads(int requested) {
  if (requested > 0)
    return requested;
  const unsigned n = std::thread::hardware_concurrency();
  return n ? (int)n : 1;
}

// Runs fn(begin, end) over [0, count) cut into contiguous pieces, one per thread.
template <typename F> void parallel_ranges(size_t count, size_t align, int threads, F fn) {
  threads = host_threads(threads);
  size_t per = (count + threads - 1) / threads;
  per = (per + align - 1) / align * align;
  if (threads == 1 || count <= per) {
    fn((size_t)0, count);
    return;
  }
  std::vector<std::thread> pool;
  for (size_t b = 0; b < count; b += per)
    pool.emplace_back(fn, b, std::min(count, b + per));
  for (auto &t : pool)
    t.join();
}

__global__ void flush_kernel(uint4 *p, size_t n, unsigned v) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    p[i] = make_uint4(v, v, v, v);
}

// splitmix64 finaliser.
static inline uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

static inline uint16_t to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u)
    return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// Standard normals 2i and 2i+1 of a stream come from counter i.
static inline void normal_pair(uint64_t key, uint64_t i, float &a, float &b) {
  const uint64_t h = mix64(key + i * 0xd1342543de82ef95ull);
  const float u1 = ((float)(uint32_t)(h >> 40) + 0.5f) * (1.0f / 16777216.0f); // (0,1)
  const float u2 = (float)(uint32_t)((h >> 8) & 0xffffffu) * (1.0f / 16777216.0f); // [0,1)
  const float r = sqrtf(-2.0f * logf(u1));
  float s, c;
  sincosf(6.28318530717958647692f * u2, &s, &c);
  a = r * c;
  b = r * s;
}

} // namespace gptoss

using namespace gptoss;

extern "C" {

int gptoss_device_count(int *count) {
  if (!count)
    return GPTOSS_ERR_BAD_ARG;
  *count = 0;
  const cudaError_t e = cudaGetDeviceCount(count);
  if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) {
    *count = 0;
    (void)cudaGetLastError();
    return GPTOSS_OK;
  }
  return cuda_status(e);
}

int gptoss_device_set(int device) { return cuda_status(cudaSetDevice(device)); }

int gptoss_device_name(int device, char *buf, int buf_len) {
  if (!buf || buf_len <= 0)
    return GPTOSS_ERR_BAD_ARG;
  cudaDeviceProp p;
  const int st = cuda_status(cudaGetDeviceProperties(&p, device));
  if (st != GPTOSS_OK)
    return st;
  strncpy(buf, p.name, (size_t)buf_len - 1);
  buf[buf_len - 1] = 0;
  return GPTOSS_OK;
}

int gptoss_device_alloc(void **ptr, size_t bytes) {
  if (!ptr)
    return GPTOSS_ERR_BAD_ARG;
  *ptr = nullptr;
  const int st = cuda_status(cudaMalloc(ptr, bytes ? bytes : 1));
  if (st == GPTOSS_OK)
    bounds_register(*ptr, bytes ? bytes : 1);
  return st;
}

int gptoss_device_free(void *ptr) {
  bounds_unregister(ptr);
  return cuda_status(cudaFree(ptr));
}

int gptoss_device_memset(void *ptr, int byte, size_t bytes, gptoss_stream_t stream) {
  if (!ptr && bytes)
    return GPTOSS_ERR_BAD_ARG;
  return cuda_status(cudaMemsetAsync(ptr, byte, bytes, as_stream(stream)));
}

int gptoss_upload(void *dst, const void *src, size_t bytes, gptoss_stream_t stream) {
  if ((!dst || !src) && bytes)
    return GPTOSS_ERR_BAD_ARG;
  return cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
}

int gptoss_download(void *dst, const void *src, size_t bytes, gptoss_stream_t stream) {
  if ((!dst || !src) && bytes)
    return GPTOSS_ERR_BAD_ARG;
  return cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
}

int gptoss_host_alloc_pinned(void **ptr, size_t bytes) {
  if (!ptr)
    return GPTOSS_ERR_BAD_ARG;
  *ptr = nullptr;
  return cuda_status(cudaMallocHost(ptr, bytes ? bytes : 1));
}

int gptoss_host_free_pinned(void *ptr) { return cuda_status(cudaFreeHost(ptr)); }

int gptoss_stream_create(gptoss_stream_t *stream) {
  if (!stream)
    return GPTOSS_ERR_BAD_ARG;
  cudaStream_t s = nullptr;
  const int st = cuda_status(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return st;
}

int gptoss_stream_destroy(gptoss_stream_t stream) {
  return cuda_status(cudaStreamDestroy(as_stream(stream)));
}

int gptoss_stream_synchronize(gptoss_stream_t stream) {
  return cuda_status(cudaStreamSynchronize(as_stream(stream)));
}

int gptoss_device_synchronize(void) { return cuda_status(cudaDeviceSynchronize()); }

int gptoss_event_create(gptoss_event_t *event) {
  if (!event)
    return GPTOSS_ERR_BAD_ARG;
  cudaEvent_t e = nullptr;
  const int st = cuda_status(cudaEventCreate(&e));
  *event = e;
  return st;
}

int gptoss_event_destroy(gptoss_event_t event) {
  return cuda_status(cudaEventDestroy((cudaEvent_t)event));
}

int gptoss_event_record(gptoss_event_t event, gptoss_stream_t stream) {
  return cuda_status(cudaEventRecord((cudaEvent_t)event, as_stream(stream)));
}

int gptoss_event_synchronize(gptoss_event_t event) {
  return cuda_status(cudaEventSynchronize((cudaEvent_t)event));
}

int gptoss_event_elapsed_ms(gptoss_event_t start, gptoss_event_t stop, float *ms) {
  if (!ms)
    return GPTOSS_ERR_BAD_ARG;
  return cuda_status(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
}

int gptoss_flush_l2(void *scratch, size_t bytes, gptoss_stream_t stream) {
  if (!scratch || bytes < 16 || !aligned16(scratch))
    return GPTOSS_ERR_BAD_ARG;
  static unsigned salt = 0;
  launch_kernel(flush_kernel, dim3(sm_count() * 4), dim3(512), 0, as_stream(stream), (uint4 *)scratch, bytes / 16,
                ++salt);
  return launch_status();
}

// Stream capture into an executable graph: what the chain driver does for a whole step, for
// callers (and the benchmark) that want to replay a few launches of their own without the
// per-launch host cost.
int gptoss_graph_begin(gptoss_stream_t stream) {
  return cuda_status(cudaStreamBeginCapture(as_stream(stream), cudaStreamCaptureModeThreadLocal));
}
int gptoss_graph_end(gptoss_stream_t stream, gptoss_graph_t *graph) {
  if (!graph)
    return GPTOSS_ERR_BAD_ARG;
  *graph = nullptr;
  cudaGraph_t g = nullptr;
  int st = cuda_status(cudaStreamEndCapture(as_stream(stream), &g));
  if (st != GPTOSS_OK || !g)
    return st != GPTOSS_OK ? st : GPTOSS_ERR_CUDA;
  cudaGraphExec_t exec = nullptr;
  st = cuda_status(cudaGraphInstantiate(&exec, g, 0));
  (void)cudaGraphDestroy(g);
  if (st == GPTOSS_OK)
    *graph = exec;
  return st;
}
int gptoss_graph_launch(gptoss_graph_t graph, gptoss_stream_t stream) {
  if (!graph)
    return GPTOSS_ERR_BAD_ARG;
  return cuda_status(cudaGraphLaunch((cudaGraphExec_t)graph, as_stream(stream)));
}
int gptoss_graph_destroy(gptoss_graph_t graph) {
  return graph ? cuda_status(cudaGraphExecDestroy((cudaGraphExec_t)graph)) : GPTOSS_OK;
}

int gptoss_build_rope_tables(int n_pos, int head_dim, float theta, float factor, float orig_ctx,
                             float beta_fast, float beta_slow, float *cos_host, float *sin_host) {
  if (n_pos <= 0 || head_dim <= 0 || head_dim % 2 != 0 || !cos_host || !sin_host || !(theta > 1.0f))
    return GPTOSS_ERR_BAD_ARG;
  const int half = head_dim / 2;
  // Per-pair rotation rate and the YaRN amplitude; float arithmetic throughout
  // except the division by 2*pi*beta, which the CPU program does in double.
  std::vector<float> rate(half);
  float amplitude = 1.0f;
  if (factor > 1.0f) {
    amplitude = 0.1f * logf(factor) + 1.0f;
    const float ln_theta = logf(theta);
    const float lo = (float)half * logf((float)((double)orig_ctx / ((double)(beta_fast * 2.0f) * M_PI))) / ln_theta;
    const float hi = (float)half * logf((float)((double)orig_ctx / ((double)(beta_slow * 2.0f) * M_PI))) / ln_theta;
    if (!(0 < lo && lo < hi && hi < half - 1))
      return GPTOSS_ERR_BAD_ARG; // the CPU program asserts the same
    for (int i = 0; i < half; i++) {
      const float f = powf(theta, ((float)(2 * i)) / (float)head_dim);
      const float scaled = 1.0f / (factor * f), plain = 1.0f / f;
      float ramp = ((float)i - lo) / (hi - lo);
      ramp = ramp < 0 ? 0 : (ramp > 1 ? 1 : ramp);
      const float keep = 1.0f - ramp;
      rate[i] = scaled * (1.0f - keep) + plain * keep;
    }
  } else {
    for (int i = 0; i < half; i++)
      rate[i] = 1.0f / powf(theta, ((float)(2 * i)) / (float)head_dim);
  }
  parallel_ranges((size_t)n_pos, 1, 0, [&](size_t b, size_t e) {
    for (size_t p = b; p < e; p++)
      for (int j = 0; j < half; j++) {
        const float angle = (float)(int)p * rate[j];
        cos_host[p * half + j] = cosf(angle) * amplitude;
        sin_host[p * half + j] = sinf(angle) * amplitude;
      }
  });
  return GPTOSS_OK;
}

int gptoss_synth_normal(void *dst, gptoss_dtype_t dtype, size_t count, uint64_t seed,
                        uint64_t stream_id, float mean, float sd, int threads) {
  if ((!dst && count) || !valid_dtype(dtype))
    return GPTOSS_ERR_BAD_ARG;
  const uint64_t key = mix64(seed ^ mix64(stream_id * 0x9e3779b97f4a7c15ull + 0x1234567ull));
  parallel_ranges(count, 2, threads, [=](size_t b, size_t e) {
    for (size_t j = b; j < e; j += 2) {
      float a, c;
      normal_pair(key, j >> 1, a, c);
      a = mean + sd * a;
      c = mean + sd * c;
      if (dtype == GPTOSS_F32) {
        float *p = (float *)dst;
        p[j] = a;
        if (j + 1 < e)
          p[j + 1] = c;
      } else {
        uint16_t *p = (uint16_t *)dst;
        p[j] = to_bf16(a);
        if (j + 1 < e)
          p[j + 1] = to_bf16(c);
      }
    }
  });
  return GPTOSS_OK;
}

int gptoss_synth_uniform_int(int *dst, size_t count, uint64_t seed, uint64_t stream_id, int lo,
                             int hi) {
  if ((!dst && count) || hi <= lo)
    return GPTOSS_ERR_BAD_ARG;
  const uint64_t key = mix64(seed ^ mix64(stream_id * 0x9e3779b97f4a7c15ull + 0x7654321ull));
  const uint64_t span = (uint64_t)((long)hi - (long)lo);
  for (size_t j = 0; j < count; j++) {
    const uint64_t h = mix64(key + j * 0xd1342543de82ef95ull);
    dst[j] = lo + (int)(((h >> 32) * span) >> 32);
  }
  return GPTOSS_OK;
}

} // extern "C"
