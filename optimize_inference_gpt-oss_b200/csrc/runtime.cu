// Library-wide host helpers: version, status text, per-thread CUDA error memory,
// cached device properties.
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace gptoss {

static thread_local int g_last_cuda_error = 0;
thread_local bool tl_pdl = false;
thread_local long tl_generic_launches = 0;
thread_local cudaError_t tl_launch_error = cudaSuccess;

void note_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int sm_count() {
  static std::atomic<int> cached[64]; // zero-initialised; threads may race to fill a slot with the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Bounded waits that ran out, per device; kernels get the word's address as an argument.
static __device__ unsigned int g_wait_giveups;

unsigned int *wait_giveups_word() {
  static std::atomic<unsigned int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return nullptr;
  unsigned int *p = cached[dev].load(std::memory_order_acquire);
  if (!p) {
    void *q = nullptr;
    if (cudaGetSymbolAddress(&q, g_wait_giveups) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    p = static_cast<unsigned int *>(q);
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}

#ifdef GPTOSS_BOUNDS
namespace {
struct Span {
  uintptr_t begin, end;
};
std::mutex g_bounds_mu;
Span g_spans[4096];
int g_n_spans = 0;
std::atomic<long> g_host_violations{0}, g_unchecked{0}, g_checked{0};
__device__ unsigned int g_bounds_device_word;
} // namespace

void bounds_register(const void *p, size_t bytes) {
  if (!p)
    return;
  std::lock_guard<std::mutex> lock(g_bounds_mu);
  if (g_n_spans < 4096)
    g_spans[g_n_spans++] = Span{(uintptr_t)p, (uintptr_t)p + bytes};
}
void bounds_unregister(const void *p) {
  std::lock_guard<std::mutex> lock(g_bounds_mu);
  for (int i = 0; i < g_n_spans; i++)
    if (g_spans[i].begin == (uintptr_t)p) {
      g_spans[i] = g_spans[--g_n_spans];
      return;
    }
}
size_t bounds_room(const void *p) {
  std::lock_guard<std::mutex> lock(g_bounds_mu);
  const uintptr_t a = (uintptr_t)p;
  for (int i = 0; i < g_n_spans; i++)
    if (a >= g_spans[i].begin && a < g_spans[i].end)
      return (size_t)(g_spans[i].end - a);
  return SIZE_MAX;
}
bool bounds_span_ok(const void *p, size_t bytes, const char *what) {
  const size_t room = bounds_room(p);
  if (room == SIZE_MAX) {
    g_unchecked++;
    return true;
  }
  g_checked++;
  if (bytes <= room)
    return true;
  g_host_violations++;
  fprintf(stderr, "gptoss bounds: %s needs %zu bytes, its allocation has %zu left\n", what, bytes, room);
  return false;
}
unsigned int *bounds_device_word() {
  static std::atomic<unsigned int *> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return nullptr;
  unsigned int *p = cached[dev].load(std::memory_order_acquire);
  if (!p) {
    void *q = nullptr;
    if (cudaGetSymbolAddress(&q, g_bounds_device_word) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    p = static_cast<unsigned int *>(q);
    cached[dev].store(p, std::memory_order_release);
  }
  return p;
}
#endif

int occupancy_cached(const void *kernel, int threads, size_t smem) {
  struct Entry {
    const void *fn;
    int dev, threads;
    size_t smem;
    int blocks;
  };
  static std::mutex mu;
  static Entry table[512];
  static int used = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess)
    return 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++)
      if (table[i].fn == kernel && table[i].dev == dev && table[i].threads == threads &&
          table[i].smem == smem)
        return table[i].blocks;
  }
  int blocks = 0;
  // Above the 48 KB default the kernel's limit is raised to all the device offers, not to this
  // request: the attribute belongs to the kernel, and a later, smaller request must not lower
  // it under the feet of a configuration that is already in this table.
  // (The limit covers static and dynamic shared memory together, so the dynamic part that can be
  // asked for is the device's figure less the kernel's static arrays.)
  int optin = 0;
  cudaFuncAttributes fa = {};
  if (smem > 48 * 1024 &&
      (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
       cudaFuncGetAttributes(&fa, kernel) != cudaSuccess || smem + fa.sharedSizeBytes > (size_t)optin ||
       cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                            optin - (int)fa.sharedSizeBytes) != cudaSuccess)) {
    (void)cudaGetLastError();
    blocks = 0;
  } else if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, threads, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    blocks = 0;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (used < 512)
    table[used++] = Entry{kernel, dev, threads, smem, blocks};
  return blocks;
}

} // namespace gptoss

extern "C" const char *gptoss_version(void) { return "0.1.0"; }

extern "C" long gptoss_generic_launch_count(void) { return gptoss::tl_generic_launches; }

extern "C" const char *gptoss_status_string(int status) {
  switch (status) {
  case GPTOSS_OK:
    return "ok";
  case GPTOSS_ERR_BAD_ARG:
    return "bad argument (null pointer, negative size or misaligned base)";
  case GPTOSS_ERR_UNSUPPORTED:
    return "shape or dtype not supported by the kernels";
  case GPTOSS_ERR_CUDA:
    return "CUDA error (launch failed or no usable device)";
  default:
    return "unknown status";
  }
}

extern "C" int gptoss_last_cuda_error(void) { return gptoss::g_last_cuda_error; }

extern "C" long gptoss_wait_giveups(void) {
  unsigned int *p = gptoss::wait_giveups_word(), v = 0;
  if (!p || cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  return (long)v;
}

extern "C" int gptoss_bounds_enabled(void) {
#ifdef GPTOSS_BOUNDS
  return 1;
#else
  return 0;
#endif
}

extern "C" long gptoss_bounds_violations(void) {
#ifdef GPTOSS_BOUNDS
  unsigned int *p = gptoss::bounds_device_word(), v = 0;
  if (p && cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  return gptoss::g_host_violations.load() + (long)v;
#else
  return 0;
#endif
}

extern "C" long gptoss_bounds_checked_spans(void) {
#ifdef GPTOSS_BOUNDS
  return gptoss::g_checked.load();
#else
  return 0;
#endif
}
