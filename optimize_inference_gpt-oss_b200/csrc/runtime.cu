// Library-wide host helpers: version, status text, per-thread CUDA error memory,
// cached device properties.
#include "common.cuh"

namespace gptoss {

static thread_local int g_last_cuda_error = 0;

void note_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
    return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

} // namespace gptoss

extern "C" const char *gptoss_version(void) { return "0.1.0"; }

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
