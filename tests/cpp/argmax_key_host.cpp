// include/gptoss_argmax_key.cuh compiled for the host, so that a CPU test can hold its key
// formula against the reference's (tests/test_oracle_pins.py).  The CUDA qualifiers and the two
// device functions the header uses get plain C++ meanings; the atomic fold is not called.
#include <stdint.h>
#include <string.h>
#define __device__
#define __forceinline__ inline
static inline uint32_t __float_as_uint(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  return u;
}
static inline unsigned long long atomicMax(unsigned long long *at, unsigned long long v) {
  const unsigned long long old = *at;
  if (v > old)
    *at = v;
  return old;
}
#include "gptoss_argmax_key.cuh"

extern "C" void host_argmax_keys(long n, const float *x, const int *col, unsigned long long *keys) {
  for (long i = 0; i < n; i++)
    keys[i] = gptoss_argmax_key(x[i], (unsigned)col[i]);
}
extern "C" void host_argmax_columns(long n, const unsigned long long *keys, int *col) {
  for (long i = 0; i < n; i++)
    col[i] = gptoss_argmax_column(keys[i]);
}
