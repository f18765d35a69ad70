/*
 * gptoss_argmax_key.cuh -- the device-side half of the greedy-argmax merge, for
 * kernels that produce logits and do not want to write them out.
 *
 * The reference fuses the greedy pick into its LM-head GEMM epilogue: every
 * output tile folds its values into one 64-bit word per row with atomicMax and
 * the 412 MB of logits are never stored (kernels/fast_gemm.hpp:94-104
 * `argmax_key`, :367-417 `argmax_rows`, :706-714 `argmax_keys_kernel`).  This
 * header is that contract for a CUDA producer (for instance an sm_100 GEMM
 * epilogue): include it, call gptoss_argmax_fold() for every (row, column,
 * value) the kernel computes, then let gptoss_argmax_keys_finish()
 * (gptoss_kernels.h) turn the words into token ids.
 *
 * The key orders like the value, then like the complemented column: the
 * largest key of a row names the column greedy decoding picks -- the largest
 * value, the lowest column among equal values, -0 equal to +0.  A NaN maps to
 * key 0 and can never win.  keys[] must be zero before the producer runs;
 * gptoss_argmax_keys_finish() leaves it zero again.
 */
#ifndef GPTOSS_ARGMAX_KEY_CUH
#define GPTOSS_ARGMAX_KEY_CUH

#include <stdint.h>

/* Key of value x in column col (col < 2^31). */
__device__ __forceinline__ unsigned long long gptoss_argmax_key(float x, unsigned col) {
  if (x != x)
    return 0ull;
  uint32_t u = x == 0.0f ? 0u : __float_as_uint(x);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned)~col;
}

/* The better of two keys (for reductions inside a warp or block before the atomic). */
__device__ __forceinline__ unsigned long long gptoss_argmax_better(unsigned long long a,
                                                                   unsigned long long b) {
  return a > b ? a : b;
}

/* Folds a (partial) result into the row's word in global memory. */
__device__ __forceinline__ void gptoss_argmax_fold(unsigned long long *keys, int row,
                                                   unsigned long long key) {
  if (key)
    atomicMax(keys + row, key);
}

/* Column named by a merged key; 0 when nothing was folded in (an all-NaN row). */
__device__ __forceinline__ int gptoss_argmax_column(unsigned long long key) {
  return key ? (int)~(uint32_t)(key & 0xffffffffull) : 0;
}

#endif /* GPTOSS_ARGMAX_KEY_CUH */
