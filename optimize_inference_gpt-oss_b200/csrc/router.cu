// Router top-k + softmax (gptoss_router_topk).
//
// One warp per row.  Lane l holds experts l, l + 32, ... (at most 8 of them for
// E <= 256) as order-preserving 32-bit keys; each of the k rounds picks the
// warp-wide maximum key with redux.sync, then the lowest expert number among
// the lanes that hold it, so equal scores resolve to the lower expert exactly
// as a stable descending sort does.  The softmax over the k winners repeats the
// CPU's rounding sequence (double maximum and sum, glibc's expf, one division).
// The kernel moves a few hundred bytes per row: it is latency-bound, and short.
#include "common.cuh"
#include "exact_math.cuh"

namespace gptoss {
namespace {

constexpr int kRowsPerBlock = 8; // warps per block

// Key that orders like the float: larger value, larger key; -0 and +0 share a
// key; NaN gets the smallest key so it is never taken ahead of a number.
__device__ __forceinline__ uint32_t order_key(float v) {
  if (v != v)
    return 0u;
  uint32_t u = v == 0.0f ? 0u : __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// kSlots = experts per lane = ceil(E / 32), a template parameter so that the
// common E = 32 case scans one value per lane instead of eight predicated ones.
template <typename LT, int kSlots>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
    router_rows(const LT *__restrict__ logits, int E, int k, float *__restrict__ topk_w,
                int *__restrict__ topk_e, int T, const int *__restrict__ done,
                const int *__restrict__ slot_of) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= T)
    return;
  const LT *r = logits + (size_t)row * E;
  float val[kSlots];
  uint32_t key[kSlots];
#pragma unroll
  for (int j = 0; j < kSlots; j++) {
    const int e = lane + 32 * j;
    val[j] = e < E ? load1(r + e) : 0.0f;
    key[j] = e < E ? order_key(val[j]) : 0u;
  }
  const bool finished = done && done[row] != 0;
  unsigned taken = 0; // bit j: this lane's expert lane + 32 j was picked already
  float my_val = 0.0f;
  int my_e = 0;
  for (int round = 0; round < k; round++) {
    // this lane's best remaining expert: largest key, lowest slot on ties
    uint32_t bk = 0u;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kSlots; j++) {
      const int e = lane + 32 * j;
      const bool free_slot = e < E && !((taken >> j) & 1u);
      if (free_slot && (be == 0x7fffffff || key[j] > bk)) {
        bk = key[j];
        be = e;
      }
    }
    const uint32_t top = __reduce_max_sync(0xffffffffu, bk);
    // among lanes whose best equals the maximum, the lowest expert number
    const unsigned cand = (be != 0x7fffffff && bk == top) ? (unsigned)be : 0x7fffffffu;
    const int win = (int)__reduce_min_sync(0xffffffffu, cand);
    if ((win & 31) == lane && win == be)
      taken |= 1u << (win >> 5);
    // the winner's value, from the lane that owns it
    float wv = 0.0f;
#pragma unroll
    for (int j = 0; j < kSlots; j++)
      if ((win >> 5) == j)
        wv = val[j];
    wv = __shfl_sync(0xffffffffu, wv, win & 31);
    if (lane == round) {
      my_val = wv;
      my_e = win;
    }
  }
  if (finished) {
    if (lane < k) {
      topk_w[(size_t)row * k + lane] = 0.0f;
      topk_e[(size_t)row * k + lane] = -1;
    }
    return;
  }
  // softmax over the k picks, lane j owning pick j (run.cpp:335-353)
  double top = (double)__shfl_sync(0xffffffffu, my_val, 0);
  for (int j = 1; j < k; j++) {
    const float v = __shfl_sync(0xffffffffu, my_val, j);
    if ((double)v > top)
      top = (double)v;
  }
  const float ex = glibc_expf((float)__dsub_rn((double)my_val, top));
  double total = 0.0;
  for (int j = 0; j < k; j++)
    total = __dadd_rn(total, (double)__shfl_sync(0xffffffffu, ex, j));
  if (lane < k) {
    topk_w[(size_t)row * k + lane] = (float)__ddiv_rn((double)ex, total);
    topk_e[(size_t)row * k + lane] = slot_of ? slot_of[my_e] : my_e;
  }
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_router_topk(gptoss_stream_t stream, int T, const void *logits,
                                  gptoss_dtype_t logits_dtype, int E, int k, float *topk_w,
                                  int *topk_e, const int *done, const int *slot_of,
                                  unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (T < 0 || E <= 0 || k <= 0 || k > E || !valid_dtype(logits_dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (E > GPTOSS_MAX_EXPERTS || k > GPTOSS_MAX_TOPK)
    return GPTOSS_ERR_UNSUPPORTED;
  if (T == 0)
    return GPTOSS_OK;
  if (!logits || !topk_w || !topk_e)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(logits, (size_t)T * E * dtype_size(logits_dtype));
  GPTOSS_SPAN(topk_w, (size_t)T * k * 4);
  GPTOSS_SPAN(topk_e, (size_t)T * k * 4);
  GPTOSS_SPAN(done, (size_t)T * 4);
  GPTOSS_SPAN(slot_of, (size_t)E * 4);
  const int grid = (T + kRowsPerBlock - 1) / kRowsPerBlock;
  cudaStream_t s = as_stream(stream);
  const int slots = (E + 31) / 32;
#define GPTOSS_ROUTER_CASE(LT_, SLOTS_)                                                           \
  launch_kernel(router_rows<LT_, SLOTS_>, dim3(grid), dim3(kRowsPerBlock * 32), 0, s,             \
                static_cast<const LT_ *>(logits), E, k, topk_w, topk_e, T, done, slot_of)
  if (logits_dtype == GPTOSS_F32) {
    if (slots <= 1)
      GPTOSS_ROUTER_CASE(float, 1);
    else if (slots <= 2)
      GPTOSS_ROUTER_CASE(float, 2);
    else if (slots <= 4)
      GPTOSS_ROUTER_CASE(float, 4);
    else
      GPTOSS_ROUTER_CASE(float, 8);
  } else {
    if (slots <= 1)
      GPTOSS_ROUTER_CASE(uint16_t, 1);
    else if (slots <= 2)
      GPTOSS_ROUTER_CASE(uint16_t, 2);
    else if (slots <= 4)
      GPTOSS_ROUTER_CASE(uint16_t, 4);
    else
      GPTOSS_ROUTER_CASE(uint16_t, 8);
  }
#undef GPTOSS_ROUTER_CASE
  return launch_status();
}
