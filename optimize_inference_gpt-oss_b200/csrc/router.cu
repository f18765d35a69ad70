// Router top-k + softmax (gptoss_router_topk).
//
// One warp per row.  Lane l holds experts l, l + 32, ... (at most 8 of them for
// E <= 256) as order-preserving 32-bit keys; each of the k rounds picks the
// warp-wide maximum key with redux.sync, then the lowest expert number among
// the lanes that hold it, so equal scores resolve to the lower expert exactly
// as a stable descending sort does.  The softmax over the k winners repeats the
// CPU's rounding sequence (double maximum and sum, glibc's expf, one division).
// The kernel moves a few hundred bytes per row: it is latency-bound, and short.
//
// The model family's shapes (k = 4; E = 32 or 128) have a kernel of their own,
// router_rows_top4, with a shorter dependent chain, which is all this kernel's time is: lane
// l holds experts S l .. S l + S - 1 (one vector load); with bf16 scores key and expert number
// share a 32-bit word, so a round is one redux and the winner's value comes back out of the
// key; the rounds are unrolled; and the table of the exact expf is fetched together with the
// scores, one entry per lane, and looked up by shuffle instead of by a dependent load in the
// middle of the softmax.  On B200, behind the programmatic-launch attribute: 2.0 us per launch
// instead of 2.7 at 512 rows, 3.0 instead of 3.9 at 4096 (E = 32); 3.3 instead of 5.5 at 4096
// rows of 128 experts.  Same bits as the general kernel.
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

// ---- k = 4, E = 32 * S -------------------------------------------------------------------

// Rows per warp (their rounds interleave, and one pass of the softmax serves them all, lane
// 4 r + j owning pick j of row r).  More rows per warp mean fewer instructions per row and a
// longer chain per warp; measured in the 24-layer chain on B200, 1 and 2 are level, 4 is 0.4 us
// per launch slower at 512 rows (level at 4096), 8 is 1.2-1.8 us slower everywhere.
constexpr int kTop4Rows = 1;
constexpr int kTop4Warps = 8; // warps per block: 4 measured level, 2 and 1 slower at 4096 rows (3.4 and 4.4 us per launch)

// Keys for this kernel: every score's key is at least 1 (NaN: 1, below -inf), so 0 can stand
// for "taken" and for rows past the end.  -0 and +0 share a key; value_of_key gives +0 back
// for both, which the softmax cannot tell apart (exp(x - top) is the same for either zero).
__device__ __forceinline__ uint32_t key32(float v) {
  const uint32_t u = __float_as_uint(v);
  if ((u & 0x7fffffffu) > 0x7f800000u)
    return 1u;
  if ((u & 0x7fffffffu) == 0u)
    return 0x80000000u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float value_of_key32(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
// bf16 bits (low 16 of b) -> 16-bit key, same rules
__device__ __forceinline__ uint32_t key16(uint32_t b) {
  b &= 0xffffu;
  if ((b & 0x7fffu) > 0x7f80u)
    return 1u;
  if ((b & 0x7fffu) == 0u)
    return 0x8000u;
  return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
}
__device__ __forceinline__ float value_of_key16(uint32_t key) {
  const uint32_t b = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
  return __uint_as_float(b << 16);
}

template <typename LT, int S>
__global__ void __launch_bounds__(kTop4Warps * 32)
    router_rows_top4(const LT *__restrict__ logits, float *__restrict__ topk_w, int *__restrict__ topk_e, int T,
                     const int *__restrict__ done, const int *__restrict__ slot_of) {
  constexpr int E = 32 * S;
  constexpr bool kPacked = sizeof(LT) == 2; // bf16: key << 16 | (0xffff - expert) in one word
  constexpr unsigned kAll = 0xffffffffu;
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x * kTop4Warps + (threadIdx.x >> 5)) * kTop4Rows;
  if (row0 >= T)
    return; // the whole warp
  // Lane l keeps experts S l .. S l + S - 1 of each of the warp's rows, entry l of the expf table,
  // and (the lanes that own a pick) the finished flag of row l / 4: everything the warp reads,
  // asked for at once.
  const unsigned long long tab = kExp2Tab32[lane];
  const int my_row = row0 + (lane >> 2);
  const bool writes = lane < 4 * kTop4Rows && my_row < T;
  const int fin = (done && writes) ? done[my_row] : 0;
  uint32_t key[kTop4Rows][S];
#pragma unroll
  for (int r = 0; r < kTop4Rows; r++) {
    const bool live = row0 + r < T;
    const LT *src = logits + (size_t)(live ? row0 + r : row0) * E + lane * S;
    if constexpr (kPacked) {
      uint32_t b[S];
      if constexpr (S == 4) {
        const uint2 q = *reinterpret_cast<const uint2 *>(src);
        b[0] = q.x, b[1] = q.x >> 16, b[2] = q.y, b[3] = q.y >> 16;
      } else {
        static_assert(S == 1, "one or four experts per lane");
        b[0] = *src;
      }
#pragma unroll
      for (int j = 0; j < S; j++)
        key[r][j] = live ? (key16(b[j]) << 16) | (0xffffu - (unsigned)(lane * S + j)) : 0u;
    } else {
      float v[S];
      if constexpr (S == 4) {
        const float4 q = *reinterpret_cast<const float4 *>(src);
        v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
      } else {
        static_assert(S == 1, "one or four experts per lane");
        v[0] = *src;
      }
#pragma unroll
      for (int j = 0; j < S; j++)
        key[r][j] = live ? key32(v[j]) : 0u;
    }
  }
  // Four rounds; in each, the rows' reductions are independent of one another.  Lane
  // 4 r + round keeps row r's pick of that round.
  uint32_t my_key = 0u, my_e = 0u;
#pragma unroll
  for (int round = 0; round < 4; round++) {
#pragma unroll
    for (int r = 0; r < kTop4Rows; r++) {
      uint32_t best = key[r][0];
#pragma unroll
      for (int j = 1; j < S; j++)
        best = max(best, key[r][j]);
      const uint32_t top = __reduce_max_sync(kAll, best);
      if constexpr (kPacked) { // packed words are distinct within a row: the maximum names its slot
#pragma unroll
        for (int j = 0; j < S; j++)
          key[r][j] = key[r][j] == top ? 0u : key[r][j];
        if (lane == 4 * r + round)
          my_key = top;
      } else { // the lowest expert number among the slots that hold the maximum
        uint32_t cand = 0xffffffffu;
#pragma unroll
        for (int j = S - 1; j >= 0; j--)
          cand = key[r][j] == top ? (unsigned)(lane * S + j) : cand;
        const uint32_t win = __reduce_min_sync(kAll, cand);
#pragma unroll
        for (int j = 0; j < S; j++)
          key[r][j] = (unsigned)(lane * S + j) == win ? 0u : key[r][j];
        if (lane == 4 * r + round)
          my_key = top, my_e = win;
      }
    }
  }
  float v;
  if constexpr (kPacked) {
    v = value_of_key16(my_key >> 16);
    my_e = 0xffffu - (my_key & 0xffffu);
  } else {
    v = value_of_key32(my_key);
  }
  // softmax over each row's four picks (lanes 4 r .. 4 r + 3; the first is the largest), in the
  // CPU's rounding sequence (run.cpp:335-353).  The lanes past the last pick run along on zeros.
  const int first = lane & ~3;
  const double top_v = (double)__shfl_sync(kAll, v, first);
  const uint32_t tab_lo = (uint32_t)tab, tab_hi = (uint32_t)(tab >> 32);
  const float ex = glibc_expf_with<true>((float)__dsub_rn((double)v, top_v), [&](uint32_t i) {
    const uint32_t lo = __shfl_sync(kAll, tab_lo, (int)i), hi = __shfl_sync(kAll, tab_hi, (int)i);
    return ((unsigned long long)hi << 32) | lo;
  });
  double total = 0.0;
#pragma unroll
  for (int j = 0; j < 4; j++)
    total = __dadd_rn(total, (double)__shfl_sync(kAll, ex, first + j));
  if (!writes)
    return;
  float w = (float)__ddiv_rn((double)ex, total);
  int e = (int)my_e;
  if (fin != 0)
    w = 0.0f, e = -1;
  else if (slot_of)
    e = slot_of[e];
  topk_w[(size_t)row0 * 4 + lane] = w;
  topk_e[(size_t)row0 * 4 + lane] = e;
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
  cudaStream_t s = as_stream(stream);
#ifndef GPTOSS_ROUTER_GENERAL_ONLY
  if (k == 4 && (E == 32 || E == 128)) {
    const size_t lane_bytes = (size_t)(E / 32) * dtype_size(logits_dtype);
    if (reinterpret_cast<uintptr_t>(logits) % lane_bytes == 0) {
      const int rows_per_block = kTop4Rows * kTop4Warps;
      const dim3 grid4((T + rows_per_block - 1) / rows_per_block), block4(kTop4Warps * 32);
#define GPTOSS_TOP4_CASE(LT_, S_)                                                                 \
  launch_kernel(router_rows_top4<LT_, S_>, grid4, block4, 0, s, static_cast<const LT_ *>(logits), \
                topk_w, topk_e, T, done, slot_of)
      if (logits_dtype == GPTOSS_F32) {
        if (E == 32)
          GPTOSS_TOP4_CASE(float, 1);
        else
          GPTOSS_TOP4_CASE(float, 4);
      } else {
        if (E == 32)
          GPTOSS_TOP4_CASE(uint16_t, 1);
        else
          GPTOSS_TOP4_CASE(uint16_t, 4);
      }
#undef GPTOSS_TOP4_CASE
      return launch_status();
    }
  }
#endif
  const int grid = (T + kRowsPerBlock - 1) / kRowsPerBlock;
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
