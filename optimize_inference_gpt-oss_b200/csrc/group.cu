// Grouping of (token, choice) pairs by expert (gptoss_moe_group): the integer
// bookkeeping between the router and the expert GEMMs that also produces the
// row map the combine reads through.
//
// One thread block per local expert, as in the reference.  Thread t owns the
// contiguous run of pairs [t * S, (t + 1) * S); a first pass counts, per
// thread, the pairs of lower local experts (their total is the expert's first
// row) and the pairs of this expert; a block-wide exclusive scan of the latter
// gives every thread the row of its first hit, so a second pass can place the
// hits in pair order.  All data (a few tens of KB of expert ids) is L2-resident;
// the kernel is latency-bound and kept short.
#include "common.cuh"

namespace gptoss {
namespace {

constexpr int kGroupThreads = 256;

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o)
      v += n;
  }
  return v;
}

__global__ void __launch_bounds__(kGroupThreads)
    moe_group_rows(const int *__restrict__ topk_e, int n_pairs, int e_begin, int e_count,
                   int *__restrict__ counts, int *__restrict__ offsets, int *__restrict__ row_pair,
                   int *__restrict__ own_row) {
  pdl_prologue();
  __shared__ int warp_hits[kGroupThreads / 32], warp_below[kGroupThreads / 32];
  const int e = blockIdx.x, ge = e_begin + e;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int per = (n_pairs + kGroupThreads - 1) / kGroupThreads;
  const int p0 = min(t * per, n_pairs), p1 = min(p0 + per, n_pairs);

  int below = 0, hits = 0;
  for (int p = p0; p < p1; p++) {
    const int x = __ldg(topk_e + p);
    below += (x >= e_begin && x < ge);
    hits += (x == ge);
    // pairs of experts held elsewhere (or of finished tokens, expert -1) get no row;
    // each block marks its share so that every such pair is written exactly once
    if ((x < e_begin || x >= e_begin + e_count) && (p % e_count) == e)
      own_row[p] = -1;
  }
  const int incl = warp_inclusive_scan(hits, lane);
  int below_w = below;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    below_w += __shfl_xor_sync(0xffffffffu, below_w, o);
  if (lane == 31)
    warp_hits[warp] = incl;
  if (lane == 0)
    warp_below[warp] = below_w;
  __syncthreads();
  // rows of lower experts; hits of this expert in earlier warps; all hits
  int base = 0, before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kGroupThreads / 32; w++) {
    base += warp_below[w];
    total += warp_hits[w];
    if (w < warp)
      before += warp_hits[w];
  }
  int row = base + before + incl - hits; // row of this thread's first hit
  if (t == 0) {
    counts[e] = total;
    offsets[e] = base;
    if (e == e_count - 1)
      offsets[e_count] = base + total;
  }
  for (int p = p0; p < p1; p++)
    if (__ldg(topk_e + p) == ge) {
      row_pair[row] = p;
      own_row[p] = row;
      row++;
    }
}

// The same grouping with a block of 1024 threads that keeps its pairs in registers: thread
// t owns the 4 * V4 pairs from t * 4 * V4 on, fetched as V4 16-byte loads issued together,
// counts them, takes part in one block-wide scan, and places its hits from the registers.
// For up to 65,536 pairs (V4 <= 16) this replaces two serial passes of 64 to 256 scalar
// loads per thread.
constexpr int kWideThreads = 1024;

template <int V4>
__global__ void __launch_bounds__(kWideThreads)
    moe_group_wide(const int *__restrict__ topk_e, int n_pairs, int e_begin, int e_count,
                   int *__restrict__ counts, int *__restrict__ offsets, int *__restrict__ row_pair,
                   int *__restrict__ own_row) {
  pdl_prologue();
  __shared__ int warp_hits[32], warp_below[32], warp_before[32], s_base, s_total;
  const int e = blockIdx.x, ge = e_begin + e;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int p0 = t * 4 * V4;
  constexpr int kNone = -0x7fffffff - 1; // beyond the end: matches no expert and is never marked

  int x[4 * V4];
#pragma unroll
  for (int j = 0; j < V4; j++) {
    const int p = p0 + 4 * j;
    if (p + 3 < n_pairs) {
      const int4 v = __ldg(reinterpret_cast<const int4 *>(topk_e + p));
      x[4 * j] = v.x, x[4 * j + 1] = v.y, x[4 * j + 2] = v.z, x[4 * j + 3] = v.w;
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++)
        x[4 * j + i] = p + i < n_pairs ? __ldg(topk_e + p + i) : kNone;
    }
  }
  int below = 0, hits = 0;
#pragma unroll
  for (int i = 0; i < 4 * V4; i++) {
    below += (x[i] >= e_begin && x[i] < ge);
    hits += (x[i] == ge);
    // pairs of experts held elsewhere (or of finished tokens, expert -1) get no row;
    // each block marks its share so that every such pair is written exactly once
    if (x[i] != kNone && (x[i] < e_begin || x[i] >= e_begin + e_count) && ((p0 + i) % e_count) == e)
      own_row[p0 + i] = -1;
  }
  const int incl = warp_inclusive_scan(hits, lane);
  int below_w = below;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    below_w += __shfl_xor_sync(0xffffffffu, below_w, o);
  if (lane == 31)
    warp_hits[warp] = incl;
  if (lane == 0)
    warp_below[warp] = below_w;
  __syncthreads();
  if (warp == 0) { // the 32 warp totals: hits of earlier warps for each warp, and the block's sums
    const int h = warp_hits[lane];
    const int hs = warp_inclusive_scan(h, lane);
    int b = warp_below[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      b += __shfl_xor_sync(0xffffffffu, b, o);
    warp_before[lane] = hs - h;
    if (lane == 31)
      s_total = hs;
    if (lane == 0)
      s_base = b;
  }
  __syncthreads();
  const int base = s_base, total = s_total;
  int row = base + warp_before[warp] + incl - hits; // row of this thread's first hit
  if (t == 0) {
    counts[e] = total;
    offsets[e] = base;
    if (e == e_count - 1)
      offsets[e_count] = base + total;
  }
#pragma unroll
  for (int i = 0; i < 4 * V4; i++)
    if (x[i] == ge) {
      row_pair[row] = p0 + i;
      own_row[p0 + i] = row;
      row++;
    }
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_moe_group(gptoss_stream_t stream, const int *topk_e, int n_pairs, int e_begin,
                                int e_count, int *counts, int *offsets, int *row_pair, int *own_row,
                                unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (n_pairs < 0 || e_begin < 0 || e_count <= 0)
    return GPTOSS_ERR_BAD_ARG;
  if (!counts || !offsets)
    return GPTOSS_ERR_BAD_ARG;
  if (n_pairs > 0 && (!topk_e || !row_pair || !own_row))
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(topk_e, (size_t)n_pairs * 4);
  GPTOSS_SPAN(counts, (size_t)e_count * 4);
  GPTOSS_SPAN(offsets, ((size_t)e_count + 1) * 4);
  GPTOSS_SPAN(row_pair, (size_t)n_pairs * 4);
  GPTOSS_SPAN(own_row, (size_t)n_pairs * 4);
  cudaStream_t s = as_stream(stream);
  const long per_thread = ((long)n_pairs + kWideThreads - 1) / kWideThreads; // pairs a thread of the wide form holds
  if (aligned16(topk_e) && per_thread <= 64) {
#define GPTOSS_GROUP_CASE(V4_)                                                                              \
  if (per_thread <= 4 * V4_) {                                                                              \
    launch_kernel(moe_group_wide<V4_>, dim3(e_count), dim3(kWideThreads), 0, s, topk_e, n_pairs, e_begin,   \
                  e_count, counts, offsets, row_pair, own_row);                                             \
    return launch_status();                                                                                 \
  }
    GPTOSS_GROUP_CASE(1)
    GPTOSS_GROUP_CASE(2)
    GPTOSS_GROUP_CASE(4)
    GPTOSS_GROUP_CASE(8)
    GPTOSS_GROUP_CASE(16)
#undef GPTOSS_GROUP_CASE
  }
  launch_kernel(moe_group_rows, dim3(e_count), dim3(kGroupThreads), 0, s, topk_e, n_pairs, e_begin, e_count,
                counts, offsets, row_pair, own_row);
  return launch_status();
}
