// Clamped SwiGLU (gptoss_swiglu).
//
// A pure stream: 2 inputs (gate, up; interleaved) per output.  Because rows are
// contiguous, output element n reads input elements 2n and 2n+1 whatever the
// row length, so the kernel runs over flat groups of 8 outputs: two (bf16) or
// four (fp32) 128-bit loads in, one or two 128-bit stores out.  Each thread
// fetches kUnroll groups before computing, which keeps 64-256 B of loads in
// flight per thread.  The fast form costs about 13 instructions per output (two
// of them on the special-function unit), which at 4 outputs per 24 bytes moved
// keeps the SM's issue slots well below the memory time.
#include "common.cuh"
#include "exact_math.cuh"

namespace gptoss {
namespace {

// Groups per thread.  The fast form is a pure stream and wants bytes in flight: 2 groups
// (1, 3 and 4 measured the same or slower on B200).  The exact form spends ~45 instructions per
// output, nine of them in double precision: there the memory system is kept busy by other
// blocks' loads while a block computes, so smaller pieces of work per block overlap better:
// 1 group per thread 126 us per launch at 16,384 x 5760 fp32, 2 groups 139 us, 4 groups 175 us;
// blocks of 128 threads another 3 % over 256 or 512.
#ifndef GPTOSS_SWIGLU_UNROLL
#define GPTOSS_SWIGLU_UNROLL 2
#endif
#ifndef GPTOSS_SWIGLU_UNROLL_EXACT
#define GPTOSS_SWIGLU_UNROLL_EXACT 1
#endif
#ifndef GPTOSS_SWIGLU_THREADS_EXACT
#define GPTOSS_SWIGLU_THREADS_EXACT 128
#endif
template <bool EXACT> struct Shape {
  static constexpr int unroll = EXACT ? GPTOSS_SWIGLU_UNROLL_EXACT : GPTOSS_SWIGLU_UNROLL;
  static constexpr int threads = EXACT ? GPTOSS_SWIGLU_THREADS_EXACT : 256;
};

template <bool EXACT> __device__ __forceinline__ float swiglu_one(float g, float u, float limit) {
  if (EXACT) { // run.cpp:709-722, every step rounded to fp32
    if (g > limit)
      g = limit;
    if (u > limit)
      u = limit;
    if (u < -limit)
      u = -limit;
    // 1.0f / (1.0f + e): the correctly rounded reciprocal is that quotient
    const float sig = __frcp_rn(__fadd_rn(1.0f, glibc_expf(__fmul_rn(-1.702f, g))));
    g = __fmul_rn(g, sig);
    return __fmul_rn(g, __fadd_rn(u, 1.0f));
  }
  // the reference's fast form (kernels/fast_misc.hpp:136-139):
  // g / (1 + e^(-1.702 g)) * (u + 1), with e^x as 2^(x log2 e)
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  const float e = fast_exp2(g * (-1.702f * 1.44269504088896341f));
  return (g * fast_rcp(1.0f + e)) * (u + 1.0f);
}

// One group = 8 outputs = 16 inputs: kIn 16-byte loads (2 for bf16, 4 for fp32),
// kept as loaded until they are used.  One-shot grid: block b owns groups
// [b * 256 * kUnroll, (b + 1) * 256 * kUnroll), a contiguous tile, and exits;
// the hardware scheduler keeps every SM stocked with fresh blocks, which
// measured ~10 % faster on B200 than a grid-stride loop over the same data.
template <typename YT, typename GT, bool EXACT>
__global__ void __launch_bounds__(Shape<EXACT>::threads)
    swiglu_flat(const YT *__restrict__ Y, GT *__restrict__ G, size_t n_groups, float limit) {
  pdl_prologue();
  constexpr int kIn = sizeof(YT);         // 16-byte loads per group
  constexpr int kPer = 16 / sizeof(YT);   // inputs per load
  constexpr int kUnroll = Shape<EXACT>::unroll, kThreads = Shape<EXACT>::threads;
  const size_t base = (size_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
  uint4 raw[kUnroll][kIn];
#pragma unroll
  for (int u = 0; u < kUnroll; u++) {
    // past the end: fetch the last group again; its result is not stored
    const size_t g = base + u * kThreads < n_groups ? base + u * kThreads : n_groups - 1;
#pragma unroll
    for (int j = 0; j < kIn; j++)
      raw[u][j] = ld_stream(Y + g * 16 + j * kPer);
  }
#pragma unroll
  for (int u = 0; u < kUnroll; u++) {
    Vec8 o;
    if constexpr (sizeof(YT) == 2) { // each 32-bit word holds one (gate, up) pair
#pragma unroll
      for (int j = 0; j < 2; j++) {
        const uint32_t w[4] = {raw[u][j].x, raw[u][j].y, raw[u][j].z, raw[u][j].w};
#pragma unroll
        for (int i = 0; i < 4; i++)
          o.v[4 * j + i] = swiglu_one<EXACT>(bf16_lo(w[i]), bf16_hi(w[i]), limit);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        o.v[2 * j] = swiglu_one<EXACT>(__uint_as_float(raw[u][j].x), __uint_as_float(raw[u][j].y), limit);
        o.v[2 * j + 1] = swiglu_one<EXACT>(__uint_as_float(raw[u][j].z), __uint_as_float(raw[u][j].w), limit);
      }
    }
    if (base + u * kThreads < n_groups)
      store8(G, (base + u * kThreads) * 8, o);
  }
}

// Tail elements and misaligned buffers: one output per thread step.
template <typename YT, typename GT, bool EXACT>
__global__ void swiglu_scalar(const YT *__restrict__ Y, GT *__restrict__ G, size_t first,
                              size_t n_out, float limit) {
  pdl_prologue();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t n = first + (size_t)blockIdx.x * blockDim.x + threadIdx.x; n < n_out; n += stride)
    store1(G + n, swiglu_one<EXACT>(load1(Y + 2 * n), load1(Y + 2 * n + 1), limit));
}

template <typename YT, typename GT, bool EXACT>
int launch(cudaStream_t s, const void *Y, void *G, size_t n_out, float limit) {
  const YT *yp = static_cast<const YT *>(Y);
  GT *gp = static_cast<GT *>(G);
  constexpr int threads = Shape<EXACT>::threads, kUnroll = Shape<EXACT>::unroll;
  size_t n_groups = (aligned16(Y) && aligned16(G)) ? n_out / 8 : 0;
  if (n_groups > 0) {
    const size_t blocks = (n_groups + (size_t)threads * kUnroll - 1) / ((size_t)threads * kUnroll);
    if (blocks > 0x7fffffffull)
      return GPTOSS_ERR_UNSUPPORTED;
    launch_kernel(swiglu_flat<YT, GT, EXACT>, dim3((unsigned)blocks), dim3(threads), 0, s, yp, gp, n_groups, limit);
    const int st = launch_status();
    if (st != GPTOSS_OK)
      return st;
  }
  const size_t done = n_groups * 8;
  if (done < n_out) {
    const size_t rest = n_out - done;
    const long blocks = (long)((rest + threads - 1) / threads);
    note_generic_launch();
    launch_kernel(swiglu_scalar<YT, GT, EXACT>, dim3(row_grid(blocks, 8)), dim3(threads), 0, s, yp, gp, done, n_out, limit);
    return launch_status();
  }
  return GPTOSS_OK;
}

template <bool EXACT>
int launch_types(cudaStream_t s, const void *Y, gptoss_dtype_t yd, void *G, gptoss_dtype_t gd,
                 size_t n_out, float limit) {
  if (yd == GPTOSS_F32)
    return gd == GPTOSS_F32 ? launch<float, float, EXACT>(s, Y, G, n_out, limit)
                            : launch<float, uint16_t, EXACT>(s, Y, G, n_out, limit);
  return gd == GPTOSS_F32 ? launch<uint16_t, float, EXACT>(s, Y, G, n_out, limit)
                          : launch<uint16_t, uint16_t, EXACT>(s, Y, G, n_out, limit);
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_swiglu(gptoss_stream_t stream, const void *Y, gptoss_dtype_t y_dtype, void *G,
                             gptoss_dtype_t g_dtype, size_t R, int I, float limit,
                             unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (I <= 0 || !valid_dtype(y_dtype) || !valid_dtype(g_dtype) || !(limit >= 0.0f))
    return GPTOSS_ERR_BAD_ARG;
  if (R == 0)
    return GPTOSS_OK;
  if (!Y || !G)
    return GPTOSS_ERR_BAD_ARG;
  if (R > ((size_t)1 << 40) / (size_t)I)
    return GPTOSS_ERR_UNSUPPORTED;
  const size_t n_out = R * (size_t)I;
  GPTOSS_SPAN(Y, 2 * n_out * dtype_size(y_dtype));
  GPTOSS_SPAN(G, n_out * dtype_size(g_dtype));
  cudaStream_t s = as_stream(stream);
  return (flags & GPTOSS_EXACT) ? launch_types<true>(s, Y, y_dtype, G, g_dtype, n_out, limit)
                                : launch_types<false>(s, Y, y_dtype, G, g_dtype, n_out, limit);
}
