// Clamped SwiGLU (gptoss_swiglu).
//
// A pure stream: 2 inputs (gate, up; interleaved) per output.  Because rows are
// contiguous, output element n reads input elements 2n and 2n+1 whatever the
// row length, so the kernel runs over flat groups of 8 outputs: two (bf16) or
// four (fp32) 128-bit loads in, one or two 128-bit stores out.  Each thread
// fetches kUnroll groups before computing, which keeps 64-256 B of loads in
// flight per thread.
#include "common.cuh"
#include "exact_math.cuh"

namespace gptoss {
namespace {

constexpr int kUnroll = 2;

template <bool EXACT> __device__ __forceinline__ float swiglu_one(float g, float u, float limit) {
  if (EXACT) { // run.cpp:709-722, every step rounded to fp32
    if (g > limit)
      g = limit;
    if (u > limit)
      u = limit;
    if (u < -limit)
      u = -limit;
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, glibc_expf(__fmul_rn(-1.702f, g))));
    g = __fmul_rn(g, sig);
    return __fmul_rn(g, __fadd_rn(u, 1.0f));
  }
  // the reference's fast form (kernels/fast_misc.hpp:136-139)
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  g = __fdividef(g, 1.0f + __expf(-1.702f * g));
  return g * (u + 1.0f);
}

template <typename YT, typename GT, bool EXACT>
__global__ void swiglu_flat(const YT *__restrict__ Y, GT *__restrict__ G, size_t n_groups,
                            float limit) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < n_groups;
       base += stride * kUnroll) {
    Vec8 lo[kUnroll], hi[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const size_t g = base + u * stride;
      live[u] = g < n_groups;
      if (live[u]) {
        lo[u] = load8<kStream>(Y, g * 16);
        hi[u] = load8<kStream>(Y, g * 16 + 8);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++)
      if (live[u]) {
        Vec8 o;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          o.v[i] = swiglu_one<EXACT>(lo[u].v[2 * i], lo[u].v[2 * i + 1], limit);
          o.v[4 + i] = swiglu_one<EXACT>(hi[u].v[2 * i], hi[u].v[2 * i + 1], limit);
        }
        store8(G, (base + u * stride) * 8, o);
      }
  }
}

// Tail elements and misaligned buffers: one output per thread step.
template <typename YT, typename GT, bool EXACT>
__global__ void swiglu_scalar(const YT *__restrict__ Y, GT *__restrict__ G, size_t first,
                              size_t n_out, float limit) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t n = first + (size_t)blockIdx.x * blockDim.x + threadIdx.x; n < n_out; n += stride)
    store1(G + n, swiglu_one<EXACT>(load1(Y + 2 * n), load1(Y + 2 * n + 1), limit));
}

template <typename YT, typename GT, bool EXACT>
int launch(cudaStream_t s, const void *Y, void *G, size_t n_out, float limit) {
  const YT *yp = static_cast<const YT *>(Y);
  GT *gp = static_cast<GT *>(G);
  constexpr int threads = 256;
  size_t n_groups = (aligned16(Y) && aligned16(G)) ? n_out / 8 : 0;
  if (n_groups > 0) {
    static int occ = 0;
    auto k = swiglu_flat<YT, GT, EXACT>;
    const size_t want = (n_groups + (size_t)threads * kUnroll - 1) / ((size_t)threads * kUnroll);
    k<<<row_grid((long)want, blocks_per_sm(k, threads, &occ)), threads, 0, s>>>(yp, gp, n_groups,
                                                                                limit);
    const int st = launch_status();
    if (st != GPTOSS_OK)
      return st;
  }
  const size_t done = n_groups * 8;
  if (done < n_out) {
    const size_t rest = n_out - done;
    const long blocks = (long)((rest + threads - 1) / threads);
    swiglu_scalar<YT, GT, EXACT><<<row_grid(blocks, 8), threads, 0, s>>>(yp, gp, done, n_out, limit);
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
  if (I <= 0 || !valid_dtype(y_dtype) || !valid_dtype(g_dtype) || !(limit >= 0.0f))
    return GPTOSS_ERR_BAD_ARG;
  if (R == 0)
    return GPTOSS_OK;
  if (!Y || !G)
    return GPTOSS_ERR_BAD_ARG;
  if (R > ((size_t)1 << 40) / (size_t)I)
    return GPTOSS_ERR_UNSUPPORTED;
  const size_t n_out = R * (size_t)I;
  cudaStream_t s = as_stream(stream);
  return (flags & GPTOSS_EXACT) ? launch_types<true>(s, Y, y_dtype, G, g_dtype, n_out, limit)
                                : launch_types<false>(s, Y, y_dtype, G, g_dtype, n_out, limit);
}
