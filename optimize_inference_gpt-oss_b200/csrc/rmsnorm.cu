// Residual add fused with RMSNorm (gptoss_add_rmsnorm).
//
// HBM-bound: per row the kernel must read x (4H bytes) and y (aH), and write x
// (4H) and out (aH).  One thread block handles one row at a time; each thread
// owns NC chunks of 8 consecutive elements, issues all of its 128-bit loads
// before the first use, reduces the sum of squares with warp shuffles, and
// writes the row back.  Blocks walk the rows with a grid stride so a launch
// keeps every SM busy with several rows in flight.
#include "common.cuh"

namespace gptoss {
namespace {

struct NoY {}; // tag: no residual delta, the row is only normalised

template <typename YT, typename OT, bool EXACT, int NC>
__global__ void add_rmsnorm_rows(float *x, const YT *__restrict__ y,
                                 const float *__restrict__ w, OT *out, int T, int H) {
  constexpr bool HAS_Y = !std::is_same<YT, NoY>::value;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  __shared__ Acc scratch[2][32];
  const int n_chunks = H >> 3;
  int flip = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, flip ^= 1) {
    float *xr = x + (size_t)row * H;
    Vec8 xs[NC], ws[NC];
    [[maybe_unused]] Vec8 ys[NC];
    bool has[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) {
      const int chunk = threadIdx.x + c * blockDim.x;
      has[c] = chunk < n_chunks;
      if (has[c]) {
        xs[c] = load8<kPlain>(xr, (size_t)chunk * 8);
        if constexpr (HAS_Y)
          ys[c] = load8<kStream>(y + (size_t)row * H, (size_t)chunk * 8);
        ws[c] = load8<kTable>(w, (size_t)chunk * 8);
      }
    }
    Acc ss = 0;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if constexpr (HAS_Y)
            xs[c].v[i] = __fadd_rn(xs[c].v[i], ys[c].v[i]);
          if constexpr (EXACT)
            ss = __dadd_rn(ss, (double)__fmul_rn(xs[c].v[i], xs[c].v[i]));
          else
            ss = fmaf(xs[c].v[i], xs[c].v[i], ss);
        }
      }
    ss = block_sum<Acc>(ss, scratch[flip]);
    OT *orow = out + (size_t)row * H;
    if constexpr (EXACT) {
      // run.cpp:326-331: mean and eps in double, reciprocal root in float,
      // both scalings in double, one rounding.
      double m = __ddiv_rn(ss, (double)H);
      m = __dadd_rn(m, (double)GPTOSS_RMS_EPS);
      const double inv = (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
#pragma unroll
      for (int c = 0; c < NC; c++)
        if (has[c]) {
          const size_t e = (size_t)(threadIdx.x + c * blockDim.x) * 8;
          if constexpr (HAS_Y)
            store8(xr, e, xs[c], false);
          Vec8 o;
#pragma unroll
          for (int i = 0; i < 8; i++)
            o.v[i] = (float)__dmul_rn((double)ws[c].v[i], __dmul_rn(inv, (double)xs[c].v[i]));
          store8(orow, e, o);
        }
    } else {
      const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), GPTOSS_RMS_EPS)));
#pragma unroll
      for (int c = 0; c < NC; c++)
        if (has[c]) {
          const size_t e = (size_t)(threadIdx.x + c * blockDim.x) * 8;
          if constexpr (HAS_Y)
            store8(xr, e, xs[c], false);
          Vec8 o;
#pragma unroll
          for (int i = 0; i < 8; i++)
            o.v[i] = __fmul_rn(ws[c].v[i], __fmul_rn(inv, xs[c].v[i]));
          store8(orow, e, o);
        }
    }
  }
}

// Any H, any alignment: scalar accesses, the row is read twice (the second
// time from cache).  256 threads per row.
template <typename YT, typename OT, bool EXACT>
__global__ void add_rmsnorm_rows_generic(float *x, const YT *__restrict__ y,
                                         const float *__restrict__ w, OT *out, int T, int H) {
  constexpr bool HAS_Y = !std::is_same<YT, NoY>::value;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  __shared__ Acc scratch[2][32];
  int flip = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, flip ^= 1) {
    float *xr = x + (size_t)row * H;
    Acc ss = 0;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      float v = xr[j];
      if constexpr (HAS_Y) {
        v = __fadd_rn(v, load1(y + (size_t)row * H + j));
        xr[j] = v;
      }
      if constexpr (EXACT)
        ss = __dadd_rn(ss, (double)__fmul_rn(v, v));
      else
        ss = fmaf(v, v, ss);
    }
    ss = block_sum<Acc>(ss, scratch[flip]);
    OT *orow = out + (size_t)row * H;
    if constexpr (EXACT) {
      double m = __dadd_rn(__ddiv_rn(ss, (double)H), (double)GPTOSS_RMS_EPS);
      const double inv = (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
      for (int j = threadIdx.x; j < H; j += blockDim.x)
        store1(orow + j, (float)__dmul_rn((double)w[j], __dmul_rn(inv, (double)xr[j])));
    } else {
      const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), GPTOSS_RMS_EPS)));
      for (int j = threadIdx.x; j < H; j += blockDim.x)
        store1(orow + j, __fmul_rn(w[j], __fmul_rn(inv, xr[j])));
    }
  }
}

template <typename YT, typename OT, bool EXACT>
int launch(cudaStream_t s, int T, float *x, const void *y, const float *w, void *out, int H) {
  const bool vec = (H % 8 == 0) && aligned16(x) && aligned16(w) && aligned16(out) &&
                   (y == nullptr || aligned16(y)) && H <= 8 * 512 * 4;
  const YT *yp = static_cast<const YT *>(y);
  OT *op = static_cast<OT *>(out);
  if (!vec) {
    add_rmsnorm_rows_generic<YT, OT, EXACT><<<row_grid(T, 8), 256, 0, s>>>(x, yp, w, op, T, H);
    return launch_status();
  }
  const int n_chunks = H / 8;
  const int nc = n_chunks <= 512 ? 1 : (n_chunks <= 1024 ? 2 : 4);
  int threads = (n_chunks + nc - 1) / nc;
  threads = (threads + 31) / 32 * 32;
  static int occ[3][33];
  int *slot = &occ[nc == 1 ? 0 : (nc == 2 ? 1 : 2)][threads / 32];
  if (nc == 1) {
    auto k = add_rmsnorm_rows<YT, OT, EXACT, 1>;
    k<<<row_grid(T, blocks_per_sm(k, threads, slot)), threads, 0, s>>>(x, yp, w, op, T, H);
  } else if (nc == 2) {
    auto k = add_rmsnorm_rows<YT, OT, EXACT, 2>;
    k<<<row_grid(T, blocks_per_sm(k, threads, slot)), threads, 0, s>>>(x, yp, w, op, T, H);
  } else {
    auto k = add_rmsnorm_rows<YT, OT, EXACT, 4>;
    k<<<row_grid(T, blocks_per_sm(k, threads, slot)), threads, 0, s>>>(x, yp, w, op, T, H);
  }
  return launch_status();
}

template <typename YT, bool EXACT>
int launch_out(cudaStream_t s, int T, float *x, const void *y, const float *w, void *out,
               gptoss_dtype_t out_dtype, int H) {
  return out_dtype == GPTOSS_F32 ? launch<YT, float, EXACT>(s, T, x, y, w, out, H)
                                 : launch<YT, uint16_t, EXACT>(s, T, x, y, w, out, H);
}

template <bool EXACT>
int launch_y(cudaStream_t s, int T, float *x, const void *y, gptoss_dtype_t y_dtype,
             const float *w, void *out, gptoss_dtype_t out_dtype, int H) {
  if (!y)
    return launch_out<NoY, EXACT>(s, T, x, nullptr, w, out, out_dtype, H);
  return y_dtype == GPTOSS_F32 ? launch_out<float, EXACT>(s, T, x, y, w, out, out_dtype, H)
                               : launch_out<uint16_t, EXACT>(s, T, x, y, w, out, out_dtype, H);
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_add_rmsnorm(gptoss_stream_t stream, int T, float *x, const void *y,
                                  gptoss_dtype_t y_dtype, const float *weight, void *out,
                                  gptoss_dtype_t out_dtype, int H, unsigned flags) {
  using namespace gptoss;
  if (T < 0 || H <= 0 || !valid_dtype(out_dtype) || (y && !valid_dtype(y_dtype)))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!x || !weight || !out)
    return GPTOSS_ERR_BAD_ARG;
  // In-place norm is only defined for an fp32 output of the same row layout.
  if (out == (void *)x && out_dtype != GPTOSS_F32)
    return GPTOSS_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  return (flags & GPTOSS_EXACT) ? launch_y<true>(s, T, x, y, y_dtype, weight, out, out_dtype, H)
                                : launch_y<false>(s, T, x, y, y_dtype, weight, out, out_dtype, H);
}
