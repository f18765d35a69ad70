// Residual add fused with RMSNorm (gptoss_add_rmsnorm).
//
// HBM-bound: per row the kernel must read x (4H bytes) and y (aH), and write x
// (4H) and out (aH).  One thread block works on one row at a time and walks
// the rows with a grid stride.  Rows are staged through a ring of shared-memory
// buffers filled by cp.async: while a block normalises row r, the copies of the
// next STAGES-1 rows of its walk are already in flight, so an SM keeps 100-200
// KB of reads outstanding regardless of register pressure.  A thread owns NC
// chunks of 8 consecutive elements, copies exactly those chunks and reads only
// them back, so the data needs no block barrier; the one barrier per row is the
// sum-of-squares reduction (warp shuffles, then one shared-memory hop).
#include "common.cuh"

namespace gptoss {
namespace {

struct NoY {}; // tag: no residual delta, the row is only normalised

template <typename YT> struct YSize {
  static constexpr int value = sizeof(YT);
};
template <> struct YSize<NoY> {
  static constexpr int value = 0;
};

// fp32 mode scale: run.cpp:326-331 -- mean and eps in double, reciprocal root
// in float.  bf16 mode: kernels/fast_misc.hpp:29 in fp32.
__device__ __forceinline__ double exact_inv_rms(double ss, int H) {
  double m = __ddiv_rn(ss, (double)H);
  m = __dadd_rn(m, (double)GPTOSS_RMS_EPS);
  return (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
}
__device__ __forceinline__ float fast_inv_rms(float ss, int H) {
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), GPTOSS_RMS_EPS)));
}

template <typename YT, typename OT, bool EXACT, int NC, int STAGES>
__global__ void add_rmsnorm_rows(float *x, const YT *__restrict__ y, const float *__restrict__ w,
                                 OT *out, int T, int H) {
  pdl_prologue();
  constexpr bool HAS_Y = !std::is_same<YT, NoY>::value;
  constexpr int SY = YSize<YT>::value;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  extern __shared__ __align__(16) unsigned char ring[];
  __shared__ Acc scratch[2][32];
  const size_t stage_bytes = (size_t)H * (4 + SY);
  const int n_chunks = H >> 3;

  // this thread's chunks and their gains, the same for every row
  bool has[NC];
  Vec8 ws[NC];
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const int chunk = threadIdx.x + c * blockDim.x;
    has[c] = chunk < n_chunks;
    if (has[c])
      ws[c] = load8<kTable>(w, (size_t)chunk * 8);
  }

  auto issue = [&](long row, int stage) {
    unsigned char *sx = ring + (size_t)stage * stage_bytes;
    const float *xr = x + (size_t)row * H;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        const int chunk = threadIdx.x + c * blockDim.x;
        cp_async16(sx + (size_t)chunk * 32, xr + (size_t)chunk * 8);
        cp_async16(sx + (size_t)chunk * 32 + 16, xr + (size_t)chunk * 8 + 4);
        if constexpr (HAS_Y) {
          unsigned char *sy = sx + (size_t)H * 4;
          const YT *yr = y + (size_t)row * H + (size_t)chunk * 8;
          cp_async16(sy + (size_t)chunk * 8 * SY, yr);
          if constexpr (SY == 4)
            cp_async16(sy + (size_t)chunk * 32 + 16, yr + 4);
        }
      }
  };

  const long step = gridDim.x;
  long row = blockIdx.x;
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if (row + s * step < T)
      issue(row + s * step, s);
    cp_async_commit();
  }
  int stage = 0, flip = 0;
  for (; row < T; row += step, flip ^= 1) {
    {
      const long ahead = row + (STAGES - 1) * step;
      const int fill = stage == 0 ? STAGES - 1 : stage - 1;
      if (ahead < T)
        issue(ahead, fill);
      cp_async_commit();
    }
    cp_async_wait<STAGES - 1>(); // this row's copies have landed

    const unsigned char *sx = ring + (size_t)stage * stage_bytes;
    Vec8 xs[NC];
    Acc ss = 0;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        const int chunk = threadIdx.x + c * blockDim.x;
        const uint4 a = *reinterpret_cast<const uint4 *>(sx + (size_t)chunk * 32);
        const uint4 b = *reinterpret_cast<const uint4 *>(sx + (size_t)chunk * 32 + 16);
        xs[c].v[0] = __uint_as_float(a.x), xs[c].v[1] = __uint_as_float(a.y),
        xs[c].v[2] = __uint_as_float(a.z), xs[c].v[3] = __uint_as_float(a.w),
        xs[c].v[4] = __uint_as_float(b.x), xs[c].v[5] = __uint_as_float(b.y),
        xs[c].v[6] = __uint_as_float(b.z), xs[c].v[7] = __uint_as_float(b.w);
        if constexpr (HAS_Y) {
          const unsigned char *sy = sx + (size_t)H * 4 + (size_t)chunk * 8 * SY;
          Vec8 ys;
          if constexpr (SY == 2) {
            ys = widen8(*reinterpret_cast<const uint4 *>(sy));
          } else {
            const uint4 p = *reinterpret_cast<const uint4 *>(sy), q = *reinterpret_cast<const uint4 *>(sy + 16);
            ys.v[0] = __uint_as_float(p.x), ys.v[1] = __uint_as_float(p.y), ys.v[2] = __uint_as_float(p.z),
            ys.v[3] = __uint_as_float(p.w), ys.v[4] = __uint_as_float(q.x), ys.v[5] = __uint_as_float(q.y),
            ys.v[6] = __uint_as_float(q.z), ys.v[7] = __uint_as_float(q.w);
          }
#pragma unroll
          for (int i = 0; i < 8; i++)
            xs[c].v[i] = __fadd_rn(xs[c].v[i], ys.v[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if constexpr (EXACT)
            ss = __dadd_rn(ss, (double)__fmul_rn(xs[c].v[i], xs[c].v[i]));
          else
            ss = fmaf(xs[c].v[i], xs[c].v[i], ss);
        }
      }
    ss = block_sum<Acc>(ss, scratch[flip]);
    float *xr = x + (size_t)row * H;
    OT *orow = out + (size_t)row * H;
    [[maybe_unused]] double inv_d = 0.0;
    [[maybe_unused]] float inv_f = 0.0f;
    if constexpr (EXACT)
      inv_d = exact_inv_rms(ss, H);
    else
      inv_f = fast_inv_rms(ss, H);
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        const size_t e = (size_t)(threadIdx.x + c * blockDim.x) * 8;
        if constexpr (HAS_Y)
          store8(xr, e, xs[c], false);
        Vec8 o;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if constexpr (EXACT)
            o.v[i] = (float)__dmul_rn((double)ws[c].v[i], __dmul_rn(inv_d, (double)xs[c].v[i]));
          else
            o.v[i] = __fmul_rn(ws[c].v[i], __fmul_rn(inv_f, xs[c].v[i]));
        }
        store8(orow, e, o);
      }
    stage = stage + 1 == STAGES ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

// Any H, any alignment: scalar accesses, the row is read twice (the second
// time from cache).  256 threads per row.
template <typename YT, typename OT, bool EXACT>
__global__ void add_rmsnorm_rows_generic(float *x, const YT *__restrict__ y,
                                         const float *__restrict__ w, OT *out, int T, int H) {
  pdl_prologue();
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
      const double inv = exact_inv_rms(ss, H);
      for (int j = threadIdx.x; j < H; j += blockDim.x)
        store1(orow + j, (float)__dmul_rn((double)w[j], __dmul_rn(inv, (double)xr[j])));
    } else {
      const float inv = fast_inv_rms(ss, H);
      for (int j = threadIdx.x; j < H; j += blockDim.x)
        store1(orow + j, __fmul_rn(w[j], __fmul_rn(inv, xr[j])));
    }
  }
}

template <typename YT, typename OT, bool EXACT, int NC, int STAGES>
int launch_pipe(cudaStream_t s, int T, float *x, const YT *y, const float *w, OT *out, int H,
                int threads, size_t smem) {
  auto k = add_rmsnorm_rows<YT, OT, EXACT, NC, STAGES>;
  const int per_sm = blocks_per_sm_smem(k, threads, smem);
  if (per_sm < 1)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(k, dim3(row_grid(T, per_sm)), dim3(threads), smem, s, x, y, w, out, T, H);
  return launch_status();
}

template <typename YT, typename OT, bool EXACT>
int launch(cudaStream_t s, int T, float *x, const void *y, const float *w, void *out, int H) {
  const YT *yp = static_cast<const YT *>(y);
  OT *op = static_cast<OT *>(out);
  const size_t stage_bytes = (size_t)H * (4 + YSize<YT>::value);
  const int stages = pick_stages(stage_bytes);
  const bool vec = (H % 8 == 0) && aligned16(x) && aligned16(w) && aligned16(out) &&
                   (y == nullptr || aligned16(y)) && H <= 8 * 512 * 4 && stages > 0;
  if (vec) {
    const int n_chunks = H / 8;
    const int nc = n_chunks <= 512 ? 1 : (n_chunks <= 1024 ? 2 : 4);
    const int threads = ((n_chunks + nc - 1) / nc + 31) / 32 * 32;
    const size_t smem = stage_bytes * stages;
    int st = GPTOSS_ERR_UNSUPPORTED;
#define GPTOSS_NORM_CASE(NC_, ST_)                                                                \
  if (nc == NC_ && stages == ST_)                                                                 \
  st = launch_pipe<YT, OT, EXACT, NC_, ST_>(s, T, x, yp, w, op, H, threads, smem)
    GPTOSS_NORM_CASE(1, 4);
    GPTOSS_NORM_CASE(1, 3);
    GPTOSS_NORM_CASE(2, 4);
    GPTOSS_NORM_CASE(2, 3);
    GPTOSS_NORM_CASE(2, 2);
    GPTOSS_NORM_CASE(4, 3);
    GPTOSS_NORM_CASE(4, 2);
#undef GPTOSS_NORM_CASE
    if (st != GPTOSS_ERR_UNSUPPORTED)
      return st;
  }
  launch_kernel(add_rmsnorm_rows_generic<YT, OT, EXACT>, dim3(row_grid(T, 8)), dim3(256), 0, s, x, yp, w, op, T, H);
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
  const PdlScope pdl(flags);
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
