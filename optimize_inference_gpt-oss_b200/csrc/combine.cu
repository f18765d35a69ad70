// Weighted expert combine fused with the residual and, optionally, the next
// RMSNorm (gptoss_moe_combine).
//
// Per token the kernel reads the residual row, k expert-output rows (through
// the own_row indirection) and k weights, and writes the residual row and,
// with the norm, one normalised row.  One thread block per token at a time;
// each thread owns NC chunks of 8 consecutive elements and issues the loads of
// the residual chunk and of all k expert chunks (up to 9 x 16-32 B per chunk)
// before the first use, so a block keeps a whole token (about 34 KB at H = 2880,
// k = 4, bf16 experts) in flight.
#include "common.cuh"

namespace gptoss {
namespace {

template <typename ZT> struct RawChunk { // 8 elements as loaded
  uint4 q[sizeof(ZT) / 2];
};

template <typename ZT> __device__ __forceinline__ RawChunk<ZT> load_raw(const ZT *p) {
  RawChunk<ZT> r;
  r.q[0] = ld_stream(p);
  if constexpr (sizeof(ZT) == 4)
    r.q[1] = ld_stream(p + 4);
  return r;
}

template <typename ZT> __device__ __forceinline__ Vec8 widen(const RawChunk<ZT> &r) {
  if constexpr (sizeof(ZT) == 2) {
    return widen8(r.q[0]);
  } else {
    Vec8 v;
    v.v[0] = __uint_as_float(r.q[0].x), v.v[1] = __uint_as_float(r.q[0].y),
    v.v[2] = __uint_as_float(r.q[0].z), v.v[3] = __uint_as_float(r.q[0].w),
    v.v[4] = __uint_as_float(r.q[1].x), v.v[5] = __uint_as_float(r.q[1].y),
    v.v[6] = __uint_as_float(r.q[1].z), v.v[7] = __uint_as_float(r.q[1].w);
    return v;
  }
}

// MODE 0: fast (choice order, FMA).  MODE 1: exact (increasing expert, separate
// product and sum).  MODE 2: exact order with FMA.
template <typename ZT, typename OT, int MODE, bool NORM, int KM, int NC>
__global__ void combine_rows(float *x, const ZT *__restrict__ Z, const int *__restrict__ own_row,
                             const float *__restrict__ topk_w, const int *__restrict__ topk_e,
                             int k, int H, const int *__restrict__ phys_of,
                             const float *__restrict__ norm_w, OT *__restrict__ out, int T) {
  constexpr bool EXACT = MODE != 0;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  __shared__ Acc scratch[2][32];
  const int n_chunks = H >> 3;
  int flip = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, flip ^= 1) {
    float *xr = x + (size_t)row * H;
    const bool live = __ldg(topk_e + (size_t)row * k) >= 0;
    // order in which the choices are added
    int ord[KM];
#pragma unroll
    for (int j = 0; j < KM; j++)
      ord[j] = j;
    if (EXACT && live) {
      int key[KM];
#pragma unroll
      for (int j = 0; j < KM; j++) {
        const int e = j < k ? __ldg(topk_e + (size_t)row * k + j) : 0x7fffffff;
        key[j] = (phys_of && e >= 0 && e != 0x7fffffff) ? __ldg(phys_of + e) : e;
      }
#pragma unroll
      for (int i = 1; i < KM; i++)
#pragma unroll
        for (int j = i; j > 0; j--)
          if (key[j] < key[j - 1]) { // stable insertion sort, fully unrolled
            const int tk = key[j], to = ord[j];
            key[j] = key[j - 1], ord[j] = ord[j - 1];
            key[j - 1] = tk, ord[j - 1] = to;
          }
    }
    const ZT *zrow[KM];
    float wgt[KM];
#pragma unroll
    for (int j = 0; j < KM; j++) {
      zrow[j] = Z;
      wgt[j] = 0.0f;
      if (live && j < k) {
        const size_t p = (size_t)row * k + ord[j];
        const size_t zr = own_row ? (size_t)__ldg(own_row + p) : p;
        zrow[j] = Z + zr * H;
        wgt[j] = __ldg(topk_w + p);
      }
    }
    Vec8 xs[NC];
    [[maybe_unused]] Vec8 ws[NC];
    bool has[NC];
    Acc ss = 0;
#pragma unroll
    for (int c = 0; c < NC; c++) {
      const int chunk = threadIdx.x + c * blockDim.x;
      has[c] = chunk < n_chunks;
      if (!has[c])
        continue;
      const size_t e = (size_t)chunk * 8;
      xs[c] = load8<kPlain>(xr, e);
      if constexpr (NORM)
        ws[c] = load8<kTable>(norm_w, e);
      if (live) {
        RawChunk<ZT> zr[KM];
#pragma unroll
        for (int j = 0; j < KM; j++)
          if (j < k)
            zr[j] = load_raw(zrow[j] + e);
        Vec8 acc;
#pragma unroll
        for (int i = 0; i < 8; i++)
          acc.v[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < KM; j++)
          if (j < k) {
            const Vec8 z = widen(zr[j]);
#pragma unroll
            for (int i = 0; i < 8; i++)
              acc.v[i] = MODE == 1 ? __fadd_rn(acc.v[i], __fmul_rn(z.v[i], wgt[j]))
                                   : __fmaf_rn(z.v[i], wgt[j], acc.v[i]);
          }
#pragma unroll
        for (int i = 0; i < 8; i++)
          xs[c].v[i] = __fadd_rn(xs[c].v[i], acc.v[i]);
        store8(xr, e, xs[c], false);
      }
      if constexpr (NORM) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          if constexpr (EXACT)
            ss = __dadd_rn(ss, (double)__fmul_rn(xs[c].v[i], xs[c].v[i]));
          else
            ss = fmaf(xs[c].v[i], xs[c].v[i], ss);
        }
      }
    }
    if constexpr (NORM) {
      ss = block_sum<Acc>(ss, scratch[flip]);
      OT *orow = out + (size_t)row * H;
      [[maybe_unused]] double inv_d = 0.0;
      [[maybe_unused]] float inv_f = 0.0f;
      if constexpr (EXACT) {
        const double m = __dadd_rn(__ddiv_rn(ss, (double)H), (double)GPTOSS_RMS_EPS);
        inv_d = (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
      } else {
        inv_f = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), GPTOSS_RMS_EPS)));
      }
#pragma unroll
      for (int c = 0; c < NC; c++)
        if (has[c]) {
          Vec8 o;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            if constexpr (EXACT)
              o.v[i] = (float)__dmul_rn((double)ws[c].v[i], __dmul_rn(inv_d, (double)xs[c].v[i]));
            else
              o.v[i] = __fmul_rn(ws[c].v[i], __fmul_rn(inv_f, xs[c].v[i]));
          }
          store8(orow, (size_t)(threadIdx.x + c * blockDim.x) * 8, o);
        }
    }
  }
}

// Any H, k <= GPTOSS_MAX_TOPK, any alignment: scalar accesses.
template <typename ZT, typename OT, int MODE, bool NORM>
__global__ void combine_rows_generic(float *x, const ZT *__restrict__ Z,
                                     const int *__restrict__ own_row,
                                     const float *__restrict__ topk_w,
                                     const int *__restrict__ topk_e, int k, int H,
                                     const int *__restrict__ phys_of,
                                     const float *__restrict__ norm_w, OT *__restrict__ out,
                                     int T) {
  constexpr bool EXACT = MODE != 0;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  __shared__ Acc scratch[2][32];
  int flip = 0;
  for (int row = blockIdx.x; row < T; row += gridDim.x, flip ^= 1) {
    float *xr = x + (size_t)row * H;
    const bool live = topk_e[(size_t)row * k] >= 0;
    int ord[GPTOSS_MAX_TOPK];
    for (int j = 0; j < k; j++)
      ord[j] = j;
    if (EXACT && live)
      for (int i = 1; i < k; i++)
        for (int j = i; j > 0; j--) {
          const int ea = topk_e[(size_t)row * k + ord[j]], eb = topk_e[(size_t)row * k + ord[j - 1]];
          const int ka = phys_of && ea >= 0 ? phys_of[ea] : ea, kb = phys_of && eb >= 0 ? phys_of[eb] : eb;
          if (!(ka < kb))
            break;
          const int t = ord[j];
          ord[j] = ord[j - 1];
          ord[j - 1] = t;
        }
    Acc ss = 0;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = xr[i];
      if (live) {
        float acc = 0.0f;
        for (int j = 0; j < k; j++) {
          const size_t p = (size_t)row * k + ord[j];
          const size_t zr = own_row ? (size_t)own_row[p] : p;
          const float z = load1(Z + zr * H + i), w = topk_w[p];
          acc = MODE == 1 ? __fadd_rn(acc, __fmul_rn(z, w)) : __fmaf_rn(z, w, acc);
        }
        v = __fadd_rn(v, acc);
        xr[i] = v;
      }
      if constexpr (NORM) {
        if constexpr (EXACT)
          ss = __dadd_rn(ss, (double)__fmul_rn(v, v));
        else
          ss = fmaf(v, v, ss);
      }
    }
    if constexpr (NORM) {
      ss = block_sum<Acc>(ss, scratch[flip]);
      OT *orow = out + (size_t)row * H;
      if constexpr (EXACT) {
        const double m = __dadd_rn(__ddiv_rn(ss, (double)H), (double)GPTOSS_RMS_EPS);
        const double inv = (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
        for (int i = threadIdx.x; i < H; i += blockDim.x)
          store1(orow + i, (float)__dmul_rn((double)norm_w[i], __dmul_rn(inv, (double)xr[i])));
      } else {
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), GPTOSS_RMS_EPS)));
        for (int i = threadIdx.x; i < H; i += blockDim.x)
          store1(orow + i, __fmul_rn(norm_w[i], __fmul_rn(inv, xr[i])));
      }
    }
  }
}

struct Args {
  int T;
  float *x;
  const void *Z;
  const int *own_row;
  const float *topk_w;
  const int *topk_e;
  int k, H;
  const int *phys_of;
  const float *norm_w;
  void *out;
};

template <typename ZT, typename OT, int MODE, bool NORM, int KM, int NC>
int launch_kernel(cudaStream_t s, const Args &a, int threads) {
  static int occ[33];
  auto kern = combine_rows<ZT, OT, MODE, NORM, KM, NC>;
  kern<<<row_grid(a.T, blocks_per_sm(kern, threads, &occ[threads / 32])), threads, 0, s>>>(
      a.x, static_cast<const ZT *>(a.Z), a.own_row, a.topk_w, a.topk_e, a.k, a.H, a.phys_of,
      a.norm_w, static_cast<OT *>(a.out), a.T);
  return launch_status();
}

template <typename ZT, typename OT, int MODE, bool NORM> int launch(cudaStream_t s, const Args &a) {
  const bool vec = a.H % 8 == 0 && a.H <= 8 * 512 * 4 && aligned16(a.x) && aligned16(a.Z) &&
                   (!NORM || (aligned16(a.norm_w) && aligned16(a.out)));
  if (!vec) {
    combine_rows_generic<ZT, OT, MODE, NORM><<<row_grid(a.T, 8), 256, 0, s>>>(
        a.x, static_cast<const ZT *>(a.Z), a.own_row, a.topk_w, a.topk_e, a.k, a.H, a.phys_of,
        a.norm_w, static_cast<OT *>(a.out), a.T);
    return launch_status();
  }
  const int n_chunks = a.H / 8;
  const int nc = n_chunks <= 512 ? 1 : 4;
  int threads = ((n_chunks + nc - 1) / nc + 31) / 32 * 32;
  if (a.k <= 4)
    return nc == 1 ? launch_kernel<ZT, OT, MODE, NORM, 4, 1>(s, a, threads)
                   : launch_kernel<ZT, OT, MODE, NORM, 4, 4>(s, a, threads);
  return nc == 1 ? launch_kernel<ZT, OT, MODE, NORM, 8, 1>(s, a, threads)
                 : launch_kernel<ZT, OT, MODE, NORM, 8, 4>(s, a, threads);
}

template <typename ZT, int MODE>
int launch_norm(cudaStream_t s, const Args &a, gptoss_dtype_t out_dtype) {
  if (!a.norm_w)
    return launch<ZT, float, MODE, false>(s, a);
  return out_dtype == GPTOSS_F32 ? launch<ZT, float, MODE, true>(s, a)
                                 : launch<ZT, uint16_t, MODE, true>(s, a);
}

template <typename ZT>
int launch_mode(cudaStream_t s, const Args &a, gptoss_dtype_t out_dtype, unsigned flags) {
  if (!(flags & GPTOSS_EXACT))
    return launch_norm<ZT, 0>(s, a, out_dtype);
  return (flags & GPTOSS_FMA) ? launch_norm<ZT, 2>(s, a, out_dtype)
                              : launch_norm<ZT, 1>(s, a, out_dtype);
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_moe_combine(gptoss_stream_t stream, int T, float *x, const void *Z,
                                  gptoss_dtype_t z_dtype, const int *own_row,
                                  const float *topk_w, const int *topk_e, int k, int H,
                                  const int *phys_of, const float *norm_w, void *out,
                                  gptoss_dtype_t out_dtype, unsigned flags) {
  using namespace gptoss;
  if (T < 0 || k <= 0 || H <= 0 || !valid_dtype(z_dtype) || (norm_w && !valid_dtype(out_dtype)))
    return GPTOSS_ERR_BAD_ARG;
  if (k > GPTOSS_MAX_TOPK)
    return GPTOSS_ERR_UNSUPPORTED;
  if (T == 0)
    return GPTOSS_OK;
  if (!x || !Z || !topk_w || !topk_e || (norm_w && !out))
    return GPTOSS_ERR_BAD_ARG;
  const Args a{T, x, Z, own_row, topk_w, topk_e, k, H, phys_of, norm_w, out};
  cudaStream_t s = as_stream(stream);
  return z_dtype == GPTOSS_F32 ? launch_mode<float>(s, a, out_dtype, flags)
                               : launch_mode<uint16_t>(s, a, out_dtype, flags);
}
