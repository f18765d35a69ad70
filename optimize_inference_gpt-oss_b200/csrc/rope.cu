// QKV bias add fused with YaRN RoPE (gptoss_qkv_bias_rope).
//
// Per row the kernel reads the fused q|k|v row once and writes it once; the
// bias (one row) and the cos/sin row of the token's position stay in cache.
// A work item is (head, piece): 8 consecutive elements of the head's first
// half together with the 8 elements head_dim/2 further on -- the two halves of
// eight rotation pairs -- so every global access is 128 bits wide and a thread
// never needs data from another thread.  Value heads use the same items, they
// just skip the rotation.  One thread block walks the rows with a grid stride.
#include "common.cuh"

namespace gptoss {
namespace {

template <typename IT, typename OT, bool EXACT, bool FMA>
__global__ void bias_rope_rows(const IT *qkv_in, long in_stride, const float *__restrict__ bias,
                               const int *__restrict__ pos, int pos_scalar,
                               const float *__restrict__ cos_tab,
                               const float *__restrict__ sin_tab, int n_pos, int n_rot_heads,
                               int n_heads, int head_dim, OT *qkv_out, long out_stride, int T) {
  const int half = head_dim >> 1, pieces = half >> 3, items = n_heads * pieces;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    int p = pos ? __ldg(pos + row) : pos_scalar;
    p = p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
    const float *cs = cos_tab + (size_t)p * half, *sn = sin_tab + (size_t)p * half;
    const IT *in = qkv_in + (size_t)row * in_stride;
    OT *out = qkv_out + (size_t)row * out_stride;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
      const int head = item / pieces, piece = item - head * pieces;
      const size_t lo = (size_t)head * head_dim + piece * 8, hi = lo + half;
      Vec8 a = load8<kStream>(in, lo), b = load8<kStream>(in, hi);
      if (bias) {
        const Vec8 ba = load8<kTable>(bias, lo), bb = load8<kTable>(bias, hi);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          a.v[i] = __fadd_rn(a.v[i], ba.v[i]);
          b.v[i] = __fadd_rn(b.v[i], bb.v[i]);
        }
      }
      if (head < n_rot_heads) {
        const Vec8 c = load8<kTable>(cs, piece * 8), s = load8<kTable>(sn, piece * 8);
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float x1 = a.v[i], x2 = b.v[i];
          if (EXACT && !FMA) { // run.cpp:519-520 built without FMA: four products, then -, +
            a.v[i] = __fsub_rn(__fmul_rn(x1, c.v[i]), __fmul_rn(x2, s.v[i]));
            b.v[i] = __fadd_rn(__fmul_rn(x2, c.v[i]), __fmul_rn(x1, s.v[i]));
          } else { // the reference's GPU form (kernels/fast_common.hpp:25-28)
            a.v[i] = __fmaf_rn(x1, c.v[i], -__fmul_rn(x2, s.v[i]));
            b.v[i] = __fmaf_rn(x2, c.v[i], __fmul_rn(x1, s.v[i]));
          }
        }
      }
      store8(out, lo, a);
      store8(out, hi, b);
    }
  }
}

// Any head_dim (even) and alignment: one rotation pair per thread step.
template <typename IT, typename OT, bool EXACT, bool FMA>
__global__ void bias_rope_rows_generic(const IT *qkv_in, long in_stride,
                                       const float *__restrict__ bias,
                                       const int *__restrict__ pos, int pos_scalar,
                                       const float *__restrict__ cos_tab,
                                       const float *__restrict__ sin_tab, int n_pos,
                                       int n_rot_heads, int n_heads, int head_dim, OT *qkv_out,
                                       long out_stride, int T) {
  const int half = head_dim >> 1, items = n_heads * half;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    int p = pos ? pos[row] : pos_scalar;
    p = p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
    const float *cs = cos_tab + (size_t)p * half, *sn = sin_tab + (size_t)p * half;
    const IT *in = qkv_in + (size_t)row * in_stride;
    OT *out = qkv_out + (size_t)row * out_stride;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
      const int head = item / half, i = item - head * half;
      const size_t lo = (size_t)head * head_dim + i, hi = lo + half;
      float x1 = load1(in + lo), x2 = load1(in + hi);
      if (bias) {
        x1 = __fadd_rn(x1, bias[lo]);
        x2 = __fadd_rn(x2, bias[hi]);
      }
      float o1 = x1, o2 = x2;
      if (head < n_rot_heads) {
        const float c = cs[i], s = sn[i];
        if (EXACT && !FMA) {
          o1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
          o2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
        } else {
          o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
          o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
        }
      }
      store1(out + lo, o1);
      store1(out + hi, o2);
    }
  }
}

struct Args {
  const void *in;
  long in_stride;
  const float *bias;
  const int *pos;
  int pos_scalar;
  const float *cos_tab, *sin_tab;
  int n_pos, n_q, n_kv, head_dim;
  void *out;
  long out_stride;
  int T;
};

template <typename IT, typename OT, bool EXACT, bool FMA> int launch(cudaStream_t s, const Args &a) {
  const int n_heads = a.n_q + 2 * a.n_kv, n_rot = a.n_q + a.n_kv;
  const IT *in = static_cast<const IT *>(a.in);
  OT *out = static_cast<OT *>(a.out);
  const bool vec = a.head_dim % 16 == 0 && aligned16(a.in) && aligned16(a.out) &&
                   (a.in_stride * sizeof(IT)) % 16 == 0 && (a.out_stride * sizeof(OT)) % 16 == 0 &&
                   (!a.bias || aligned16(a.bias)) && aligned16(a.cos_tab) && aligned16(a.sin_tab) &&
                   (a.head_dim / 2 * sizeof(float)) % 16 == 0;
  if (!vec) {
    bias_rope_rows_generic<IT, OT, EXACT, FMA><<<row_grid(a.T, 8), 256, 0, s>>>(
        in, a.in_stride, a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab, a.n_pos, n_rot, n_heads,
        a.head_dim, out, a.out_stride, a.T);
    return launch_status();
  }
  const int items = n_heads * (a.head_dim / 16);
  int threads = (items + 31) / 32 * 32;
  if (threads > 512)
    threads = 512;
  static int occ[17];
  auto k = bias_rope_rows<IT, OT, EXACT, FMA>;
  k<<<row_grid(a.T, blocks_per_sm(k, threads, &occ[threads / 32])), threads, 0, s>>>(
      in, a.in_stride, a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab, a.n_pos, n_rot, n_heads,
      a.head_dim, out, a.out_stride, a.T);
  return launch_status();
}

template <typename IT, typename OT> int launch_mode(cudaStream_t s, const Args &a, unsigned flags) {
  if (flags & GPTOSS_EXACT)
    return (flags & GPTOSS_FMA) ? launch<IT, OT, true, true>(s, a) : launch<IT, OT, true, false>(s, a);
  return launch<IT, OT, false, true>(s, a);
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_qkv_bias_rope(gptoss_stream_t stream, int T, const void *qkv_in,
                                    gptoss_dtype_t in_dtype, long in_row_stride,
                                    const float *bias, const int *pos, int pos_scalar,
                                    const float *cos_tab, const float *sin_tab, int n_pos,
                                    int n_q_heads, int n_kv_heads, int head_dim, void *qkv_out,
                                    gptoss_dtype_t out_dtype, long out_row_stride,
                                    unsigned flags) {
  using namespace gptoss;
  if (T < 0 || n_q_heads < 0 || n_kv_heads < 0 || n_q_heads + n_kv_heads <= 0 || head_dim <= 0 ||
      head_dim % 2 != 0 || n_pos <= 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype))
    return GPTOSS_ERR_BAD_ARG;
  const long width = (long)(n_q_heads + 2 * n_kv_heads) * head_dim;
  if (in_row_stride < width || out_row_stride < width)
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!qkv_in || !qkv_out || !cos_tab || !sin_tab)
    return GPTOSS_ERR_BAD_ARG;
  // In place only with identical layout: a thread overwrites exactly what it read.
  if (qkv_in == qkv_out && (in_dtype != out_dtype || in_row_stride != out_row_stride))
    return GPTOSS_ERR_BAD_ARG;
  const Args a{qkv_in, in_row_stride, bias,      pos,        pos_scalar,     cos_tab, sin_tab,
               n_pos,  n_q_heads,     n_kv_heads, head_dim,   qkv_out,        out_row_stride, T};
  cudaStream_t s = as_stream(stream);
  if (in_dtype == GPTOSS_F32)
    return out_dtype == GPTOSS_F32 ? launch_mode<float, float>(s, a, flags)
                                   : launch_mode<float, uint16_t>(s, a, flags);
  return out_dtype == GPTOSS_F32 ? launch_mode<uint16_t, float>(s, a, flags)
                                 : launch_mode<uint16_t, uint16_t>(s, a, flags);
}
