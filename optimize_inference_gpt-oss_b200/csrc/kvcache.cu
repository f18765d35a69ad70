// KV-cache write of one decode step (gptoss_kv_cache_write): the step on the far
// side of the RoPE kernel.  From each biased, rotated qkv row it stores the key
// heads as bf16 and the value heads as int8 codes plus one fp32 scale per
// (slot, head), in the layouts the reference's decode attention reads
// ("chunk64": a sequence's cache is cut into chunks of 64 slots and, inside a
// chunk, every key/value head keeps its 64 slots together).
//
// One block per row, one warp per key/value head at a time: lane l holds
// elements l and l + 32 of the 64-wide head, so the value head's max |v| is a
// 5-step shuffle reduction and the key head leaves as two coalesced 64-byte
// runs.  The op moves ~3 KB per row; it is latency-bound and short.
#include "common.cuh"

namespace gptoss {
namespace {

constexpr int kHeadDim = 64;

// Element (b, slot, g, i) of a chunk64 cache with kv_dim = n_kv_heads * 64.
__device__ __forceinline__ size_t chunk64_index(int b, int slot, int g, int i, int slots, int kv_dim) {
  return ((size_t)b * slots + (size_t)(slot & ~63)) * kv_dim + (size_t)g * 64 * 64 + (size_t)(slot & 63) * 64 + i;
}
// Byte of value code (b, slot, g, i): chunk64 blocks at one byte per element; inside a
// 16-slot tile the 4 codes of slots 4q..4q+3 for one dim sit together.
__device__ __forceinline__ size_t vcode_index(int b, int slot, int g, int i, int slots, int kv_dim) {
  return chunk64_index(b, slot & ~15, g, 0, slots, kv_dim) + ((slot >> 2) & 3) * 256 + (i >> 2) * 16 +
         (i & 3) * 4 + (slot & 3);
}
__device__ __forceinline__ size_t vscale_index(int b, int slot, int g, int slots, int kv_dim) {
  return chunk64_index(b, slot, g, 0, slots, kv_dim) / 64;
}

// What turns a raw qkv row into the row the cache is written from, for the launch that
// writes the cache from the rotation's INPUT (gptoss_qkv_bias_rope_kv at shapes its fused
// kernel does not take): bias, positions and the cos/sin tables.  A lane's two elements l and
// l + 32 of a 64-wide key head are one rotation pair.  tables == nullptr: rows are final.
struct Prep {
  const float *bias; // may be nullptr
  const int *pos;
  int pos_scalar;
  const float *cos_tab, *sin_tab; // [n_pos, 32]
  int n_pos;
  int separate_products; // the CPU build's form (no FMA): x1*c - x2*s from two rounded products
};

template <typename QT>
__global__ void __launch_bounds__(256)
    kv_cache_write_rows(const QT *__restrict__ qkv, long row_stride, int n_q_heads, int n_kv_heads,
                        uint16_t *__restrict__ kc, int8_t *__restrict__ vq, float *__restrict__ vs, int slots,
                        const int *__restrict__ slot_of_row, int slot_scalar, int T, Prep prep) {
  pdl_prologue();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int kv_dim = n_kv_heads * kHeadDim;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    int slot = slot_of_row ? __ldg(slot_of_row + row) : slot_scalar;
    if (slot < 0 || slot >= slots)
      continue; // a row without a place in the cache writes nothing
    const QT *k = qkv + (size_t)row * row_stride + (size_t)n_q_heads * kHeadDim;
    const QT *v = k + kv_dim;
    for (int g = warp; g < n_kv_heads; g += n_warps) {
      float k0 = load1(k + g * kHeadDim + lane), k1 = load1(k + g * kHeadDim + 32 + lane);
      float v0 = load1(v + g * kHeadDim + lane), v1 = load1(v + g * kHeadDim + 32 + lane);
      if (prep.cos_tab) { // the row is the rotation's input: bias, then rotate the key pair
        if (prep.bias) {
          const float *bk = prep.bias + (size_t)n_q_heads * kHeadDim + g * kHeadDim, *bv = bk + kv_dim;
          k0 = __fadd_rn(k0, bk[lane]), k1 = __fadd_rn(k1, bk[32 + lane]);
          v0 = __fadd_rn(v0, bv[lane]), v1 = __fadd_rn(v1, bv[32 + lane]);
        }
        int p = prep.pos ? __ldg(prep.pos + row) : prep.pos_scalar;
        p = p < 0 ? 0 : (p >= prep.n_pos ? prep.n_pos - 1 : p);
        const float c = prep.cos_tab[(size_t)p * 32 + lane], sn = prep.sin_tab[(size_t)p * 32 + lane];
        const float x1 = k0, x2 = k1;
        if (prep.separate_products) {
          k0 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
          k1 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
        } else {
          k0 = __fmaf_rn(x1, c, -__fmul_rn(x2, sn));
          k1 = __fmaf_rn(x2, c, __fmul_rn(x1, sn));
        }
      }
      // keys: bf16, round to nearest even (exact when the input already is bf16)
      kc[chunk64_index(row, slot, g, lane, slots, kv_dim)] = (uint16_t)f32_to_bf16_bits(k0);
      kc[chunk64_index(row, slot, g, 32 + lane, slots, kv_dim)] = (uint16_t)f32_to_bf16_bits(k1);
      // values: scale = max|v| / 127, code = round(v * 127 / max|v|)   (kernels/fast_misc.hpp:79-87)
      float amax = fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
      const float c0 = fminf(fmaxf(rintf(__fmul_rn(v0, inv)), -127.0f), 127.0f);
      const float c1 = fminf(fmaxf(rintf(__fmul_rn(v1, inv)), -127.0f), 127.0f);
      vq[vcode_index(row, slot, g, lane, slots, kv_dim)] = (int8_t)c0;
      vq[vcode_index(row, slot, g, 32 + lane, slots, kv_dim)] = (int8_t)c1;
      if (lane == 0)
        vs[vscale_index(row, slot, g, slots, kv_dim)] = __fdiv_rn(amax, 127.0f);
    }
  }
}

int launch_cache_write(cudaStream_t s, int T, const void *qkv, gptoss_dtype_t qkv_dtype, long row_stride,
                       int n_q_heads, int n_kv_heads, uint16_t *kc, int8_t *vq, float *vs, int slots,
                       const int *slot_of_row, int slot_scalar, const Prep &prep) {
  const int grid = row_grid(T, 8);
  if (qkv_dtype == GPTOSS_F32)
    launch_kernel(kv_cache_write_rows<float>, dim3(grid), dim3(256), 0, s, static_cast<const float *>(qkv),
                  row_stride, n_q_heads, n_kv_heads, kc, vq, vs, slots, slot_of_row, slot_scalar, T, prep);
  else
    launch_kernel(kv_cache_write_rows<uint16_t>, dim3(grid), dim3(256), 0, s,
                  static_cast<const uint16_t *>(qkv), row_stride, n_q_heads, n_kv_heads, kc, vq, vs, slots,
                  slot_of_row, slot_scalar, T, prep);
  return launch_status();
}

} // namespace

// The cache write of gptoss_qkv_bias_rope_kv as a launch of its own, from the rotation's
// input rows: the same fp32 values the fused kernel holds in registers, whatever type the
// rotated rows are stored as.  64-wide heads; arguments already validated by the caller.
int kv_cache_write_from_input(cudaStream_t s, int T, const void *qkv_in, gptoss_dtype_t in_dtype,
                              long in_row_stride, const float *bias, const int *pos, int pos_scalar,
                              const float *cos_tab, const float *sin_tab, int n_pos, int n_q_heads,
                              int n_kv_heads, uint16_t *kc, int8_t *vq, float *vs, int slots,
                              const int *slot_of_row, int slot_scalar, unsigned flags) {
  const Prep prep = {bias, pos, pos_scalar, cos_tab, sin_tab, n_pos,
                     (flags & GPTOSS_EXACT) && !(flags & GPTOSS_FMA)};
  return launch_cache_write(s, T, qkv_in, in_dtype, in_row_stride, n_q_heads, n_kv_heads, kc, vq, vs, slots,
                            slot_of_row, slot_scalar, prep);
}

} // namespace gptoss

extern "C" int gptoss_kv_cache_write(gptoss_stream_t stream, int T, const void *qkv, gptoss_dtype_t qkv_dtype,
                                     long row_stride, int n_q_heads, int n_kv_heads, int head_dim,
                                     uint16_t *kc, int8_t *vq, float *vs, int slots, const int *slot_of_row,
                                     int slot_scalar, unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (T < 0 || n_q_heads < 0 || n_kv_heads <= 0 || slots <= 0 || !valid_dtype(qkv_dtype) ||
      row_stride < (long)(n_q_heads + 2 * n_kv_heads) * head_dim)
    return GPTOSS_ERR_BAD_ARG;
  if (head_dim != kHeadDim || slots % 64 != 0)
    return GPTOSS_ERR_UNSUPPORTED; // the chunk64 layouts are defined for 64-wide heads and whole chunks
  if (T == 0)
    return GPTOSS_OK;
  if (!qkv || !kc || !vq || !vs)
    return GPTOSS_ERR_BAD_ARG;
  {
    [[maybe_unused]] const size_t per_row = (size_t)slots * n_kv_heads * kHeadDim;
    GPTOSS_SPAN(qkv, strided_bytes(T, row_stride, (long)(n_q_heads + 2 * n_kv_heads) * head_dim, dtype_size(qkv_dtype)));
    GPTOSS_SPAN(kc, (size_t)T * per_row * 2);
    GPTOSS_SPAN(vq, (size_t)T * per_row);
    GPTOSS_SPAN(vs, (size_t)T * per_row / 64 * 4);
    GPTOSS_SPAN(slot_of_row, (size_t)T * 4);
  }
  const Prep none = {};
  return launch_cache_write(as_stream(stream), T, qkv, qkv_dtype, row_stride, n_q_heads, n_kv_heads, kc, vq, vs,
                            slots, slot_of_row, slot_scalar, none);
}
