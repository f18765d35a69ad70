// QKV bias add fused with YaRN RoPE (gptoss_qkv_bias_rope).
//
// Per row the kernel reads the fused q|k|v row once and writes it once; the
// bias (one row for the launch) and the cos/sin row of the token's position are
// small.  A thread owns one (head, piece) item for the whole launch: 8
// consecutive elements of the head's first half and the 8 elements head_dim/2
// further on -- the two halves of eight rotation pairs -- so its slice of the
// bias lives in registers, every access is 128 bits wide, and no thread needs
// another thread's row data.  Value heads use the same items and skip the
// rotation.  Rows are staged through a ring of two shared-memory buffers filled by
// cp.async (the next row of the block's walk is in flight while this one is
// rotated; three blocks per SM); the cos/sin row of each staged token travels with
// it, one copy per warp, so the arithmetic of a row waits on nothing but its own stage.
#include "common.cuh"

namespace gptoss {
namespace {

template <typename T> __device__ __forceinline__ Vec8 smem_load8(const unsigned char *p) {
  if constexpr (sizeof(T) == 2) {
    return widen8(*reinterpret_cast<const uint4 *>(p));
  } else {
    const uint4 a = *reinterpret_cast<const uint4 *>(p), b = *reinterpret_cast<const uint4 *>(p + 16);
    Vec8 v;
    v.v[0] = __uint_as_float(a.x), v.v[1] = __uint_as_float(a.y), v.v[2] = __uint_as_float(a.z),
    v.v[3] = __uint_as_float(a.w), v.v[4] = __uint_as_float(b.x), v.v[5] = __uint_as_float(b.y),
    v.v[6] = __uint_as_float(b.z), v.v[7] = __uint_as_float(b.w);
    return v;
  }
}

template <typename T> __device__ __forceinline__ void smem_store8(unsigned char *p, const Vec8 &v) {
  if constexpr (sizeof(T) == 2) {
    *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf16(v.v[0], v.v[1]), pack_bf16(v.v[2], v.v[3]),
                                               pack_bf16(v.v[4], v.v[5]), pack_bf16(v.v[6], v.v[7]));
  } else {
    *reinterpret_cast<uint4 *>(p) = make_uint4(__float_as_uint(v.v[0]), __float_as_uint(v.v[1]),
                                               __float_as_uint(v.v[2]), __float_as_uint(v.v[3]));
    *reinterpret_cast<uint4 *>(p + 16) = make_uint4(__float_as_uint(v.v[4]), __float_as_uint(v.v[5]),
                                                    __float_as_uint(v.v[6]), __float_as_uint(v.v[7]));
  }
}

template <bool EXACT, bool FMA>
__device__ __forceinline__ void rotate8(Vec8 &a, Vec8 &b, const Vec8 &c, const Vec8 &s) {
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

// Where the rotated keys and the values of a row also go when the launch writes the KV
// cache (gptoss_qkv_bias_rope_kv): the caches in the chunk64 layouts, 64-wide heads.
struct Cache {
  uint16_t *kc;
  int8_t *vq;
  float *vs;
  int slots;
  const int *slot_of_row;
  int slot_scalar;
  int n_q_heads, n_kv_heads;
};

// Element (b, slot, g, i) of a chunk64 cache with kv_dim = n_kv_heads * 64.
__device__ __forceinline__ size_t chunk64_at(int b, int slot, int g, int i, int slots, int kv_dim) {
  return ((size_t)b * slots + (size_t)(slot & ~63)) * kv_dim + (size_t)g * 64 * 64 + (size_t)(slot & 63) * 64 + i;
}

// blockDim.x >= n_heads * (head_dim / 16); thread t owns item t.
// Stage layout: [row: width * sizeof(IT)] [per warp: cos (half floats), sin (half floats)].
// KV: the launch also writes the row's keys (bf16) and values (int8 codes + scale) into
// the caches, from the fp32 values it holds in registers (head_dim is 64 then, so a head is
// the 4 consecutive lanes of its 4 pieces and the value head's max |v| is two shuffles).
template <typename IT, typename OT, bool EXACT, bool FMA, int STAGES, bool KV>
__global__ void bias_rope_rows(const IT *qkv_in, long in_stride, const float *__restrict__ bias,
                               const int *__restrict__ pos, int pos_scalar,
                               const float *__restrict__ cos_tab,
                               const float *__restrict__ sin_tab, int n_pos, int n_rot_heads,
                               int n_heads, int head_dim, OT *qkv_out, long out_stride, int T,
                               Cache cache) {
  pdl_prologue();
  constexpr int SI = sizeof(IT);
  extern __shared__ __align__(16) unsigned char ring[];
  const int half = head_dim >> 1, pieces = half >> 3, items = n_heads * pieces;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const size_t row_bytes = (size_t)n_heads * head_dim * SI;
  const size_t trig_bytes = (size_t)half * 8; // cos + sin of one position
  const size_t stage_bytes = row_bytes + (size_t)n_warps * trig_bytes;

  const bool active = (int)threadIdx.x < items;
  const int head = active ? threadIdx.x / pieces : 0, piece = active ? threadIdx.x - head * pieces : 0;
  const size_t lo = (size_t)head * head_dim + piece * 8, hi = lo + half;
  const bool rotates = head < n_rot_heads;
  Vec8 ba, bb;
#pragma unroll
  for (int i = 0; i < 8; i++)
    ba.v[i] = bb.v[i] = 0.0f;
  if (bias && active) {
    ba = load8<kTable>(bias, lo);
    bb = load8<kTable>(bias, hi);
  }

  auto position = [&](long row) {
    int p = pos ? __ldg(pos + row) : pos_scalar;
    return p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
  };
  auto issue = [&](long row, int stage, int p) {
    unsigned char *sr = ring + (size_t)stage * stage_bytes;
    if (active) {
      const IT *in = qkv_in + (size_t)row * in_stride;
      cp_async16(sr + lo * SI, in + lo);
      cp_async16(sr + hi * SI, in + hi);
      if constexpr (SI == 4) {
        cp_async16(sr + lo * SI + 16, in + lo + 4);
        cp_async16(sr + hi * SI + 16, in + hi + 4);
      }
    }
    // this warp's copy of the token's cos and sin rows: 16-byte pieces, one per lane
    unsigned char *st = sr + row_bytes + (size_t)warp * trig_bytes;
    const int per_table = half >> 2;
    for (int q = lane; q < 2 * per_table; q += 32) {
      const float *src = q < per_table ? cos_tab + (size_t)p * half + q * 4
                                       : sin_tab + (size_t)p * half + (q - per_table) * 4;
      cp_async16_cached(st + (size_t)q * 16, src);
    }
  };

  const long step = gridDim.x;
  long row = blockIdx.x;
  if (row >= T)
    return;
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if (row + s * step < T)
      issue(row + s * step, s, position(row + s * step));
    cp_async_commit();
  }
  int ahead_pos = (row + (STAGES - 1) * step < T) ? position(row + (STAGES - 1) * step) : 0;
  int stage = 0;
  for (; row < T; row += step) {
    {
      const long ahead = row + (STAGES - 1) * step;
      const int fill = stage == 0 ? STAGES - 1 : stage - 1;
      if (ahead < T)
        issue(ahead, fill, ahead_pos);
      cp_async_commit();
    }
    if (row + STAGES * step < T)
      ahead_pos = position(row + STAGES * step);
    cp_async_wait<STAGES - 1>();
    __syncwarp(); // the cos/sin pieces were copied by other lanes of this warp

    Vec8 a, b;
    if constexpr (KV) {
#pragma unroll
      for (int i = 0; i < 8; i++)
        a.v[i] = b.v[i] = 0.0f;
    }
    if (active) {
      const unsigned char *sr = ring + (size_t)stage * stage_bytes;
      a = smem_load8<IT>(sr + lo * SI), b = smem_load8<IT>(sr + hi * SI);
      if (bias) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          a.v[i] = __fadd_rn(a.v[i], ba.v[i]);
          b.v[i] = __fadd_rn(b.v[i], bb.v[i]);
        }
      }
      if (rotates) {
        const unsigned char *st = sr + row_bytes + (size_t)warp * trig_bytes;
        const Vec8 c = smem_load8<float>(st + (size_t)piece * 32);
        const Vec8 s = smem_load8<float>(st + (size_t)half * 4 + (size_t)piece * 32);
        rotate8<EXACT, FMA>(a, b, c, s);
      }
      OT *out = qkv_out + (size_t)row * out_stride;
      store8(out, lo, a);
      store8(out, hi, b);
    }
    if constexpr (KV) {
      // max |v| over the head: every lane takes part in the shuffles, whatever its head is
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; i++)
        amax = fmaxf(amax, fmaxf(fabsf(a.v[i]), fabsf(b.v[i])));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int slot = cache.slot_of_row ? __ldg(cache.slot_of_row + row) : cache.slot_scalar;
      if (active && head >= cache.n_q_heads && slot >= 0 && slot < cache.slots) {
        const int kv_dim = cache.n_kv_heads * 64;
        const int g = head - cache.n_q_heads;
        if (g < cache.n_kv_heads) { // a key head: two runs of 8 bf16 values
          uint16_t *k = cache.kc + chunk64_at((int)row, slot, g, 0, cache.slots, kv_dim);
          uint4 lo8, hi8;
          lo8.x = f32_to_bf16_bits(a.v[0]) | (f32_to_bf16_bits(a.v[1]) << 16);
          lo8.y = f32_to_bf16_bits(a.v[2]) | (f32_to_bf16_bits(a.v[3]) << 16);
          lo8.z = f32_to_bf16_bits(a.v[4]) | (f32_to_bf16_bits(a.v[5]) << 16);
          lo8.w = f32_to_bf16_bits(a.v[6]) | (f32_to_bf16_bits(a.v[7]) << 16);
          hi8.x = f32_to_bf16_bits(b.v[0]) | (f32_to_bf16_bits(b.v[1]) << 16);
          hi8.y = f32_to_bf16_bits(b.v[2]) | (f32_to_bf16_bits(b.v[3]) << 16);
          hi8.z = f32_to_bf16_bits(b.v[4]) | (f32_to_bf16_bits(b.v[5]) << 16);
          hi8.w = f32_to_bf16_bits(b.v[6]) | (f32_to_bf16_bits(b.v[7]) << 16);
          *reinterpret_cast<uint4 *>(k + piece * 8) = lo8;
          *reinterpret_cast<uint4 *>(k + 32 + piece * 8) = hi8;
        } else { // a value head: codes and one scale (kernels/fast_misc.hpp:79-87)
          const int gv = g - cache.n_kv_heads;
          const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
          // byte of code (slot, dim i): 16-slot tile, then ((slot >> 2) & 3) * 256 + (i >> 2) * 16 + (i & 3) * 4 + (slot & 3)
          int8_t *q = cache.vq + chunk64_at((int)row, slot & ~15, gv, 0, cache.slots, kv_dim) +
                      ((slot >> 2) & 3) * 256 + (slot & 3);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int i0 = piece * 8 + j, i1 = 32 + i0;
            const float c0 = fminf(fmaxf(rintf(__fmul_rn(a.v[j], inv)), -127.0f), 127.0f);
            const float c1 = fminf(fmaxf(rintf(__fmul_rn(b.v[j], inv)), -127.0f), 127.0f);
            q[(i0 >> 2) * 16 + (i0 & 3) * 4] = (int8_t)c0;
            q[(i1 >> 2) * 16 + (i1 & 3) * 4] = (int8_t)c1;
          }
          if (piece == 0)
            cache.vs[chunk64_at((int)row, slot, gv, 0, cache.slots, kv_dim) / 64] = __fdiv_rn(amax, 127.0f);
        }
      }
    }
    __syncwarp(); // all lanes are done with this stage's cos/sin before it is refilled
    stage = stage + 1 == STAGES ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

// The ring above written out for 64-wide heads, the width of both models, so that everything
// the general form computes per row from its arguments is a constant or a register here: a
// head is 4 consecutive threads, byte offsets inside a stage are 32-bit and fixed per thread,
// shared memory is addressed by 32-bit shared-space addresses, and the row, output and position
// pointers advance by addition.  The general kernel executes 268 instructions per thread and
// row at the models' shape and keeps the issue slots 72 % busy for 17 us (ncu); the
// arithmetic itself -- 16 bias adds, 32 rotation operations, 24 conversions -- is a third of
// that.  Same staging (ring of two rows, a cos/sin copy per warp through L1), same
// arithmetic, same bits.
template <typename IT, typename OT, bool EXACT, bool FMA>
__global__ void bias_rope_rows_hd64(const IT *qkv_in, long in_stride, const float *__restrict__ bias,
                                    const int *__restrict__ pos, int pos_scalar,
                                    const float *__restrict__ cos_tab, const float *__restrict__ sin_tab,
                                    int n_pos, int n_rot_heads, int n_heads, OT *qkv_out, long out_stride, int T) {
  pdl_prologue();
  constexpr uint32_t SI = sizeof(IT), SO = sizeof(OT);
  extern __shared__ __align__(16) unsigned char ring[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  const uint32_t row_bytes = (uint32_t)n_heads * 64u * SI, stage_bytes = row_bytes + (uint32_t)n_warps * 256u;
  const int head = tid >> 2, piece = tid & 3;
  const bool active = head < n_heads, rotates = head < n_rot_heads;
  const uint32_t lo = (uint32_t)head * 64u + (uint32_t)piece * 8u; // first element of the thread's low run; the high run is 32 on

  Vec8 ba, bb;
#pragma unroll
  for (int i = 0; i < 8; i++)
    ba.v[i] = bb.v[i] = 0.0f;
  if (bias && active) {
    ba = load8<kTable>(bias, lo);
    bb = load8<kTable>(bias, lo + 32);
  }

  // where things sit inside a stage, as byte offsets from the stage's shared-memory address
  const uint32_t d_lo = lo * SI, d_hi = d_lo + 32u * SI;                        // this thread's two runs of the row
  const uint32_t t_put = row_bytes + (uint32_t)warp * 256u + (uint32_t)lane * 16u; // lanes 0..15: the piece this lane copies
  const uint32_t t_cos = row_bytes + (uint32_t)warp * 256u + (uint32_t)piece * 32u; // this thread's 8 cosines; sines 128 on
  const float *trig_src = (lane < 8 ? cos_tab : sin_tab) + (lane & 7) * 4;      // + position * 32
  uint32_t cur = smem_u32(ring), nxt = cur + stage_bytes;

  const long step = gridDim.x;
  long row = blockIdx.x;
  if (row >= T)
    return;
  const unsigned char *in_row = reinterpret_cast<const unsigned char *>(qkv_in) + (size_t)row * in_stride * SI;
  const size_t in_step = (size_t)step * in_stride * SI;
  unsigned char *out_lo = reinterpret_cast<unsigned char *>(qkv_out) + (size_t)row * out_stride * SO + lo * SO;
  const size_t out_step = (size_t)step * out_stride * SO;
  const int *pos_at = pos ? pos + row : nullptr;

  auto position = [&](const int *at) {
    int p = at ? __ldg(at) : pos_scalar;
    return p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
  };
  auto issue = [&](const unsigned char *src, uint32_t stage, int p) {
    if (active) {
      cp16_cg(stage + d_lo, src + d_lo);
      cp16_cg(stage + d_hi, src + d_hi);
      if constexpr (SI == 4) {
        cp16_cg(stage + d_lo + 16, src + d_lo + 16);
        cp16_cg(stage + d_hi + 16, src + d_hi + 16);
      }
    }
    if (lane < 16)
      cp16_ca(stage + t_put, trig_src + (size_t)p * 32);
  };

  issue(in_row, cur, position(pos_at));
  cp_async_commit();
  long ahead = row + step;
  in_row += in_step;
  if (pos_at)
    pos_at += step;
  int ahead_pos = ahead < T ? position(pos_at) : 0;
  for (; row < T; row += step) {
    if (ahead < T)
      issue(in_row, nxt, ahead_pos);
    cp_async_commit();
    ahead += step;
    in_row += in_step;
    if (pos_at)
      pos_at += step;
    if (ahead < T)
      ahead_pos = position(pos_at);
    cp_async_wait<1>();
    __syncwarp(); // the cos/sin pieces were copied by other lanes of this warp

    if (active) {
      Vec8 a, b;
      if constexpr (SI == 2) {
        a = widen8(lds16(cur + d_lo));
        b = widen8(lds16(cur + d_hi));
      } else {
        a = floats_of(lds16(cur + d_lo), lds16(cur + d_lo + 16));
        b = floats_of(lds16(cur + d_hi), lds16(cur + d_hi + 16));
      }
      if (bias) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          a.v[i] = __fadd_rn(a.v[i], ba.v[i]);
          b.v[i] = __fadd_rn(b.v[i], bb.v[i]);
        }
      }
      if (rotates) {
        const Vec8 c = floats_of(lds16(cur + t_cos), lds16(cur + t_cos + 16));
        const Vec8 sn = floats_of(lds16(cur + t_cos + 128), lds16(cur + t_cos + 144));
        rotate8<EXACT, FMA>(a, b, c, sn);
      }
      if constexpr (SO == 2) {
        st_stream(out_lo, make_uint4(pack_bf16(a.v[0], a.v[1]), pack_bf16(a.v[2], a.v[3]), pack_bf16(a.v[4], a.v[5]),
                                     pack_bf16(a.v[6], a.v[7])));
        st_stream(out_lo + 64, make_uint4(pack_bf16(b.v[0], b.v[1]), pack_bf16(b.v[2], b.v[3]),
                                          pack_bf16(b.v[4], b.v[5]), pack_bf16(b.v[6], b.v[7])));
      } else {
        st_stream(out_lo, make_uint4(__float_as_uint(a.v[0]), __float_as_uint(a.v[1]), __float_as_uint(a.v[2]),
                                     __float_as_uint(a.v[3])));
        st_stream(out_lo + 16, make_uint4(__float_as_uint(a.v[4]), __float_as_uint(a.v[5]), __float_as_uint(a.v[6]),
                                          __float_as_uint(a.v[7])));
        st_stream(out_lo + 128, make_uint4(__float_as_uint(b.v[0]), __float_as_uint(b.v[1]), __float_as_uint(b.v[2]),
                                           __float_as_uint(b.v[3])));
        st_stream(out_lo + 144, make_uint4(__float_as_uint(b.v[4]), __float_as_uint(b.v[5]), __float_as_uint(b.v[6]),
                                           __float_as_uint(b.v[7])));
      }
    }
    out_lo += out_step;
    __syncwarp(); // all lanes are done with this stage's cos/sin before it is refilled
    const uint32_t t = cur;
    cur = nxt;
    nxt = t;
  }
  cp_async_wait<0>();
}

// The same operation with every row moved by the copy engine.  One thread asks for a whole
// qkv row and the cos and sin rows of its position with three bulk copies that signal the
// stage's mbarrier; the block rotates the row out of shared memory into one of OUTS output
// buffers, also in shared memory, and one bulk store sends that to global memory.  Rows in
// flight per block are set by the ring (STAGES) and cost no registers or LSU instructions;
// the bias slice stays in registers as above.  A stage is refilled right after the barrier
// that ends its row's reads; an output buffer is reused only after the bulk store that read
// it has finished reading (the issuing thread checks before the barrier of the row before).
//
// Asked for with GPTOSS_BULK_STAGE in flags; not the default, because on B200 it measured 5-10 %
// slower than the 16-byte cp.async ring above at every ring depth tried (4096 rows: 17.7 us
// against 16.8; that form needs no block barrier at all, this one needs one per row).
#ifndef GPTOSS_ROPE_BULK_STAGES
#define GPTOSS_ROPE_BULK_STAGES 3
#endif
#ifndef GPTOSS_ROPE_BULK_OUTS
#define GPTOSS_ROPE_BULK_OUTS 2
#endif
template <typename IT, typename OT, bool EXACT, bool FMA, int STAGES, int OUTS>
__global__ void bias_rope_rows_bulk(const IT *qkv_in, long in_stride, const float *__restrict__ bias,
                                    const int *__restrict__ pos, int pos_scalar,
                                    const float *__restrict__ cos_tab, const float *__restrict__ sin_tab,
                                    int n_pos, int n_rot_heads, int n_heads, int head_dim, OT *qkv_out,
                                    long out_stride, int T, unsigned int *giveups) {
  pdl_prologue();
  constexpr int SI = sizeof(IT), SO = sizeof(OT);
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long full[STAGES];
  const int half = head_dim >> 1, pieces = half >> 3, items = n_heads * pieces;
  const uint32_t in_bytes = (uint32_t)n_heads * head_dim * SI, out_bytes = (uint32_t)n_heads * head_dim * SO;
  const uint32_t trig_bytes = (uint32_t)half * 4, stage_bytes = in_bytes + 2 * trig_bytes;
  unsigned char *outs = smem + (size_t)STAGES * stage_bytes;

  const bool active = (int)threadIdx.x < items;
  const int head = active ? threadIdx.x / pieces : 0, piece = active ? threadIdx.x - head * pieces : 0;
  const size_t lo = (size_t)head * head_dim + piece * 8, hi = lo + half;
  const bool rotates = head < n_rot_heads;

  const long step = gridDim.x;
  long row = blockIdx.x;
  if (row >= T)
    return;
  auto position = [&](long r) {
    int p = pos ? __ldg(pos + r) : pos_scalar;
    return p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
  };
  auto issue = [&](long r, int stage, int p) { // one thread
    unsigned char *sr = smem + (size_t)stage * stage_bytes;
    mbar_expect(&full[stage], stage_bytes);
    bulk_load(sr, qkv_in + (size_t)r * in_stride, in_bytes, &full[stage]);
    bulk_load(sr + in_bytes, cos_tab + (size_t)p * half, trig_bytes, &full[stage]);
    bulk_load(sr + in_bytes + trig_bytes, sin_tab + (size_t)p * half, trig_bytes, &full[stage]);
  };
  int next_pos = 0; // thread 0: position of the row the next refill asks for
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; s++)
      mbar_init(&full[s], 1);
    mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int first[STAGES + 1]; // all position reads before the first copy is asked for
#pragma unroll
    for (int s = 0; s <= STAGES; s++)
      first[s] = row + s * step < T ? position(row + s * step) : 0;
#pragma unroll
    for (int s = 0; s < STAGES; s++)
      if (row + s * step < T)
        issue(row + s * step, s, first[s]);
    next_pos = first[STAGES];
  }
  Vec8 ba, bb;
#pragma unroll
  for (int i = 0; i < 8; i++)
    ba.v[i] = bb.v[i] = 0.0f;
  if (bias && active) {
    ba = load8<kTable>(bias, lo);
    bb = load8<kTable>(bias, hi);
  }

  int stage = 0, ob = 0;
  uint32_t parity = 0;
  bool gave_up = false;
  for (; row < T; row += step) {
    if (!mbar_wait(&full[stage], parity)) {
      gave_up = true;
      break;
    }
    unsigned char *sr = smem + (size_t)stage * stage_bytes;
    unsigned char *so = outs + (size_t)ob * out_bytes;
    if (active) {
      Vec8 a = smem_load8<IT>(sr + lo * SI), b = smem_load8<IT>(sr + hi * SI);
      if (bias) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          a.v[i] = __fadd_rn(a.v[i], ba.v[i]);
          b.v[i] = __fadd_rn(b.v[i], bb.v[i]);
        }
      }
      if (rotates) {
        const Vec8 c = smem_load8<float>(sr + in_bytes + (size_t)piece * 32);
        const Vec8 sn = smem_load8<float>(sr + in_bytes + trig_bytes + (size_t)piece * 32);
        rotate8<EXACT, FMA>(a, b, c, sn);
      }
      smem_store8<OT>(so + lo * SO, a);
      smem_store8<OT>(so + hi * SO, b);
    }
    fence_async_smem();
    if (threadIdx.x == 0)
      bulk_wait_read<OUTS - 2>(); // the buffer the next row writes is no longer being read
    __syncthreads();
    if (threadIdx.x == 0) {
      bulk_store(qkv_out + (size_t)row * out_stride, so, out_bytes);
      bulk_commit();
      const long refill = row + (long)STAGES * step;
      if (refill < T) {
        issue(refill, stage, next_pos);
        if (refill + step < T)
          next_pos = position(refill + step);
      }
    }
    ob = ob + 1 == OUTS ? 0 : ob + 1;
    if (++stage == STAGES) {
      stage = 0;
      parity ^= 1;
    }
  }
  if (threadIdx.x == 0) {
    bulk_wait_read<0>(); // shared memory must outlive the stores that read it
    if (gave_up) {
      if (giveups)
        atomicAdd(giveups, 1u);
      // copies that were asked for and not consumed: each gets one more bounded chance to
      // land before the block, and with it their destination, goes away
      for (int k = 0; k < STAGES; k++) {
        if (row + (long)k * step < T)
          (void)mbar_wait(&full[stage], parity);
        if (++stage == STAGES) {
          stage = 0;
          parity ^= 1;
        }
      }
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
  pdl_prologue();
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
  Cache cache; // cache.kc == nullptr: no cache write
  bool bulk_stage; // GPTOSS_BULK_STAGE: rows moved by cp.async.bulk instead of 16-byte cp.async
};

template <typename IT, typename OT, bool EXACT, bool FMA, int STAGES, bool KV>
int launch_pipe(cudaStream_t s, const Args &a, int threads, size_t smem) {
  auto k = bias_rope_rows<IT, OT, EXACT, FMA, STAGES, KV>;
  const int per_sm = blocks_per_sm_smem(k, threads, smem);
  if (per_sm < 1)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(k, dim3(row_grid(a.T, per_sm)), dim3(threads), smem, s, 
      static_cast<const IT *>(a.in), a.in_stride, a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab,
      a.n_pos, a.n_q + a.n_kv, a.n_q + 2 * a.n_kv, a.head_dim, static_cast<OT *>(a.out),
      a.out_stride, a.T, a.cache);
  return launch_status();
}

template <typename IT, typename OT, bool EXACT, bool FMA>
int launch_bulk(cudaStream_t s, const Args &a, int threads) {
  constexpr int STAGES = GPTOSS_ROPE_BULK_STAGES, OUTS = GPTOSS_ROPE_BULK_OUTS;
  static_assert(STAGES >= 1 && OUTS >= 2, "ring of at least one row, two output buffers");
  auto k = bias_rope_rows_bulk<IT, OT, EXACT, FMA, STAGES, OUTS>;
  const size_t width = (size_t)(a.n_q + 2 * a.n_kv) * a.head_dim;
  const size_t smem = STAGES * (width * sizeof(IT) + (size_t)a.head_dim * 4) + OUTS * width * sizeof(OT);
  const int per_sm = smem <= 200 * 1024 ? blocks_per_sm_smem(k, threads, smem) : 0;
  if (per_sm < 1)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(k, dim3(row_grid(a.T, per_sm)), dim3(threads), smem, s, static_cast<const IT *>(a.in), a.in_stride,
                a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab, a.n_pos, a.n_q + a.n_kv, a.n_q + 2 * a.n_kv,
                a.head_dim, static_cast<OT *>(a.out), a.out_stride, a.T, wait_giveups_word());
  return launch_status();
}

template <typename IT, typename OT, bool EXACT, bool FMA> int launch(cudaStream_t s, const Args &a) {
  const int n_heads = a.n_q + 2 * a.n_kv, n_rot = a.n_q + a.n_kv;
  const bool vec = a.head_dim % 16 == 0 && aligned16(a.in) && aligned16(a.out) &&
                   (a.in_stride * sizeof(IT)) % 16 == 0 && (a.out_stride * sizeof(OT)) % 16 == 0 &&
                   (!a.bias || aligned16(a.bias)) && aligned16(a.cos_tab) && aligned16(a.sin_tab) &&
                   (a.head_dim / 2 * sizeof(float)) % 16 == 0;
  const int items = n_heads * (a.head_dim / 16);
  if (vec && items <= 1024) {
    const int threads = (items + 31) / 32 * 32;
    const size_t stage_bytes = (size_t)n_heads * a.head_dim * sizeof(IT) +
                               (size_t)(threads / 32) * (size_t)a.head_dim * 4;
    // A ring of two: while a row is rotated the next one of the block's walk is in flight.  Deeper
    // rings (3 and 4 rows, which fit) measured slower on B200 -- 15.3 against 14.8 us per launch at
    // 4096 rows -- as did capping registers for a fourth resident block.
    int st = GPTOSS_ERR_UNSUPPORTED;
    if (a.head_dim == 64 && !a.cache.kc && !a.bulk_stage && stage_bytes * 2 <= 220 * 1024) { // the models' head width
      auto k = bias_rope_rows_hd64<IT, OT, EXACT, FMA>;
      const int per_sm = blocks_per_sm_smem(k, threads, stage_bytes * 2);
      if (per_sm >= 1) {
        launch_kernel(k, dim3(row_grid(a.T, per_sm)), dim3(threads), stage_bytes * 2, s, static_cast<const IT *>(a.in),
                      a.in_stride, a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab, a.n_pos, n_rot, n_heads,
                      static_cast<OT *>(a.out), a.out_stride, a.T);
        return launch_status();
      }
    }
    if (a.bulk_stage && !a.cache.kc) { // the copy-engine form, on request (falls through if it does not fit)
      st = launch_bulk<IT, OT, EXACT, FMA>(s, a, threads);
      if (st != GPTOSS_ERR_UNSUPPORTED)
        return st;
    }
    if (stage_bytes * 2 <= 220 * 1024) {
      if (a.cache.kc) { // with the cache write: 64-wide heads only, 16-byte key stores
        if (a.head_dim == 64 && aligned16(a.cache.kc))
          st = launch_pipe<IT, OT, EXACT, FMA, 2, true>(s, a, threads, stage_bytes * 2);
        return st;
      }
      st = launch_pipe<IT, OT, EXACT, FMA, 2, false>(s, a, threads, stage_bytes * 2);
      if (st != GPTOSS_ERR_UNSUPPORTED)
        return st;
    }
  }
  if (a.cache.kc)
    return GPTOSS_ERR_UNSUPPORTED; // the caller falls back to the two separate launches
  note_generic_launch();
  launch_kernel(bias_rope_rows_generic<IT, OT, EXACT, FMA>, dim3(row_grid(a.T, 8)), dim3(256), 0, s, 
      static_cast<const IT *>(a.in), a.in_stride, a.bias, a.pos, a.pos_scalar, a.cos_tab, a.sin_tab,
      a.n_pos, n_rot, n_heads, a.head_dim, static_cast<OT *>(a.out), a.out_stride, a.T);
  return launch_status();
}

template <typename IT, typename OT> int launch_mode(cudaStream_t s, const Args &a, unsigned flags) {
  if (flags & GPTOSS_EXACT)
    return (flags & GPTOSS_FMA) ? launch<IT, OT, true, true>(s, a) : launch<IT, OT, true, false>(s, a);
  return launch<IT, OT, false, true>(s, a);
}

} // namespace
} // namespace gptoss

namespace gptoss {
int kv_cache_write_from_input(cudaStream_t s, int T, const void *qkv_in, gptoss_dtype_t in_dtype,
                              long in_row_stride, const float *bias, const int *pos, int pos_scalar,
                              const float *cos_tab, const float *sin_tab, int n_pos, int n_q_heads,
                              int n_kv_heads, uint16_t *kc, int8_t *vq, float *vs, int slots,
                              const int *slot_of_row, int slot_scalar, unsigned flags);
namespace {

int run_bias_rope(gptoss_stream_t stream, int T, const void *qkv_in, gptoss_dtype_t in_dtype, long in_row_stride,
                  const float *bias, const int *pos, int pos_scalar, const float *cos_tab, const float *sin_tab,
                  int n_pos, int n_q_heads, int n_kv_heads, int head_dim, void *qkv_out, gptoss_dtype_t out_dtype,
                  long out_row_stride, const Cache &cache, unsigned flags) {
  const PdlScope pdl(flags);
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
  GPTOSS_SPAN(qkv_in, strided_bytes(T, in_row_stride, width, dtype_size(in_dtype)));
  GPTOSS_SPAN(qkv_out, strided_bytes(T, out_row_stride, width, dtype_size(out_dtype)));
  GPTOSS_SPAN(bias, (size_t)width * 4);
  GPTOSS_SPAN(pos, (size_t)T * 4);
  GPTOSS_SPAN(cos_tab, (size_t)n_pos * (head_dim / 2) * 4);
  GPTOSS_SPAN(sin_tab, (size_t)n_pos * (head_dim / 2) * 4);
  if (cache.kc) { // one cache of `slots` positions per row
    [[maybe_unused]] const size_t per_row = (size_t)cache.slots * cache.n_kv_heads * 64;
    GPTOSS_SPAN(cache.kc, (size_t)T * per_row * 2);
    GPTOSS_SPAN(cache.vq, (size_t)T * per_row);
    GPTOSS_SPAN(cache.vs, (size_t)T * per_row / 64 * 4);
    GPTOSS_SPAN(cache.slot_of_row, (size_t)T * 4);
  }
  const Args a{qkv_in, in_row_stride, bias,       pos,      pos_scalar, cos_tab,        sin_tab, n_pos,
               n_q_heads, n_kv_heads, head_dim, qkv_out,  out_row_stride, T,     cache,
               (flags & GPTOSS_BULK_STAGE) != 0};
  cudaStream_t s = as_stream(stream);
  if (in_dtype == GPTOSS_F32)
    return out_dtype == GPTOSS_F32 ? launch_mode<float, float>(s, a, flags)
                                   : launch_mode<float, uint16_t>(s, a, flags);
  return out_dtype == GPTOSS_F32 ? launch_mode<uint16_t, float>(s, a, flags)
                                 : launch_mode<uint16_t, uint16_t>(s, a, flags);
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
  const gptoss::Cache none = {};
  return gptoss::run_bias_rope(stream, T, qkv_in, in_dtype, in_row_stride, bias, pos, pos_scalar, cos_tab, sin_tab,
                               n_pos, n_q_heads, n_kv_heads, head_dim, qkv_out, out_dtype, out_row_stride, none,
                               flags);
}

extern "C" int gptoss_qkv_bias_rope_kv(gptoss_stream_t stream, int T, const void *qkv_in,
                                       gptoss_dtype_t in_dtype, long in_row_stride, const float *bias,
                                       const int *pos, int pos_scalar, const float *cos_tab,
                                       const float *sin_tab, int n_pos, int n_q_heads, int n_kv_heads,
                                       int head_dim, void *qkv_out, gptoss_dtype_t out_dtype,
                                       long out_row_stride, uint16_t *kc, int8_t *vq, float *vs, int slots,
                                       const int *slot_of_row, int slot_scalar, unsigned flags) {
  if (n_kv_heads <= 0 || slots <= 0)
    return GPTOSS_ERR_BAD_ARG;
  if (head_dim != 64 || slots % 64 != 0)
    return GPTOSS_ERR_UNSUPPORTED; // the chunk64 layouts are defined for 64-wide heads and whole chunks
  if (T > 0 && (!kc || !vq || !vs))
    return GPTOSS_ERR_BAD_ARG;
  const gptoss::Cache cache = {kc, vq, vs, slots, slot_of_row, slot_scalar, n_q_heads, n_kv_heads};
  int st = gptoss::run_bias_rope(stream, T, qkv_in, in_dtype, in_row_stride, bias, pos, pos_scalar, cos_tab,
                                 sin_tab, n_pos, n_q_heads, n_kv_heads, head_dim, qkv_out, out_dtype,
                                 out_row_stride, cache, flags);
  if (st != GPTOSS_ERR_UNSUPPORTED)
    return st;
  // A shape or alignment the fused kernel does not take: two launches.  The cache is written
  // first, from the input rows (bias and rotation redone in fp32 by that launch), so that it
  // holds what the fused kernel would have stored even when qkv_out is bf16 or is qkv_in.
  if (T > 0 && (!qkv_in || !cos_tab || !sin_tab || n_pos <= 0 || !gptoss::valid_dtype(in_dtype) ||
                in_row_stride < (long)(n_q_heads + 2 * n_kv_heads) * head_dim))
    return GPTOSS_ERR_BAD_ARG;
  if (T > 0) {
    const gptoss::PdlScope pdl(flags);
    st = gptoss::kv_cache_write_from_input(gptoss::as_stream(stream), T, qkv_in, in_dtype, in_row_stride, bias, pos,
                                           pos_scalar, cos_tab, sin_tab, n_pos, n_q_heads, n_kv_heads, kc, vq, vs,
                                           slots, slot_of_row, slot_scalar, flags);
    if (st != GPTOSS_OK)
      return st;
  }
  return gptoss_qkv_bias_rope(stream, T, qkv_in, in_dtype, in_row_stride, bias, pos, pos_scalar, cos_tab, sin_tab,
                              n_pos, n_q_heads, n_kv_heads, head_dim, qkv_out, out_dtype, out_row_stride, flags);
}
