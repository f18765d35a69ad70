// Residual add fused with RMSNorm (gptoss_add_rmsnorm).
//
// HBM-bound: per row the kernel must read x (4H bytes) and y (aH), and write x
// (4H) and out (aH).  Rows of up to 4096 elements take the loop-free form
// (add_rmsnorm_tile, one row per block, further down); wider rows the ring described
// here: one thread block works on one row at a time and walks the rows with a grid stride.  Rows are staged through a ring of shared-memory
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
// in float.  bf16 mode: kernels/fast_misc.hpp:29 in fp32, with the approximate reciprocal root
// (fast_inv_rms in common.cuh).
__device__ __forceinline__ double exact_inv_rms(double ss, int H) {
  double m = __ddiv_rn(ss, (double)H);
  m = __dadd_rn(m, (double)GPTOSS_RMS_EPS);
  return (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
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

// The loop-free form of add_rmsnorm_rows for H <= 4096: a block owns R consecutive rows, asks
// for all of them at once (x and the delta, cp.async into shared memory), normalises them
// with one barrier and exits; the hardware scheduler keeps the SMs stocked with fresh
// blocks.  Same chunk-to-thread mapping and summation order as the ring with one chunk
// per thread, hence the same bits.
#ifndef GPTOSS_NORM_TILE_NC
#define GPTOSS_NORM_TILE_NC 1 // chunks of 8 elements per thread in the one-row form
#endif
template <typename YT, typename OT, bool EXACT, int NC>
__global__ void add_rmsnorm_tile(float *x, const YT *__restrict__ y, const float *__restrict__ w, OT *out,
                                 int T, int H) {
  pdl_prologue();
  constexpr bool HAS_Y = !std::is_same<YT, NoY>::value;
  constexpr uint32_t SY = YSize<YT>::value;
  using Acc = typename std::conditional<EXACT, double, float>::type;
  extern __shared__ __align__(16) unsigned char rows[]; // the x row, then the delta row
  __shared__ Acc scratch[32];
  const long row = blockIdx.x;
  const uint32_t rows_a = smem_u32(rows);
  bool has[NC];
  uint32_t my_x[NC], my_y[NC];
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const int chunk = threadIdx.x + c * blockDim.x;
    has[c] = chunk < (H >> 3);
    my_x[c] = (uint32_t)chunk * 32u, my_y[c] = (uint32_t)H * 4u + (uint32_t)chunk * 8u * SY;
  }
#pragma unroll
  for (int c = 0; c < NC; c++)
    if (has[c]) {
      const unsigned char *xr = reinterpret_cast<const unsigned char *>(x + (size_t)row * H) + my_x[c];
      cp16_cg(rows_a + my_x[c], xr);
      cp16_cg(rows_a + my_x[c] + 16, xr + 16);
      if constexpr (HAS_Y) {
        const unsigned char *yr = reinterpret_cast<const unsigned char *>(y + (size_t)row * H) + (my_y[c] - (uint32_t)H * 4u);
        cp16_cg(rows_a + my_y[c], yr);
        if constexpr (SY == 4)
          cp16_cg(rows_a + my_y[c] + 16, yr + 16);
      }
    }
  cp_async_commit();
  Vec8 ws[NC];
#pragma unroll
  for (int c = 0; c < NC; c++)
    if (has[c])
      ws[c] = load8<kTable>(w, (size_t)(threadIdx.x + c * blockDim.x) * 8);
  cp_async_wait<0>(); // a thread reads back only what it copied itself: no barrier needed

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  Vec8 xs[NC];
  Acc ss = 0;
#pragma unroll
  for (int c = 0; c < NC; c++)
    if (has[c]) {
      xs[c] = floats_of(lds16(rows_a + my_x[c]), lds16(rows_a + my_x[c] + 16));
      if constexpr (HAS_Y) {
        Vec8 ys;
        if constexpr (SY == 2)
          ys = widen8(lds16(rows_a + my_y[c]));
        else
          ys = floats_of(lds16(rows_a + my_y[c]), lds16(rows_a + my_y[c] + 16));
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
  ss = warp_sum(ss);
  if (lane == 0)
    scratch[warp] = ss;
  __syncthreads();
  Acc t = lane < n_warps ? scratch[lane] : Acc(0);
  t = warp_sum(t); // every lane takes part, also those without a chunk
  [[maybe_unused]] double inv_d = 0.0;
  [[maybe_unused]] float inv_f = 0.0f;
  if constexpr (EXACT)
    inv_d = exact_inv_rms(t, H);
  else
    inv_f = fast_inv_rms(t, H);
#pragma unroll
  for (int c = 0; c < NC; c++)
    if (has[c]) {
      const size_t e = (size_t)(threadIdx.x + c * blockDim.x) * 8;
      if constexpr (HAS_Y)
        store8(x + (size_t)row * H, e, xs[c], false);
      Vec8 o;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        if constexpr (EXACT)
          o.v[i] = (float)__dmul_rn((double)ws[c].v[i], __dmul_rn(inv_d, (double)xs[c].v[i]));
        else
          o.v[i] = __fmul_rn(ws[c].v[i], __fmul_rn(inv_f, xs[c].v[i]));
      }
      store8(out + (size_t)row * H, e, o);
    }
}

// Embedding gather fused with the norm that follows it (gptoss_embed_rmsnorm): the same
// ring, but a stage is filled from table row ids[row] (bf16 or fp32) instead of from x,
// and the widened row is stored to x as well as normalised.  Against the two separate
// launches this leaves out one read of x (4H bytes per row) and one launch.  The ids a
// block needs are fetched one iteration before their use; an id outside [0, V) stands
// for a row of zeros, as in the plain gather.
template <typename TT, typename OT, bool EXACT, int NC, int STAGES>
__global__ void embed_rmsnorm_rows(const TT *__restrict__ table, const int *__restrict__ ids, int V,
                                   float *__restrict__ x, const float *__restrict__ w,
                                   OT *__restrict__ out, int T, int H) {
  pdl_prologue();
  constexpr int ST = sizeof(TT);
  using Acc = typename std::conditional<EXACT, double, float>::type;
  extern __shared__ __align__(16) unsigned char ring[];
  __shared__ Acc scratch[2][32];
  const size_t stage_bytes = (size_t)H * ST;
  const int n_chunks = H >> 3;

  bool has[NC];
  Vec8 ws[NC];
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const int chunk = threadIdx.x + c * blockDim.x;
    has[c] = chunk < n_chunks;
    if (has[c])
      ws[c] = load8<kTable>(w, (size_t)chunk * 8);
  }

  auto row_id = [&](long row) -> int {
    if (row >= T)
      return -1;
    const int id = __ldg(ids + row);
    return id >= 0 && id < V ? id : -1;
  };
  auto issue = [&](int id, int stage) {
    if (id < 0)
      return;
    unsigned char *sx = ring + (size_t)stage * stage_bytes;
    const TT *tr = table + (size_t)id * H;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        const int chunk = threadIdx.x + c * blockDim.x;
        cp_async16(sx + (size_t)chunk * 8 * ST, tr + (size_t)chunk * 8);
        if constexpr (ST == 4)
          cp_async16(sx + (size_t)chunk * 32 + 16, tr + (size_t)chunk * 8 + 4);
      }
  };

  const long step = gridDim.x;
  long row = blockIdx.x;
  {
    int first[STAGES - 1];
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++)
      first[s] = row_id(row + s * step);
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
      issue(first[s], s);
      cp_async_commit();
    }
  }
  int id_here = row_id(row);                         // of the row being normalised
  int id_ahead = row_id(row + (STAGES - 1) * step);  // of the row whose copy is issued next
  int stage = 0, flip = 0;
  for (; row < T; row += step, flip ^= 1) {
    issue(id_ahead, stage == 0 ? STAGES - 1 : stage - 1);
    cp_async_commit();
    const bool live = id_here >= 0;
    id_here = row_id(row + step);
    id_ahead = row_id(row + STAGES * step);
    cp_async_wait<STAGES - 1>();

    const unsigned char *sx = ring + (size_t)stage * stage_bytes;
    Vec8 xs[NC];
    Acc ss = 0;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        const int chunk = threadIdx.x + c * blockDim.x;
        if (!live) {
#pragma unroll
          for (int i = 0; i < 8; i++)
            xs[c].v[i] = 0.0f;
        } else if constexpr (ST == 2) {
          xs[c] = widen8(*reinterpret_cast<const uint4 *>(sx + (size_t)chunk * 16));
        } else {
          const uint4 a = *reinterpret_cast<const uint4 *>(sx + (size_t)chunk * 32);
          const uint4 b = *reinterpret_cast<const uint4 *>(sx + (size_t)chunk * 32 + 16);
          xs[c].v[0] = __uint_as_float(a.x), xs[c].v[1] = __uint_as_float(a.y),
          xs[c].v[2] = __uint_as_float(a.z), xs[c].v[3] = __uint_as_float(a.w),
          xs[c].v[4] = __uint_as_float(b.x), xs[c].v[5] = __uint_as_float(b.y),
          xs[c].v[6] = __uint_as_float(b.z), xs[c].v[7] = __uint_as_float(b.w);
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

// The same operation without the loop, the form used whenever H <= 4096.  A block owns R
// consecutive rows and a thread one 8-element chunk of each; the block asks for all R table
// rows at once (cp.async into shared memory, so the data in flight costs no registers); the
// hardware scheduler replaces blocks as they exit (R = 4 for a 4096-row launch: 1024 blocks).
// The R sums of squares share one barrier.  Chunk-to-thread mapping and
// summation order are those of add_rmsnorm_rows with one chunk per thread, which makes the
// result the same bits as the two separate launches.
template <typename TT, typename OT, bool EXACT, int R>
__global__ void embed_rmsnorm_tile(const TT *__restrict__ table, const int *__restrict__ ids, int V,
                                   float *__restrict__ x, const float *__restrict__ w,
                                   OT *__restrict__ out, int T, int H) {
  pdl_prologue();
  constexpr int ST = sizeof(TT);
  using Acc = typename std::conditional<EXACT, double, float>::type;
  extern __shared__ __align__(16) unsigned char rows[]; // R rows of H table elements
  __shared__ Acc scratch[R][32];
  const int chunk = threadIdx.x;
  const bool has = chunk < (H >> 3);
  const long row0 = (long)blockIdx.x * R;
  const size_t row_bytes = (size_t)H * ST;

  int id[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    id[r] = -1;
    if (row0 + r < T) {
      const int v = __ldg(ids + row0 + r);
      if (v >= 0 && v < V)
        id[r] = v;
    }
  }
#pragma unroll
  for (int r = 0; r < R; r++)
    if (has && id[r] >= 0) {
      unsigned char *dst = rows + r * row_bytes + (size_t)chunk * 8 * ST;
      const TT *src = table + (size_t)id[r] * H + (size_t)chunk * 8;
      cp_async16(dst, src);
      if constexpr (ST == 4)
        cp_async16(dst + 16, src + 4);
    }
  cp_async_commit();
  Vec8 ws; // the gain: asked for now, so that its latency passes under the rows'
  if (has)
    ws = load8<kTable>(w, (size_t)chunk * 8);
  cp_async_wait<0>(); // a thread reads back only what it copied itself: no barrier needed
  auto values = [&](int r) {
    Vec8 v;
    const unsigned char *p = rows + r * row_bytes + (size_t)chunk * 8 * ST;
    if (id[r] < 0) {
#pragma unroll
      for (int i = 0; i < 8; i++)
        v.v[i] = 0.0f;
    } else if constexpr (ST == 2) {
      v = widen8(*reinterpret_cast<const uint4 *>(p));
    } else {
      const uint4 a = *reinterpret_cast<const uint4 *>(p), b = *reinterpret_cast<const uint4 *>(p + 16);
      v.v[0] = __uint_as_float(a.x), v.v[1] = __uint_as_float(a.y), v.v[2] = __uint_as_float(a.z),
      v.v[3] = __uint_as_float(a.w), v.v[4] = __uint_as_float(b.x), v.v[5] = __uint_as_float(b.y),
      v.v[6] = __uint_as_float(b.z), v.v[7] = __uint_as_float(b.w);
    }
    return v;
  };

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int r = 0; r < R; r++) {
    Acc ss = 0;
    if (has) {
      const Vec8 v = values(r);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        if constexpr (EXACT)
          ss = __dadd_rn(ss, (double)__fmul_rn(v.v[i], v.v[i]));
        else
          ss = fmaf(v.v[i], v.v[i], ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0)
      scratch[r][warp] = ss;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; r++) {
    Acc t = lane < n_warps ? scratch[r][lane] : Acc(0);
    t = warp_sum(t); // every lane takes part, also those without a chunk
    if (!has || row0 + r >= T)
      continue;
    const Vec8 v = values(r);
    const size_t e = (size_t)chunk * 8;
    store8(x + (size_t)(row0 + r) * H, e, v, false);
    Vec8 o;
    if constexpr (EXACT) {
      const double inv = exact_inv_rms(t, H);
#pragma unroll
      for (int i = 0; i < 8; i++)
        o.v[i] = (float)__dmul_rn((double)ws.v[i], __dmul_rn(inv, (double)v.v[i]));
    } else {
      const float inv = fast_inv_rms(t, H);
#pragma unroll
      for (int i = 0; i < 8; i++)
        o.v[i] = __fmul_rn(ws.v[i], __fmul_rn(inv, v.v[i]));
    }
    store8(out + (size_t)(row0 + r) * H, e, o);
  }
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
    if (nc == 1) { // H <= 4096: one row per block, no loop (measured against 2 and 4 rows per block and the ring)
      auto k = add_rmsnorm_tile<YT, OT, EXACT, GPTOSS_NORM_TILE_NC>;
      const int tile_threads = ((n_chunks + GPTOSS_NORM_TILE_NC - 1) / GPTOSS_NORM_TILE_NC + 31) / 32 * 32;
      if (blocks_per_sm_smem(k, tile_threads, stage_bytes) >= 1) {
        launch_kernel(k, dim3((unsigned)T), dim3(tile_threads), stage_bytes, s, x, yp, w, op, T, H);
        return launch_status();
      }
    }
#define GPTOSS_NORM_CASE(NC_, ST_)                                                                \
  if (nc == NC_ && stages == ST_)                                                                 \
  st = launch_pipe<YT, OT, EXACT, NC_, ST_>(s, T, x, yp, w, op, H, threads, smem)
    GPTOSS_NORM_CASE(2, 4);
    GPTOSS_NORM_CASE(2, 3);
    GPTOSS_NORM_CASE(2, 2);
    GPTOSS_NORM_CASE(4, 3);
    GPTOSS_NORM_CASE(4, 2);
#undef GPTOSS_NORM_CASE
    if (st != GPTOSS_ERR_UNSUPPORTED)
      return st;
  }
  note_generic_launch();
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

template <typename TT, typename OT, bool EXACT, int NC>
int launch_embed_pipe(cudaStream_t s, int T, const TT *table, const int *ids, int V, float *x, const float *w,
                      OT *out, int H, int threads, size_t smem) {
  auto k = embed_rmsnorm_rows<TT, OT, EXACT, NC, 4>;
  const int per_sm = blocks_per_sm_smem(k, threads, smem);
  if (per_sm < 1)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(k, dim3(row_grid(T, per_sm)), dim3(threads), smem, s, table, ids, V, x, w, out, T, H);
  return launch_status();
}

// GPTOSS_ERR_UNSUPPORTED: the shape or alignment is not one the fused kernel takes.
template <typename TT, typename OT, bool EXACT>
int launch_embed(cudaStream_t s, int T, const void *table, const int *ids, int V, float *x, const float *w,
                 void *out, int H) {
  const size_t stage_bytes = (size_t)H * sizeof(TT);
  if (H % 8 != 0 || H > 8 * 512 * 4 || stage_bytes * 4 > 200 * 1024 || !aligned16(table) || !aligned16(x) ||
      !aligned16(w) || !aligned16(out))
    return GPTOSS_ERR_UNSUPPORTED;
  const int n_chunks = H / 8;
  const int nc = n_chunks <= 512 ? 1 : (n_chunks <= 1024 ? 2 : 4);
  const int threads = ((n_chunks + nc - 1) / nc + 31) / 32 * 32;
  const TT *tp = static_cast<const TT *>(table);
  OT *op = static_cast<OT *>(out);
  if (nc == 1) {
    // rows per block: as few as still let every block be resident at once, at most 4
    // (and no more than fit in shared memory beside a second block)
    // (4 rows per block measured a little faster than 8 at 4096 and 16,384 rows: 20.0 against 20.9 us, 67.5 against 68.4)
    const int r_fit = stage_bytes * 4 <= 100 * 1024 ? 4 : (stage_bytes * 2 <= 100 * 1024 ? 2 : 1);
    int r = 1;
    while (r < r_fit) {
      const long slots = r == 1   ? (long)sm_count() * blocks_per_sm_smem(embed_rmsnorm_tile<TT, OT, EXACT, 1>, threads, stage_bytes)
                         : r == 2 ? (long)sm_count() * blocks_per_sm_smem(embed_rmsnorm_tile<TT, OT, EXACT, 2>, threads, stage_bytes * 2)
                                  : (long)sm_count() * blocks_per_sm_smem(embed_rmsnorm_tile<TT, OT, EXACT, 4>, threads, stage_bytes * 4);
      if ((T + r - 1) / r <= slots)
        break;
      r *= 2;
    }
    const unsigned blocks = (unsigned)((T + r - 1) / r);
    const size_t smem = stage_bytes * r;
#define GPTOSS_TILE_CASE(R_)                                                                              \
  if (r == R_) {                                                                                          \
    if (blocks_per_sm_smem(embed_rmsnorm_tile<TT, OT, EXACT, R_>, threads, smem) < 1)                     \
      return GPTOSS_ERR_UNSUPPORTED;                                                                      \
    launch_kernel(embed_rmsnorm_tile<TT, OT, EXACT, R_>, dim3(blocks), dim3(threads), smem, s, tp, ids, V, x, w, op, \
                  T, H);                                                                                  \
  }
    GPTOSS_TILE_CASE(1);
    GPTOSS_TILE_CASE(2);
    GPTOSS_TILE_CASE(4);
#undef GPTOSS_TILE_CASE
    return launch_status();
  }
  if (nc == 2)
    return launch_embed_pipe<TT, OT, EXACT, 2>(s, T, tp, ids, V, x, w, op, H, threads, stage_bytes * 4);
  return launch_embed_pipe<TT, OT, EXACT, 4>(s, T, tp, ids, V, x, w, op, H, threads, stage_bytes * 4);
}

template <bool EXACT>
int launch_embed_types(cudaStream_t s, int T, const void *table, gptoss_dtype_t table_dtype, const int *ids, int V,
                       float *x, const float *w, void *out, gptoss_dtype_t out_dtype, int H) {
  if (table_dtype == GPTOSS_BF16)
    return out_dtype == GPTOSS_BF16 ? launch_embed<uint16_t, uint16_t, EXACT>(s, T, table, ids, V, x, w, out, H)
                                    : launch_embed<uint16_t, float, EXACT>(s, T, table, ids, V, x, w, out, H);
  return out_dtype == GPTOSS_BF16 ? launch_embed<float, uint16_t, EXACT>(s, T, table, ids, V, x, w, out, H)
                                  : launch_embed<float, float, EXACT>(s, T, table, ids, V, x, w, out, H);
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
  GPTOSS_SPAN(x, (size_t)T * H * 4);
  GPTOSS_SPAN(y, (size_t)T * H * dtype_size(y_dtype));
  GPTOSS_SPAN(weight, (size_t)H * 4);
  GPTOSS_SPAN(out, (size_t)T * H * dtype_size(out_dtype));
  cudaStream_t s = as_stream(stream);
  return (flags & GPTOSS_EXACT) ? launch_y<true>(s, T, x, y, y_dtype, weight, out, out_dtype, H)
                                : launch_y<false>(s, T, x, y, y_dtype, weight, out, out_dtype, H);
}

extern "C" int gptoss_embed_rmsnorm(gptoss_stream_t stream, int T, const void *table, gptoss_dtype_t table_dtype,
                                    int V, const int *ids, float *x, const float *weight, void *out,
                                    gptoss_dtype_t out_dtype, int H, unsigned flags) {
  using namespace gptoss;
  if (T < 0 || H <= 0 || V <= 0 || !valid_dtype(table_dtype) || !valid_dtype(out_dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!table || !ids || !x || !weight || !out || out == (void *)x)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(table, (size_t)V * H * dtype_size(table_dtype));
  GPTOSS_SPAN(ids, (size_t)T * 4);
  GPTOSS_SPAN(x, (size_t)T * H * 4);
  GPTOSS_SPAN(weight, (size_t)H * 4);
  GPTOSS_SPAN(out, (size_t)T * H * dtype_size(out_dtype));
  int st;
  {
    const PdlScope pdl(flags);
    cudaStream_t s = as_stream(stream);
    st = (flags & GPTOSS_EXACT)
             ? launch_embed_types<true>(s, T, table, table_dtype, ids, V, x, weight, out, out_dtype, H)
             : launch_embed_types<false>(s, T, table, table_dtype, ids, V, x, weight, out, out_dtype, H);
  }
  if (st != GPTOSS_ERR_UNSUPPORTED)
    return st;
  // odd H or alignment: the two separate kernels, which take anything
  st = gptoss_embed(stream, T, table, table_dtype, V, ids, x, GPTOSS_F32, H, flags);
  return st != GPTOSS_OK ? st : gptoss_add_rmsnorm(stream, T, x, nullptr, GPTOSS_F32, weight, out, out_dtype, H, flags);
}
