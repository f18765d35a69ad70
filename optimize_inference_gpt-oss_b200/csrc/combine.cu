// Weighted expert combine fused with the residual and, optionally, the next
// RMSNorm (gptoss_moe_combine).
//
// Per token the kernel reads the residual row, k expert-output rows (through
// the own_row indirection) and k weights, and writes the residual row and,
// with the norm, one normalised row.  One thread block works on one token at a
// time and walks the tokens with a grid stride; a token's rows (about 34 KB at
// H = 2880, k = 4, bf16 experts) are staged through a ring of shared-memory
// buffers filled by cp.async one or more tokens ahead (two buffers at the model's
// shape: the next token's rows are in flight while this one is summed).  A thread owns NC chunks of 8 consecutive elements, copies
// those chunks of all k + 1 rows itself and reads only them back.  The small
// per-token routing data (row numbers, weights, expert ids) is fetched into
// registers one iteration before it is needed, so no load sits between a
// token's staged data and its arithmetic.
#include "common.cuh"

namespace gptoss {
namespace {

template <int KM> struct Routing { // weights and expert ids of one token
  float w[KM];
  int e[KM];
};
template <int KM> struct RowIds { // where the token's expert rows are, and whether it is live
  int row[KM];
  bool live;
  bool all_here; // every pair of the token has an expert row in Z (the usual case)
};

// MODE 0: fast (choice order, FMA).  MODE 1: exact (increasing expert, separate
// product and sum).  MODE 2: exact order with FMA.  KEQ: k == KM is known at compile
// time (the models' k = 4), which turns every "j < k" below into a constant.  Shared
// memory is addressed by 32-bit shared-space addresses and per-thread byte offsets
// that are fixed for the launch; a row's global addresses are one 64-bit
// multiply-add each.  (The first form of this kernel, with generic pointers and a
// run-time k throughout, executed 437 instructions per thread and token at the
// models' shape and kept the issue slots 63 % busy at 36 % occupancy.)
template <typename ZT, typename OT, int MODE, bool NORM, int KM, bool KEQ, int NC, int STAGES>
__global__ void combine_rows(float *x, const ZT *__restrict__ Z, const int *__restrict__ own_row,
                             const float *__restrict__ topk_w, const int *__restrict__ topk_e,
                             int k_arg, int H, const int *__restrict__ phys_of,
                             const float *__restrict__ norm_w, OT *__restrict__ out, int T, int z_rows,
                             int phys_n, unsigned int *oob) {
  pdl_prologue();
  constexpr bool EXACT = MODE != 0;
  constexpr uint32_t SZ = sizeof(ZT), SO = sizeof(OT);
  using Acc = typename std::conditional<EXACT, double, float>::type;
  extern __shared__ __align__(16) unsigned char ring[];
  __shared__ Acc scratch[2][32];
  const int k = KEQ ? KM : k_arg;
  const uint32_t x_bytes = (uint32_t)H * 4u, z_bytes = (uint32_t)H * SZ;
  const uint32_t stage_bytes = x_bytes + (uint32_t)k * z_bytes;
  const uint32_t ring_a = smem_u32(ring);
  const int n_chunks = H >> 3;

  // this thread's chunks: whether it has one, and its byte offset inside an fp32 row, an
  // expert row and an output row
  bool has[NC];
  uint32_t off_x[NC], off_z[NC], off_o[NC];
  [[maybe_unused]] Vec8 ws[NC];
#pragma unroll
  for (int c = 0; c < NC; c++) {
    const int chunk = threadIdx.x + c * blockDim.x;
    has[c] = chunk < n_chunks;
    off_x[c] = (uint32_t)chunk * 32u, off_z[c] = (uint32_t)chunk * 8u * SZ, off_o[c] = (uint32_t)chunk * 8u * SO;
    if constexpr (NORM)
      if (has[c])
        ws[c] = load8<kTable>(norm_w, (size_t)chunk * 8);
  }
  unsigned char *const xb = reinterpret_cast<unsigned char *>(x);
  const unsigned char *const zb = reinterpret_cast<const unsigned char *>(Z);

  // Routing data is tiny but every thread needs it.  Instead of every thread
  // loading every word, lane L of each warp loads one word of a token and the
  // warp shares them with shuffles at the point of use:
  //   "ids" word:     L < k: own_row[token*k + L];   L == k: topk_e[token*k] (liveness)
  //   "routing" word: L < k: topk_w[token*k + L];    k <= L < 2k: topk_e[token*k + L - k]
  // A pair whose own_row entry is negative has no expert row here (the grouping step writes
  // -1 for experts outside its range): nothing is read for it; its part of the stage is
  // filled with zeros by the copy instruction itself, so it adds nothing and the sum needs
  // no test per pair.  Tokens with such a pair take a path of their own (one sign test per
  // token on the broadcast row numbers); the others run the plain copies.
  const int lane = threadIdx.x & 31;
  auto load_ids_word = [&](long row) -> uint32_t {
    if (lane < k)
      return own_row ? (uint32_t)__ldg(own_row + (size_t)row * k + lane) : (uint32_t)(row * k + lane);
    if (lane == k)
      return (uint32_t)__ldg(topk_e + (size_t)row * k);
    return 0u;
  };
  auto load_routing_word = [&](long row) -> uint32_t {
    if (lane < k)
      return __float_as_uint(__ldg(topk_w + (size_t)row * k + lane));
    if (lane < 2 * k)
      return (uint32_t)__ldg(topk_e + (size_t)row * k + lane - k);
    return 0u;
  };
  auto spread_ids = [&](uint32_t word) {
    RowIds<KM> r;
    r.live = (int)__shfl_sync(0xffffffffu, word, k) >= 0;
    int any = 0; // a negative entry anywhere sets the sign bit
#pragma unroll
    for (int j = 0; j < KM; j++) {
      r.row[j] = (int)__shfl_sync(0xffffffffu, word, j < k ? j : 0);
      any |= r.row[j];
#ifdef GPTOSS_BOUNDS
      any |= (uint32_t)r.row[j] >= (uint32_t)z_rows ? -1 : 0; // checked build: also past the end of Z
#endif
    }
    r.all_here = any >= 0;
    return r;
  };
  auto spread_routing = [&](uint32_t word) {
    Routing<KM> r;
#pragma unroll
    for (int j = 0; j < KM; j++) {
      r.w[j] = __uint_as_float(__shfl_sync(0xffffffffu, word, j < k ? j : 0));
      r.e[j] = j < k ? (int)__shfl_sync(0xffffffffu, word, k + j) : 0x7fffffff;
    }
    return r;
  };
  auto issue = [&](long row, int stage, const RowIds<KM> &ids) {
    const uint32_t sx = ring_a + (uint32_t)stage * stage_bytes;
    const unsigned char *xr = xb + (size_t)row * x_bytes;
#pragma unroll
    for (int c = 0; c < NC; c++)
      if (has[c]) {
        cp16_cg(sx + off_x[c], xr + off_x[c]);
        cp16_cg(sx + off_x[c] + 16, xr + off_x[c] + 16);
        if (ids.live && ids.all_here) {
#pragma unroll
          for (int j = 0; j < KM; j++)
            if (j < k) {
              const unsigned char *zr = zb + (size_t)(uint32_t)ids.row[j] * z_bytes + off_z[c];
              const uint32_t sz = sx + x_bytes + (uint32_t)j * z_bytes + off_z[c];
              cp16_cg(sz, zr);
              if constexpr (SZ == 4)
                cp16_cg(sz + 16, zr + 16);
            }
        } else if (ids.live) { // some pair has no row here: that pair's part of the stage becomes zeros, unread
#pragma unroll
          for (int j = 0; j < KM; j++)
            if (j < k) {
              const uint32_t sz = sx + x_bytes + (uint32_t)j * z_bytes + off_z[c];
              const bool here = (unsigned)ids.row[j] < (unsigned)z_rows;
              const unsigned char *zr = zb + (size_t)(here ? (uint32_t)ids.row[j] : 0u) * z_bytes + off_z[c];
              cp16_cg_or_zeros(sz, zr, here);
              if constexpr (SZ == 4)
                cp16_cg_or_zeros(sz + 16, zr + 16, here);
#ifdef GPTOSS_BOUNDS
              if (!here && ids.row[j] >= 0 && threadIdx.x == 0 && c == 0)
                atomicAdd(oob, 1u); // a row number past the end of Z's allocation
#endif
            }
        }
      }
  };

  const long step = gridDim.x;
  long row = blockIdx.x;
  if (row >= T)
    return;
#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    const long r = row + s * step < T ? row + s * step : row;
    const RowIds<KM> ids = spread_ids(load_ids_word(r));
    if (row + s * step < T)
      issue(row + s * step, s, ids);
    cp_async_commit();
  }
  // one word per lane: routing of the current token, row ids of the token STAGES-1 ahead;
  // both are refilled one iteration before they are needed
  uint32_t routing_word = load_routing_word(row);
  uint32_t ids_word = load_ids_word(row + (STAGES - 1) * step < T ? row + (STAGES - 1) * step : row);
  int stage = 0, flip = 0;
  for (; row < T; row += step, flip ^= 1) {
    {
      const long ahead = row + (STAGES - 1) * step;
      const int fill = stage == 0 ? STAGES - 1 : stage - 1;
      const RowIds<KM> ahead_ids = spread_ids(ids_word);
      if (ahead < T)
        issue(ahead, fill, ahead_ids);
      cp_async_commit();
    }
    const Routing<KM> cur = spread_routing(routing_word);
    // fetch for the next iteration while this token's copies finish
    if (row + step < T)
      routing_word = load_routing_word(row + step);
    if (row + STAGES * step < T)
      ids_word = load_ids_word(row + STAGES * step);
    cp_async_wait<STAGES - 1>();

    const bool live = cur.e[0] >= 0;
    int ord[KM];
#pragma unroll
    for (int j = 0; j < KM; j++)
      ord[j] = j;
    if (EXACT && live) {
      int key[KM];
#pragma unroll
      for (int j = 0; j < KM; j++)
        key[j] = (phys_of && cur.e[j] >= 0 && cur.e[j] < phys_n && cur.e[j] != 0x7fffffff) ? __ldg(phys_of + cur.e[j])
                                                                                           : cur.e[j];
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

    const uint32_t sx = ring_a + (uint32_t)stage * stage_bytes;
    unsigned char *xr = xb + (size_t)row * x_bytes;
    Vec8 xs[NC];
    Acc ss = 0;
#pragma unroll
    for (int c = 0; c < NC; c++) {
      if (!has[c])
        continue;
      xs[c] = floats_of(lds16(sx + off_x[c]), lds16(sx + off_x[c] + 16));
      if (live) {
        Vec8 acc;
#pragma unroll
        for (int i = 0; i < 8; i++)
          acc.v[i] = 0.0f;
#pragma unroll
        for (int jj = 0; jj < KM; jj++)
          if (jj < k) {
            // position jj of the summation order takes choice ord[jj]
            int j = jj;
            float wj = cur.w[jj];
            if (EXACT) {
              j = ord[jj];
#pragma unroll
              for (int q = 0; q < KM; q++)
                if (q == j)
                  wj = cur.w[q];
            }
            const uint32_t sz = sx + x_bytes + (uint32_t)j * z_bytes + off_z[c];
            Vec8 z;
            if constexpr (SZ == 2)
              z = widen8(lds16(sz));
            else
              z = floats_of(lds16(sz), lds16(sz + 16));
#pragma unroll
            for (int i = 0; i < 8; i++)
              acc.v[i] = MODE == 1 ? __fadd_rn(acc.v[i], __fmul_rn(z.v[i], wj)) : __fmaf_rn(z.v[i], wj, acc.v[i]);
          }
#pragma unroll
        for (int i = 0; i < 8; i++)
          xs[c].v[i] = __fadd_rn(xs[c].v[i], acc.v[i]);
        store8(reinterpret_cast<float *>(xr + off_x[c]), 0, xs[c], false);
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
      unsigned char *orow = reinterpret_cast<unsigned char *>(out) + (size_t)row * ((size_t)H * SO);
      [[maybe_unused]] double inv_d = 0.0;
      [[maybe_unused]] float inv_f = 0.0f;
      if constexpr (EXACT) {
        const double m = __dadd_rn(__ddiv_rn(ss, (double)H), (double)GPTOSS_RMS_EPS);
        inv_d = (double)__fdiv_rn(1.0f, __fsqrt_rn((float)m));
      } else {
        inv_f = fast_inv_rms(ss, H);
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
          store8(reinterpret_cast<OT *>(orow + off_o[c]), 0, o);
        }
    }
    stage = stage + 1 == STAGES ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

// Any H, k <= GPTOSS_MAX_TOPK, any alignment: scalar accesses.
template <typename ZT, typename OT, int MODE, bool NORM>
__global__ void combine_rows_generic(float *x, const ZT *__restrict__ Z,
                                     const int *__restrict__ own_row,
                                     const float *__restrict__ topk_w,
                                     const int *__restrict__ topk_e, int k, int H,
                                     const int *__restrict__ phys_of,
                                     const float *__restrict__ norm_w, OT *__restrict__ out,
                                     int T, int z_rows, int phys_n, unsigned int *oob) {
  pdl_prologue();
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
          const int ka = phys_of && ea >= 0 && ea < phys_n ? phys_of[ea] : ea;
          const int kb = phys_of && eb >= 0 && eb < phys_n ? phys_of[eb] : eb;
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
          if (own_row && (unsigned)own_row[p] >= (unsigned)z_rows) {
#ifdef GPTOSS_BOUNDS
            if (own_row[p] >= 0 && i == 0)
              atomicAdd(oob, 1u);
#endif
            continue; // no expert row here for this pair
          }
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
        const float inv = fast_inv_rms(ss, H);
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
  int z_rows, phys_n; // extents of Z (rows) and phys_of (entries); INT_MAX when not known
  unsigned int *oob;  // the checked build's device counter
};

template <typename ZT, typename OT, int MODE, bool NORM, int KM, bool KEQ, int NC, int STAGES>
int launch_variant(cudaStream_t s, const Args &a, int threads, size_t smem) {
  auto kern = combine_rows<ZT, OT, MODE, NORM, KM, KEQ, NC, STAGES>;
  const int per_sm = blocks_per_sm_smem(kern, threads, smem);
  if (per_sm < 1)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(kern, dim3(row_grid(a.T, per_sm)), dim3(threads), smem, s, a.x, static_cast<const ZT *>(a.Z), a.own_row,
                                                   a.topk_w, a.topk_e, a.k, a.H, a.phys_of, a.norm_w,
                                                   static_cast<OT *>(a.out), a.T, a.z_rows, a.phys_n, a.oob);
  return launch_status();
}

template <typename ZT, typename OT, int MODE, bool NORM, int KM, bool KEQ, int NC>
int launch_stages(cudaStream_t s, const Args &a, int threads, size_t stage_bytes, int stages) {
  if constexpr (NC > 1) // wide rows: a stage is tens of KB, two is what fits anyway
    return launch_variant<ZT, OT, MODE, NORM, KM, KEQ, NC, 2>(s, a, threads, stage_bytes * 2);
  if (stages == 4)
    return launch_variant<ZT, OT, MODE, NORM, KM, KEQ, NC, 4>(s, a, threads, stage_bytes * 4);
  if (stages == 3)
    return launch_variant<ZT, OT, MODE, NORM, KM, KEQ, NC, 3>(s, a, threads, stage_bytes * 3);
  return launch_variant<ZT, OT, MODE, NORM, KM, KEQ, NC, 2>(s, a, threads, stage_bytes * 2);
}

template <typename ZT, typename OT, int MODE, bool NORM> int launch(cudaStream_t s, const Args &a) {
  const size_t stage_bytes = (size_t)a.H * (4 + (size_t)a.k * sizeof(ZT));
  int stages = pick_stages(stage_bytes);
  // A ring of two beats a ring of three where three stages of two blocks fill the SM's shared
  // memory (the model's shape: 34.5 KB stages, two blocks per SM by registers either way;
  // measured 32.6 against 34.3 us per launch): fewer requests outstanding stream better.
  if (stages == 3 && stage_bytes * 2 * 3 <= 220 * 1024)
    stages = 2;
  const bool vec = a.H % 8 == 0 && a.H <= 8 * 512 * 4 && aligned16(a.x) && aligned16(a.Z) && stages > 0 &&
                   (!NORM || (aligned16(a.norm_w) && aligned16(a.out)));
  if (vec) {
    const int n_chunks = a.H / 8;
    const int nc = n_chunks <= 512 ? 1 : 4;
    const int threads = ((n_chunks + nc - 1) / nc + 31) / 32 * 32;
    int st;
    if (a.k == 4 && nc == 1) // the models' shape: k known at compile time
      st = launch_stages<ZT, OT, MODE, NORM, 4, true, 1>(s, a, threads, stage_bytes, stages);
    else if (a.k <= 4)
      st = nc == 1 ? launch_stages<ZT, OT, MODE, NORM, 4, false, 1>(s, a, threads, stage_bytes, stages)
                   : launch_stages<ZT, OT, MODE, NORM, 4, false, 4>(s, a, threads, stage_bytes, stages);
    else
      st = nc == 1 ? launch_stages<ZT, OT, MODE, NORM, 8, false, 1>(s, a, threads, stage_bytes, stages)
                   : launch_stages<ZT, OT, MODE, NORM, 8, false, 4>(s, a, threads, stage_bytes, stages);
    if (st != GPTOSS_ERR_UNSUPPORTED)
      return st;
  }
  note_generic_launch();
  launch_kernel(combine_rows_generic<ZT, OT, MODE, NORM>, dim3(row_grid(a.T, 8)), dim3(256), 0, s, 
      a.x, static_cast<const ZT *>(a.Z), a.own_row, a.topk_w, a.topk_e, a.k, a.H, a.phys_of,
      a.norm_w, static_cast<OT *>(a.out), a.T, a.z_rows, a.phys_n, a.oob);
  return launch_status();
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
  const PdlScope pdl(flags);
  if (T < 0 || k <= 0 || H <= 0 || !valid_dtype(z_dtype) || (norm_w && !valid_dtype(out_dtype)))
    return GPTOSS_ERR_BAD_ARG;
  if (k > GPTOSS_MAX_TOPK)
    return GPTOSS_ERR_UNSUPPORTED;
  if (T == 0)
    return GPTOSS_OK;
  if (!x || !Z || !topk_w || !topk_e || (norm_w && !out))
    return GPTOSS_ERR_BAD_ARG;
  int z_rows = 0x7fffffff, phys_n = 0x7fffffff;
  unsigned int *oob = nullptr;
  GPTOSS_SPAN(x, (size_t)T * H * 4);
  GPTOSS_SPAN(topk_w, (size_t)T * k * 4);
  GPTOSS_SPAN(topk_e, (size_t)T * k * 4);
  GPTOSS_SPAN(own_row, (size_t)T * k * 4);
  GPTOSS_SPAN(norm_w, (size_t)H * 4);
  if (norm_w)
    GPTOSS_SPAN(out, (size_t)T * H * dtype_size(out_dtype));
#ifdef GPTOSS_BOUNDS
  { // the row map and the expert renumbering index arrays whose length the call does not state
    const size_t z_room = bounds_room(Z), p_room = phys_of ? bounds_room(phys_of) : SIZE_MAX;
    const size_t row_bytes = (size_t)H * dtype_size(z_dtype);
    if (z_room != SIZE_MAX && z_room / row_bytes < (size_t)z_rows)
      z_rows = (int)(z_room / row_bytes);
    if (p_room != SIZE_MAX && p_room / 4 < (size_t)phys_n)
      phys_n = (int)(p_room / 4);
    if (!own_row)
      GPTOSS_SPAN(Z, (size_t)T * k * row_bytes);
    oob = bounds_device_word();
    if (!oob)
      return GPTOSS_ERR_CUDA;
  }
#endif
  const Args a{T, x, Z, own_row, topk_w, topk_e, k, H, phys_of, norm_w, out, z_rows, phys_n, oob};
  cudaStream_t s = as_stream(stream);
  return z_dtype == GPTOSS_F32 ? launch_mode<float>(s, a, out_dtype, flags)
                               : launch_mode<uint16_t>(s, a, out_dtype, flags);
}
