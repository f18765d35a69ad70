// Token-embedding gather (gptoss_embed): x[t,:] = table[ids[t],:].
//
// Pure data movement: per token one id, one table row in, one row out.  Work is
// cut into 16-byte chunks; a block owns a contiguous tile of output chunks and
// every thread fetches kUnroll of them with 128-bit loads before it stores any
// (a one-shot grid: the hardware scheduler keeps the SMs stocked with blocks).  Rows are random, but each row is a
// contiguous multi-kilobyte run, so DRAM pages are still used whole.
#include "common.cuh"

namespace gptoss {
namespace {

constexpr int kUnroll = 2;

// WIDEN = false: rows are copied as raw 16-byte pieces (table and x have the
// same element type; row_bytes = H * element size).  WIDEN = true: each 16-byte
// piece holds 8 bf16 values that leave as 8 fp32 values (bits << 16).
template <bool WIDEN>
__global__ void __launch_bounds__(256)
    embed_rows(const unsigned char *__restrict__ table, const int *__restrict__ ids,
               unsigned char *__restrict__ x, long total_chunks, int chunks_per_row,
               size_t row_bytes, int V, int id_div) {
  pdl_prologue();
  // One-shot grid: block b owns output chunks [b * 256 * kUnroll, (b + 1) * 256 * kUnroll).
  const long base = (long)blockIdx.x * (256 * kUnroll) + threadIdx.x;
  uint4 v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; u++) {
    const long unit = base + u * 256;
    v[u] = make_uint4(0u, 0u, 0u, 0u);
    if (unit < total_chunks) {
      const int row = (int)(unit / chunks_per_row), c = (int)(unit - (long)row * chunks_per_row);
      const int raw = __ldg(ids + row);
      const int id = raw >= 0 ? raw / id_div : -1; // id_div = k turns a pair index into its token
      if (id >= 0 && id < V)
        v[u] = ld_stream(table + (size_t)id * row_bytes + (size_t)c * 16);
    }
  }
#pragma unroll
  for (int u = 0; u < kUnroll; u++) {
    const size_t unit = (size_t)(base + u * 256);
    if ((long)unit >= total_chunks)
      continue;
    if (WIDEN) {
      st_stream(x + unit * 32, make_uint4(v[u].x << 16, v[u].x & 0xffff0000u, v[u].y << 16,
                                          v[u].y & 0xffff0000u));
      st_stream(x + unit * 32 + 16, make_uint4(v[u].z << 16, v[u].z & 0xffff0000u,
                                               v[u].w << 16, v[u].w & 0xffff0000u));
    } else {
      st_stream(x + unit * 16, v[u]);
    }
  }
}

// Any H and alignment: one element per thread step.
template <typename TT, typename OT>
__global__ void embed_rows_generic(const TT *__restrict__ table, const int *__restrict__ ids,
                                   OT *__restrict__ x, int T, int H, int V, int id_div) {
  pdl_prologue();
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const int id = ids[row] >= 0 ? ids[row] / id_div : -1;
    const bool ok = id >= 0 && id < V;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
      if constexpr (sizeof(TT) == sizeof(OT)) // same type: move the bits untouched
        x[(size_t)row * H + j] = ok ? table[(size_t)id * H + j] : OT(0);
      else
        store1(x + (size_t)row * H + j, ok ? load1(table + (size_t)id * H + j) : 0.0f);
    }
  }
}

template <typename TT, typename OT>
int launch(cudaStream_t s, int T, const void *table, int V, const int *ids, void *x, int H,
           int id_div = 1) {
  constexpr bool widen = sizeof(TT) != sizeof(OT);
  const size_t row_bytes = (size_t)H * sizeof(TT);
  if (row_bytes % 16 != 0 || !aligned16(table) || !aligned16(x)) {
    note_generic_launch();
    launch_kernel(embed_rows_generic<TT, OT>, dim3(row_grid(T, 8)), dim3(256), 0, s, 
        static_cast<const TT *>(table), ids, static_cast<OT *>(x), T, H, V, id_div);
    return launch_status();
  }
  const int cpr = (int)(row_bytes / 16);
  const long total = (long)T * cpr;
  constexpr int threads = 256;
  const long blocks = (total + (long)threads * kUnroll - 1) / ((long)threads * kUnroll);
  if (blocks > 0x7fffffffL)
    return GPTOSS_ERR_UNSUPPORTED;
  launch_kernel(embed_rows<widen>, dim3((unsigned)blocks), dim3(threads), 0, s, 
      static_cast<const unsigned char *>(table), ids, static_cast<unsigned char *>(x), total, cpr,
      row_bytes, V, id_div);
  return launch_status();
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_embed(gptoss_stream_t stream, int T, const void *table,
                            gptoss_dtype_t table_dtype, int V, const int *ids, void *x,
                            gptoss_dtype_t x_dtype, int H, unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (T < 0 || H <= 0 || V <= 0 || !valid_dtype(table_dtype) || !valid_dtype(x_dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!table || !ids || !x)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(table, (size_t)V * H * dtype_size(table_dtype));
  GPTOSS_SPAN(ids, (size_t)T * 4);
  GPTOSS_SPAN(x, (size_t)T * H * dtype_size(x_dtype));
  cudaStream_t s = as_stream(stream);
  if (table_dtype == GPTOSS_BF16 && x_dtype == GPTOSS_F32)
    return launch<uint16_t, float>(s, T, table, V, ids, x, H);
  if (table_dtype == GPTOSS_BF16 && x_dtype == GPTOSS_BF16)
    return launch<uint16_t, uint16_t>(s, T, table, V, ids, x, H);
  if (table_dtype == GPTOSS_F32 && x_dtype == GPTOSS_F32)
    return launch<float, float>(s, T, table, V, ids, x, H);
  return GPTOSS_ERR_UNSUPPORTED; // narrowing an fp32 table would not be a bit-exact copy
}

extern "C" int gptoss_moe_gather(gptoss_stream_t stream, int R, const void *t, gptoss_dtype_t dtype,
                                 int n_tokens, const int *row_pair, int k, void *Xg, int H,
                                 unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (R < 0 || H <= 0 || n_tokens <= 0 || k <= 0 || !valid_dtype(dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (R == 0)
    return GPTOSS_OK;
  if (!t || !row_pair || !Xg)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(t, (size_t)n_tokens * H * dtype_size(dtype));
  GPTOSS_SPAN(row_pair, (size_t)R * 4);
  GPTOSS_SPAN(Xg, (size_t)R * H * dtype_size(dtype));
  cudaStream_t s = as_stream(stream);
  // the embedding gather with "ids" = pair indices divided by k
  return dtype == GPTOSS_BF16 ? launch<uint16_t, uint16_t>(s, R, t, n_tokens, row_pair, Xg, H, k)
                              : launch<float, float>(s, R, t, n_tokens, row_pair, Xg, H, k);
}
