// Greedy vocabulary argmax (gptoss_argmax).
//
// The one op on the path with real volume: V = 201,088 logits per row.  Each
// row is cut into `splits` contiguous slices, one thread block per slice, so a
// small batch still fills every SM.  A thread streams 128-bit pieces of its
// slice (kUnroll of them in flight), keeps only a running maximum and its
// index, and touches the index bookkeeping in a rarely taken branch: for each
// 16-byte piece it first reduces the 8 (bf16) or 4 (fp32) values to their
// maximum with packed max instructions and compares once.  Blocks merge through
// a 64-bit key, order-preserving value bits above the complemented index, so
// the larger value wins and, among equal values, the lower index; slices merge
// with atomicMax on one key per row, and a second tiny kernel turns keys into
// indices and zeroes them again.
#include <cuda_bf16.h>

#include "../../include/gptoss_argmax_key.cuh"
#include "common.cuh"

namespace gptoss {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// Larger value => larger key; equal values => lower index wins; -0 == +0; never 0
// for a number, so 0 can mean "nothing seen".  The formula is public
// (gptoss_argmax_key.cuh) so that a logits producer can fold into the same words.
__device__ __forceinline__ unsigned long long pick_key(float v, unsigned idx) {
  return gptoss_argmax_key(v, idx);
}

// Maximum of the values of one 16-byte piece; NaNs are ignored unless every
// value is NaN.
template <typename LT> __device__ __forceinline__ float piece_max(uint4 q) {
  if constexpr (sizeof(LT) == 2) {
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&q.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&q.y);
    __nv_bfloat162 c = *reinterpret_cast<__nv_bfloat162 *>(&q.z);
    __nv_bfloat162 d = *reinterpret_cast<__nv_bfloat162 *>(&q.w);
    a = __hmax2(__hmax2(a, b), __hmax2(c, d));
    const uint32_t m = *reinterpret_cast<uint32_t *>(&a);
    return fmaxf(bf16_lo(m), bf16_hi(m));
  } else {
    return fmaxf(fmaxf(__uint_as_float(q.x), __uint_as_float(q.y)),
                 fmaxf(__uint_as_float(q.z), __uint_as_float(q.w)));
  }
}

// Position (0-based, within the piece) of the first value equal to m.
template <typename LT> __device__ __forceinline__ int piece_first(uint4 q, float m) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  if constexpr (sizeof(LT) == 2) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if (bf16_lo(w[i]) == m)
        return 2 * i;
      if (bf16_hi(w[i]) == m)
        return 2 * i + 1;
    }
    return 0;
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (__uint_as_float(w[i]) == m)
        return i;
    return 0;
  }
}

// Block-wide maximum key; valid in thread 0.
__device__ __forceinline__ unsigned long long block_max_key(unsigned long long key,
                                                            unsigned long long *scratch) {
  key = warp_max_u64(key);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0)
    scratch[warp] = key;
  __syncthreads();
  unsigned long long best = 0;
  if (warp == 0) {
    best = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0ull;
    best = warp_max_u64(best);
  }
  return best;
}

// The CPU's answer for a row given the merged key (run.cpp:778-789): element 0
// being NaN keeps index 0; no number above -inf also leaves index 0.
template <typename LT>
__device__ __forceinline__ int decode_pick(unsigned long long key, const LT *row) {
  const float first = load1(row);
  if (first != first || key == 0ull)
    return 0;
  return (int)~(unsigned)(key & 0xffffffffull);
}

// grid = splits * T blocks; block b scans slice b % splits of row b / splits.  Vector path: V_vec elements per row, a multiple of the
// piece width, start 16-byte aligned; the scalar tail [V_vec, V) is scanned by
// the block of the last slice.
template <typename LT>
__global__ void __launch_bounds__(kThreads)
    argmax_slices(const LT *__restrict__ logits, long V, long row_stride, unsigned pieces_per_row,
                  unsigned pieces_per_slice, int splits, unsigned long long *keys, int *__restrict__ out) {
  pdl_prologue();
  constexpr unsigned kPer = 16 / sizeof(LT); // values per 16-byte piece
  __shared__ unsigned long long scratch[kThreads / 32];
  const int row = blockIdx.x / splits, slice = blockIdx.x - row * splits;
  const LT *r = logits + (size_t)row * row_stride;
  // Pieces are counted in 32 bits (a row has fewer than 2^29 of them) and the pointer to the
  // thread's next piece is carried along, so an iteration's index work is one add.
  const unsigned p0 = (unsigned)slice * pieces_per_slice;
  const unsigned p1 = min(p0 + pieces_per_slice, pieces_per_row);

  float best = __int_as_float(0xff800000); // -inf: only values above it are recorded
  long best_idx = -1;
  unsigned p = p0 + threadIdx.x;
  const uint4 *at = reinterpret_cast<const uint4 *>(r) + p; // dereferenced only where p < p1
  // whole iterations: kUnroll pieces in flight per thread, none past the slice
  for (; p + (kUnroll - 1) * kThreads < p1; p += kThreads * kUnroll, at += kThreads * kUnroll) {
    uint4 q[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; u++)
      q[u] = ld_stream(at + u * kThreads);
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
      const float m = piece_max<LT>(q[u]);
      if (m > best) { // rare after the first few pieces
        best = m;
        best_idx = (long)(p + u * kThreads) * kPer + piece_first<LT>(q[u], m);
      }
    }
  }
  // the slice's last, partly filled iteration
  if (p < p1) {
    uint4 q[kUnroll - 1];
#pragma unroll
    for (int u = 0; u < kUnroll - 1; u++) // past the slice: the thread's first piece again; the strict '>' makes a repeat harmless
      q[u] = ld_stream(at + (p + u * kThreads < p1 ? u * kThreads : 0));
#pragma unroll
    for (int u = 0; u < kUnroll - 1; u++) {
      const float m = piece_max<LT>(q[u]);
      if (m > best) {
        best = m;
        best_idx = (long)(p + u * kThreads < p1 ? p + u * kThreads : p) * kPer + piece_first<LT>(q[u], m);
      }
    }
  }
  // scalar tail of the row, by the last slice's block
  if (slice == splits - 1)
    for (long i = (long)pieces_per_row * kPer + threadIdx.x; i < V; i += kThreads) {
      const float v = load1(r + i);
      if (v > best) {
        best = v;
        best_idx = i;
      }
    }
  unsigned long long key = best_idx >= 0 ? pick_key(best, (unsigned)best_idx) : 0ull;
  key = block_max_key(key, scratch);
  if (threadIdx.x == 0) {
    if (keys)
      atomicMax(keys + row, key);
    else
      out[row] = decode_pick(key, r);
  }
}

template <typename LT>
__global__ void argmax_finish(unsigned long long *keys, const LT *__restrict__ logits,
                              long row_stride, int T, int *__restrict__ out) {
  pdl_prologue();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T)
    return;
  out[row] = decode_pick(keys[row], logits + (size_t)row * row_stride);
  keys[row] = 0ull;
}

// The decode half of a fused producer (gptoss_argmax_keys_finish).
__global__ void argmax_keys_decode(unsigned long long *keys, int T, int *__restrict__ out) {
  pdl_prologue();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T)
    return;
  out[row] = gptoss_argmax_column(keys[row]);
  keys[row] = 0ull;
}

// Slices per row.  With at least two waves of one-block rows the tail is small and a
// row stays whole (no merge, no second launch).  Below that, rows are cut so that the
// launch has about four waves of blocks -- measured 9 % faster at 1024 rows than one
// wave, the same at 128 and 512 -- each slice at least 2048 pieces (32 KB), at most 64
// slices.  A slice is a whole number of block iterations (kThreads * kUnroll pieces, the
// nearest to an even cut, at least two), so that only a row's last slice ends on a partly
// filled one: 15 us instead of 17 at 128 rows, level from 512 rows up.
constexpr long kPiecesPerIteration = (long)kThreads * kUnroll;

long plan_slice_pieces(int T, long pieces, bool has_keys) {
  if (!has_keys || T <= 0 || pieces <= 0)
    return pieces > 0 ? pieces : 1;
  const long slots = (long)sm_count() * 8;
  if (T >= 2 * slots)
    return pieces;
  long want = (4 * slots + T - 1) / T;
  const long by_size = pieces / 2048 > 0 ? pieces / 2048 : 1;
  if (want > by_size)
    want = by_size;
  if (want > 64)
    want = 64;
  if (want <= 1)
    return pieces;
  const long per_slice = (pieces + want - 1) / want;
  const long its = (per_slice + kPiecesPerIteration / 2) / kPiecesPerIteration;
  return (its < 2 ? 2 : its) * kPiecesPerIteration;
}

int plan_slices(int T, long pieces, bool has_keys) {
  const long per_slice = plan_slice_pieces(T, pieces, has_keys);
  const long n = (pieces + per_slice - 1) / per_slice;
  return n < 1 ? 1 : (int)n;
}

template <typename LT>
int launch(cudaStream_t s, int T, const void *logits, long V, long row_stride,
           unsigned long long *keys, int *out) {
  const LT *lp = static_cast<const LT *>(logits);
  constexpr long kPer = 16 / sizeof(LT);
  const bool vec = aligned16(logits) && (row_stride * sizeof(LT)) % 16 == 0;
  const long pieces = vec ? V / kPer : 0;
  const long per_slice = plan_slice_pieces(T, pieces, keys != nullptr);
  const int splits = plan_slices(T, pieces, keys != nullptr);
  if ((long)T * splits > 0x7fffffffL)
    return GPTOSS_ERR_UNSUPPORTED;
  unsigned long long *merge = splits > 1 ? keys : nullptr;
  launch_kernel(argmax_slices<LT>, dim3((unsigned)((long)T * splits)), dim3(kThreads), 0, s, lp, V, row_stride,
                (unsigned)pieces, (unsigned)per_slice, splits, merge, out);
  int st = launch_status();
  if (st != GPTOSS_OK || !merge)
    return st;
  launch_kernel(argmax_finish<LT>, dim3((T + 255) / 256), dim3(256), 0, s, keys, lp, row_stride, T, out);
  return launch_status();
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_argmax(gptoss_stream_t stream, int T, const void *logits,
                             gptoss_dtype_t logits_dtype, long V, long row_stride,
                             unsigned long long *keys, int *out, unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (T < 0 || V <= 0 || V > 0x7fffffffL || row_stride < V || !valid_dtype(logits_dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!logits || !out)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(logits, strided_bytes(T, row_stride, V, dtype_size(logits_dtype)));
  GPTOSS_SPAN(keys, (size_t)T * 8);
  GPTOSS_SPAN(out, (size_t)T * 4);
  cudaStream_t s = as_stream(stream);
  return logits_dtype == GPTOSS_F32 ? launch<float>(s, T, logits, V, row_stride, keys, out)
                                    : launch<uint16_t>(s, T, logits, V, row_stride, keys, out);
}

extern "C" int gptoss_argmax_keys_finish(gptoss_stream_t stream, int T, unsigned long long *keys,
                                         int *out, unsigned flags) {
  using namespace gptoss;
  const PdlScope pdl(flags);
  if (T < 0)
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!keys || !out)
    return GPTOSS_ERR_BAD_ARG;
  GPTOSS_SPAN(keys, (size_t)T * 8);
  GPTOSS_SPAN(out, (size_t)T * 4);
  launch_kernel(argmax_keys_decode, dim3((T + 255) / 256), dim3(256), 0, as_stream(stream), keys, T, out);
  return launch_status();
}

extern "C" int gptoss_argmax_slices(int T, long V, gptoss_dtype_t logits_dtype, int has_keys) {
  using namespace gptoss;
  if (T <= 0 || V <= 0 || !valid_dtype(logits_dtype))
    return 1;
  const long per = logits_dtype == GPTOSS_F32 ? 4 : 8;
  return plan_slices(T, V / per, has_keys != 0);
}

// ---- greedy argmax for callers that cannot allocate device memory ---------------------
#include <stdio.h>
#include <atomic>
//
// gptoss_argmax needs one 64-bit merge word per row from its caller.  Some hosts
// of this library have no way to provide that: a plug-in running inside a serving
// process whose memory manager has already claimed the whole GPU and hands out
// nothing at request time, or a step function that must never reach cudaMalloc
// because an allocation stalls every stream of the device.  For them the merge
// words live in this fixed array, which is part of the library image: each GPU
// that loads the library holds these 128 KB from load until the process exits.
static __device__ __align__(256) unsigned long long g_noalloc_keys[GPTOSS_ARGMAX_NOALLOC_MAX_ROWS];

namespace gptoss {
namespace {

// Device address of g_noalloc_keys on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel can
// use, so the address is asked for once per device (with that device current)
// and remembered.  Returns nullptr and sets *status on failure.
unsigned long long *noalloc_keys_on_current_device(int *status) {
  // two threads asking at once both get the same answer from the runtime; the atomic only
  // makes the publication of the pointer well defined
  static std::atomic<unsigned long long *> address_of[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    *status = GPTOSS_ERR_CUDA;
    return nullptr;
  }
  if (dev < 0 || dev >= 64) {
    *status = GPTOSS_ERR_UNSUPPORTED;
    return nullptr;
  }
  if (!address_of[dev].load(std::memory_order_acquire)) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_keys);
    if (e != cudaSuccess || !p) {
      note_cuda_error(e);
      (void)cudaGetLastError();
      *status = GPTOSS_ERR_CUDA;
      return nullptr;
    }
    address_of[dev].store(static_cast<unsigned long long *>(p), std::memory_order_release);
  }
  return address_of[dev].load(std::memory_order_acquire);
}

} // namespace
} // namespace gptoss

extern "C" int gptoss_argmax_noalloc(gptoss_stream_t stream, int T, const void *logits,
                                     gptoss_dtype_t logits_dtype, long V, long row_stride,
                                     int *out) {
  using namespace gptoss;
  if (T < 0 || V <= 0 || V > 0x7fffffffL || row_stride < V || !valid_dtype(logits_dtype))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!logits || !out)
    return GPTOSS_ERR_BAD_ARG;
  if (T > GPTOSS_ARGMAX_NOALLOC_MAX_ROWS) {
    fprintf(stderr,
            "gptoss_argmax_noalloc: %d rows exceed the built-in scratch of %d rows; split the "
            "batch or use gptoss_argmax with caller-provided keys\n",
            T, GPTOSS_ARGMAX_NOALLOC_MAX_ROWS);
    return GPTOSS_ERR_UNSUPPORTED;
  }
  int st = GPTOSS_OK;
  unsigned long long *keys = noalloc_keys_on_current_device(&st);
  if (!keys)
    return st;
  cudaStream_t s = as_stream(stream);
  // The array still holds whatever the previous call (of any thread) left
  // there: the merge words of this call's rows must start from zero.
  const cudaError_t e = cudaMemsetAsync(keys, 0, (size_t)T * sizeof(unsigned long long), s);
  if (e != cudaSuccess) {
    note_cuda_error(e);
    (void)cudaGetLastError();
    return GPTOSS_ERR_CUDA;
  }
  return logits_dtype == GPTOSS_F32 ? launch<float>(s, T, logits, V, row_stride, keys, out)
                                    : launch<uint16_t>(s, T, logits, V, row_stride, keys, out);
}
