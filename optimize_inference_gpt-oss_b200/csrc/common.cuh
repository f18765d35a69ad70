// Shared device helpers of the fused gpt-oss kernels (sm_100a): 128-bit global
// loads and stores, bf16 packing, warp and block reductions, launch plumbing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "../../include/gptoss_kernels.h"

namespace gptoss {

constexpr int kWarp = 32;

// ---- host-side plumbing -----------------------------------------------------

// Remembers the last CUDA error seen by this thread (gptoss_last_cuda_error).
void note_cuda_error(cudaError_t e);

// Streaming multiprocessors of the current device (cached per device).
int sm_count();

inline cudaStream_t as_stream(gptoss_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Set by an entry point for the duration of its call (GPTOSS_PDL in flags): kernels
// are then launched with programmatic stream serialization, so their blocks may be
// scheduled while the previous kernel in the stream is still draining.
extern thread_local bool tl_pdl;
extern thread_local cudaError_t tl_launch_error;
// Launches by this thread that fell to a scalar "generic" kernel (odd sizes, misaligned
// bases, shapes the vector kernels do not take): see gptoss_generic_launch_count().
extern thread_local long tl_generic_launches;
inline void note_generic_launch() { tl_generic_launches++; }
struct PdlScope {
  bool prev;
  explicit PdlScope(unsigned flags) : prev(tl_pdl) { tl_pdl = (flags & GPTOSS_PDL) != 0; }
  ~PdlScope() { tl_pdl = prev; }
};

// kernel<<<grid, block, smem, stream>>>(args...), with the launch attribute above when asked for.
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tl_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess)
    tl_launch_error = e;
}

// After a launch: GPTOSS_OK or GPTOSS_ERR_CUDA, from what cudaLaunchKernelEx returned for this
// launch.  The thread's "last error" is not polled: an error an application left there before
// calling in is the application's to find, not this launch's failure.  A failed launch of ours
// is taken out of that slot again, since it is reported through the status.
inline int launch_status() {
  const cudaError_t e = tl_launch_error;
  tl_launch_error = cudaSuccess;
  if (e == cudaSuccess)
    return GPTOSS_OK;
  (void)cudaGetLastError();
  note_cuda_error(e);
  return GPTOSS_ERR_CUDA;
}

// Thread blocks of a kernel that fit on one SM at `threads` threads and `smem`
// bytes of dynamic shared memory per block; above the 48 KB default the
// kernel's limit is raised first.  Remembered per (kernel, device, threads,
// smem).  0 means it does not fit.
int occupancy_cached(const void *kernel, int threads, size_t smem);

template <typename K> inline int blocks_per_sm(K kernel, int threads, int * /*unused*/ = nullptr) {
  const int n = occupancy_cached(reinterpret_cast<const void *>(kernel), threads, 0);
  return n > 0 ? n : 1;
}
template <typename K> inline int blocks_per_sm_smem(K kernel, int threads, size_t smem) {
  return occupancy_cached(reinterpret_cast<const void *>(kernel), threads, smem);
}

// Grid for a row-strided kernel: every SM full, never more blocks than rows.
inline int row_grid(long rows, int per_sm) {
  const long full = (long)sm_count() * per_sm;
  return (int)(rows < full ? rows : full);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_dtype(gptoss_dtype_t d) { return d == GPTOSS_F32 || d == GPTOSS_BF16; }
inline size_t dtype_size(gptoss_dtype_t d) { return d == GPTOSS_F32 ? 4 : 2; }

// First statement of every kernel: returns once the previous kernel in the stream has
// completed and its writes are visible; a no-op for a kernel launched the ordinary way.
// Nothing, not even a table, is read before it, so scheduling a kernel's blocks early
// (GPTOSS_PDL) only hides launch latency and never changes what a kernel sees.
//
// No kernel here signals its dependents early (griddepcontrol.launch_dependents): the
// next kernel's blocks become schedulable only when this grid's blocks have exited.
// Signalling at block start was measured on B200 more than once: with an earlier form of the
// kernels it made the 24-layer chain 15 % slower (blocks of kernels ahead in the stream
// became resident, sat in their wait, and took the SM slots that the persistent grids of
// the kernels actually running count on having all at once); with the current kernels
// 0.5 % slower at 4096 tokens and 8 % slower at 512 than the attribute alone (2 % slower at 512
// when only the one-shot grids signal).  Signalling
// late (a row kernel's block when it starts its last row) was 1 % slower than not
// signalling.  The attribute alone -- the launch may be set up while the previous kernel
// drains, and its completion need not be flushed to the host's view first -- is what pays:
// 3.14 -> 3.08 ms per step at 4096 tokens, 0.606 -> 0.541 ms at 512.
__device__ __forceinline__ void pdl_prologue() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- the checked build (-DGPTOSS_BOUNDS) --------------------------------------------
//
// Stands in for a memory checker on machines where none can be run.  The library keeps a
// table of the device allocations made through it (gptoss_device_alloc, the chain's
// buffers); every entry point works out, from its shape arguments, how many bytes it will
// touch behind each pointer and refuses the call (GPTOSS_ERR_BAD_ARG, nothing launched) when
// a pointer that lies inside a known allocation would be walked past that allocation's end.
// Pointers into memory the table does not know are let through and counted as unchecked.
// Indices that come out of device data and have no extent in the call's arguments (the
// combine's row map and expert renumbering) get their extent from the same table, and a
// kernel that meets one outside it skips the access and counts it in a device word.  Nothing
// traps.  gptoss_bounds_violations() adds both counts up.  In the ordinary build all of this
// compiles to nothing.
#ifdef GPTOSS_BOUNDS
void bounds_register(const void *p, size_t bytes);
void bounds_unregister(const void *p);
bool bounds_span_ok(const void *p, size_t bytes, const char *what);
size_t bounds_room(const void *p); // bytes from p to the end of its allocation; SIZE_MAX when unknown
unsigned int *bounds_device_word();
#define GPTOSS_SPAN(ptr, bytes)                                                                   \
  do {                                                                                            \
    if ((ptr) && !gptoss::bounds_span_ok((ptr), (size_t)(bytes), #ptr))                           \
      return GPTOSS_ERR_BAD_ARG;                                                                  \
  } while (0)
#else
inline void bounds_register(const void *, size_t) {}
inline void bounds_unregister(const void *) {}
#define GPTOSS_SPAN(ptr, bytes)                                                                   \
  do {                                                                                            \
  } while (0)
#endif
// Bytes behind the first element of T rows of `width` elements `stride` elements apart.
inline size_t strided_bytes(long T, long stride, long width, size_t elem) {
  return T <= 0 ? 0 : ((size_t)(T - 1) * (size_t)stride + (size_t)width) * elem;
}

// ---- 128-bit memory access ----------------------------------------------------

// Read-once data (activations streamed through the kernel): do not keep the
// line in L1.  A coherent load, so in-place operation (the same thread later
// overwrites what it read) stays well defined.
__device__ __forceinline__ uint4 ld_stream(const void *p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Data that is read, then written back by the same thread (the residual row):
// plain coherent load.
__device__ __forceinline__ uint4 ld_plain(const void *p) {
  return *reinterpret_cast<const uint4 *>(p);
}

// Small tables shared by every row (gains, bias, cos/sin): keep them cached.
__device__ __forceinline__ uint4 ld_table(const void *p) {
  return __ldg(reinterpret_cast<const uint4 *>(p));
}

// Written once, not read again by this kernel.
#ifndef GPTOSS_STORE_POLICY
#define GPTOSS_STORE_POLICY 0 // 0: evict-first (.cs)   1: default write-back   2: no L1, write-back (.cg)
#endif
__device__ __forceinline__ void st_stream(void *p, uint4 v) {
#if GPTOSS_STORE_POLICY == 0
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
#elif GPTOSS_STORE_POLICY == 1
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
#else
  asm volatile("st.global.cg.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
#endif
}

__device__ __forceinline__ void st_stream8(void *p, uint2 v) {
  asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// ---- asynchronous global -> shared copies (row staging) -------------------------
//
// The row kernels stage whole rows in shared memory with cp.async: a thread
// queues 16-byte copies for rows several iterations ahead, so the bytes in
// flight per SM are set by the shared-memory ring (100-200 KB), not by how many
// registers a thread can spare.  Every thread only ever reads back the pieces
// it copied itself, so cp.async.wait_group is the only synchronisation the data
// needs (a hardware wait, not a software spin).

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
// The same through L1 (.ca): for small read-only tables that many rows, warps and
// blocks of an SM ask for again and again (a position's cos/sin row).  Kept in L1, the
// repeats never reach L2 -- when a whole batch sits at one position every block wants
// the same two cache lines, and without L1 that single L2 line becomes a hot spot.
__device__ __forceinline__ void cp_async16_cached(void *smem_dst, const void *gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- bulk asynchronous copies (one instruction per row) ----------------------------
//
// cp.async.bulk moves a whole contiguous run (a row of 5-20 KB here) between global and
// this block's shared memory with one instruction issued by one thread; the copy engine
// does the address generation that the 16-byte cp.async form spends hundreds of LSU
// instructions per row on.  A load signals an mbarrier in shared memory with the bytes it
// delivered; a store belongs to the issuing thread's bulk group.  Both ends must be 16-byte
// aligned and the size a multiple of 16.  Source and destination are this GPU's memory and
// this block's shared memory only.
//
// Waiting on an mbarrier is the one software wait in the library, so it is bounded: after
// kWaitCycles SM clocks (half a second) without the phase completing, mbar_wait gives up and returns false;
// the kernel then counts the event in a device word (wait_giveups_word(), read back by
// gptoss_wait_giveups) and winds down instead of hanging the GPU.

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void *bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
// Makes freshly initialised barriers visible to the copy engine (then __syncthreads()).
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// One arrival that also announces `bytes` of copies to come in this phase.
__device__ __forceinline__ void mbar_expect(void *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
constexpr long long kWaitCycles = 1000000000ll; // about half a second of SM clock
__device__ __forceinline__ bool mbar_wait(void *bar, uint32_t parity) {
  const uint32_t a = smem_u32(bar);
  const long long t0 = clock64();
  for (;;) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(a), "r"(parity)
                 : "memory");
    if (done)
      return true;
    if (clock64() - t0 > kWaitCycles)
      return false;
  }
}
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, void *bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void *gmem_dst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most N of this thread's bulk groups are still reading their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Orders this thread's ordinary shared-memory writes before later reads by the copy engine.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Device word counting bounded waits that ran out (current device); nullptr if unavailable.
unsigned int *wait_giveups_word();

// The same copies and the read-back by 32-bit shared-space address (smem_u32 of the buffer plus
// a byte offset kept in a register): no generic-pointer arithmetic in a kernel's inner loop.
__device__ __forceinline__ void cp16_cg(uint32_t smem_dst, const void *gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp16_ca(uint32_t smem_dst, const void *gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
// With the source optional: when `take` is false nothing is read and the 16 bytes are filled
// with zeros (the instruction's source-size operand), so a caller can leave a piece out
// without a branch.  gmem_src must still be a valid address.
__device__ __forceinline__ void cp16_cg_or_zeros(uint32_t smem_dst, const void *gmem_src, bool take) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(take ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// Ring depth for a row kernel whose stage takes stage_bytes of shared memory:
// deep enough to keep >= ~100 KB per SM in flight, shallow enough that two or
// more blocks still fit on an SM (227 KB); 0 if even two stages do not fit.
inline int pick_stages(size_t stage_bytes) {
  if (stage_bytes * 4 <= 72 * 1024)
    return 4;
  if (stage_bytes * 3 <= 110 * 1024)
    return 3;
  if (stage_bytes * 2 <= 220 * 1024)
    return 2;
  return 0;
}

// ---- bf16 <-> fp32 --------------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) {
  return __uint_as_float(pair & 0xffff0000u);
}

// Round to nearest even on the upper 16 bits; a NaN stays a (quiet) NaN.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u)
    return (u >> 16) | 0x40u;
  u += 0x7fffu + ((u >> 16) & 1u);
  return u >> 16;
}

// Two fp32 values to a bf16 pair in one instruction (round to nearest even;
// a NaN becomes the canonical quiet NaN 0x7fff).
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Fast 2^x and 1/x (about 2 ulp and 1 ulp; flush denormals), one MUFU each.
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Eight consecutive values of a row held by one thread.
struct Vec8 {
  float v[8];
};
__device__ __forceinline__ Vec8 floats_of(uint4 a, uint4 b) {
  Vec8 v;
  v.v[0] = __uint_as_float(a.x), v.v[1] = __uint_as_float(a.y), v.v[2] = __uint_as_float(a.z),
  v.v[3] = __uint_as_float(a.w), v.v[4] = __uint_as_float(b.x), v.v[5] = __uint_as_float(b.y),
  v.v[6] = __uint_as_float(b.z), v.v[7] = __uint_as_float(b.w);
  return v;
}

// 1 / sqrt(ss / H + eps) of the bf16-activation mode: one reciprocal, one fused multiply-add, one
// reciprocal square root on the special-function unit (about 2 ulp).  The IEEE division, root
// and division of the fp32 mode cost some 30 instructions per thread and row, a tenth of a row
// kernel's whole instruction count.
__device__ __forceinline__ float fast_inv_rms(float ss, int H) {
  const float m = fmaf(ss, fast_rcp((float)H), GPTOSS_RMS_EPS);
  float r;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(m));
  return r;
}

enum { kStream = 0, kPlain = 1, kTable = 2 };

template <int KIND> __device__ __forceinline__ uint4 ld16(const void *p) {
  if (KIND == kStream)
    return ld_stream(p);
  if (KIND == kPlain)
    return ld_plain(p);
  return ld_table(p);
}

template <int KIND> __device__ __forceinline__ Vec8 load8_f32(const float *base, size_t e) {
  const uint4 a = ld16<KIND>(base + e), b = ld16<KIND>(base + e + 4);
  Vec8 r;
  r.v[0] = __uint_as_float(a.x), r.v[1] = __uint_as_float(a.y), r.v[2] = __uint_as_float(a.z),
  r.v[3] = __uint_as_float(a.w), r.v[4] = __uint_as_float(b.x), r.v[5] = __uint_as_float(b.y),
  r.v[6] = __uint_as_float(b.z), r.v[7] = __uint_as_float(b.w);
  return r;
}

__device__ __forceinline__ Vec8 widen8(uint4 a) {
  Vec8 r;
  r.v[0] = bf16_lo(a.x), r.v[1] = bf16_hi(a.x), r.v[2] = bf16_lo(a.y), r.v[3] = bf16_hi(a.y),
  r.v[4] = bf16_lo(a.z), r.v[5] = bf16_hi(a.z), r.v[6] = bf16_lo(a.w), r.v[7] = bf16_hi(a.w);
  return r;
}

template <int KIND> __device__ __forceinline__ Vec8 load8_bf16(const uint16_t *base, size_t e) {
  return widen8(ld16<KIND>(base + e));
}

// dtype-generic: T is float or uint16_t (bf16 bits).
template <int KIND, typename T> __device__ __forceinline__ Vec8 load8(const T *base, size_t e) {
  if constexpr (sizeof(T) == 4)
    return load8_f32<KIND>(reinterpret_cast<const float *>(base), e);
  else
    return load8_bf16<KIND>(reinterpret_cast<const uint16_t *>(base), e);
}

__device__ __forceinline__ void store8_f32(float *base, size_t e, const Vec8 &r, bool stream) {
  const uint4 a = make_uint4(__float_as_uint(r.v[0]), __float_as_uint(r.v[1]),
                             __float_as_uint(r.v[2]), __float_as_uint(r.v[3]));
  const uint4 b = make_uint4(__float_as_uint(r.v[4]), __float_as_uint(r.v[5]),
                             __float_as_uint(r.v[6]), __float_as_uint(r.v[7]));
  if (stream) {
    st_stream(base + e, a);
    st_stream(base + e + 4, b);
  } else {
    *reinterpret_cast<uint4 *>(base + e) = a;
    *reinterpret_cast<uint4 *>(base + e + 4) = b;
  }
}

__device__ __forceinline__ void store8_bf16(uint16_t *base, size_t e, const Vec8 &r) {
  st_stream(base + e, make_uint4(pack_bf16(r.v[0], r.v[1]), pack_bf16(r.v[2], r.v[3]),
                                 pack_bf16(r.v[4], r.v[5]), pack_bf16(r.v[6], r.v[7])));
}

template <typename T>
__device__ __forceinline__ void store8(T *base, size_t e, const Vec8 &r, bool stream = true) {
  if constexpr (sizeof(T) == 4)
    store8_f32(reinterpret_cast<float *>(base), e, r, stream);
  else
    store8_bf16(reinterpret_cast<uint16_t *>(base), e, r);
}

// Scalar element access for the generic (unaligned / odd-sized) kernels.
template <typename T> __device__ __forceinline__ float load1(const T *p) {
  if constexpr (sizeof(T) == 4)
    return *reinterpret_cast<const float *>(p);
  else
    return __uint_as_float((uint32_t)*reinterpret_cast<const uint16_t *>(p) << 16);
}
template <typename T> __device__ __forceinline__ void store1(T *p, float v) {
  if constexpr (sizeof(T) == 4)
    *reinterpret_cast<float *>(p) = v;
  else
    *reinterpret_cast<uint16_t *>(p) = (uint16_t)f32_to_bf16_bits(v);
}

// ---- reductions ---------------------------------------------------------------

template <typename T> __device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the block; every thread receives it.  scratch: 32 values of T in
// shared memory, reusable after the next __syncthreads().
template <typename T> __device__ __forceinline__ T block_sum(T v, T *scratch) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  if (lane == 0)
    scratch[warp] = v;
  __syncthreads();
  T t = lane < n_warps ? scratch[lane] : T(0);
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

} // namespace gptoss
