/*
 * gptoss_kernels.h -- C ABI of the fused per-layer kernels of the gpt-oss engine,
 * built for NVIDIA B200 (sm_100a).
 *
 * One entry point per launch site of the reference engine's forward loop
 * (getp-csrc/engine/gpu_engine.hpp:461-621 of n30nd/Optimize_Inference_GPT-OSS).
 * Each comment names the reference launcher or kernel the entry point stands in
 * for.  Conventions, the same as the reference's launchers:
 *
 *   - every pointer is a DEVICE pointer owned by the caller; nothing here
 *     allocates, frees or synchronises; work is queued on `stream` and returns;
 *   - tensors are row-major and contiguous unless a row stride is an argument;
 *   - the residual stream `x` is fp32 and is updated in place;
 *   - `T` is the number of token rows (the reference's `B`); T == 0 is a no-op.
 *
 * Unlike the reference (which aborts the process in HIP_CHECK,
 * gpu_engine.hpp:41-49) every call returns a status: GPTOSS_OK, or an error for
 * bad arguments / unsupported shapes (checked before anything is queued) or a
 * failed launch.  There is no CPU fallback: without a CUDA device every compute
 * entry point returns GPTOSS_ERR_CUDA.
 *
 * Arithmetic modes (flags):
 *   GPTOSS_EXACT  follow the CPU program's rounding sequence (run.cpp): double
 *                 sum of squares, glibc's expf algorithm, products and sums
 *                 rounded separately, experts combined in increasing expert
 *                 number.  Meant for fp32 tensors ("fp32 mode").
 *   (default)     the reference's fast path: fp32 math with fused multiply-adds,
 *                 tree sums, fast exponential; bf16 where a result feeds a matrix
 *                 multiply ("bf16-activation mode").
 *   GPTOSS_FMA    with GPTOSS_EXACT: contract x1*c - x2*s, x2*c + x1*s and
 *                 agg += z*w into fused multiply-adds, as a CPU build with
 *                 -march=native and the reference's *_exact HIP kernels do.
 *
 * Launch option (flags), independent of the arithmetic:
 *   GPTOSS_PDL    launch with programmatic stream serialization: the kernel's
 *                 thread blocks may be scheduled as soon as the previous
 *                 kernel in the stream allows it (a producer that signals
 *                 launch completion early, e.g. a GEMM epilogue), which hides
 *                 this kernel's launch latency.  Results do not change: every
 *                 kernel starts with a grid-dependency wait and reads nothing,
 *                 not even its tables, before the previous kernel has
 *                 completed.  These kernels do not signal early themselves;
 *                 between two of them the flag still saves part of the launch
 *                 (the layer chain sets it: a 123-launch step measured 0.5-2 %
 *                 shorter at 4096 tokens, 7-11 % at 512).
 *   GPTOSS_BULK_STAGE  gptoss_qkv_bias_rope only: rows are staged in shared memory by
 *                 the copy engine (cp.async.bulk, one instruction per row, completion on
 *                 an mbarrier, rows written back by a bulk store) instead of by 16-byte
 *                 cp.async copies.  Same bits.  Slower than the default on B200 at every
 *                 size measured, so off unless asked for; ignored by the other kernels.
 */
#ifndef GPTOSS_KERNELS_H
#define GPTOSS_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GPTOSS_API __attribute__((visibility("default")))
#else
#define GPTOSS_API
#endif

/* Opaque CUDA stream handle (a cudaStream_t); NULL is the default stream. */
typedef void *gptoss_stream_t;

typedef enum {
  GPTOSS_F32 = 0,  /* IEEE binary32 */
  GPTOSS_BF16 = 1, /* bfloat16, stored as the upper 16 bits of a binary32 */
} gptoss_dtype_t;

enum {
  GPTOSS_OK = 0,
  GPTOSS_ERR_BAD_ARG = 1,     /* null pointer, negative size, misaligned base */
  GPTOSS_ERR_UNSUPPORTED = 2, /* a shape or dtype the kernels do not cover */
  GPTOSS_ERR_CUDA = 3,        /* launch failed or no usable device; see gptoss_last_cuda_error */
};

enum {
  GPTOSS_EXACT = 1u,
  GPTOSS_FMA = 2u,
  GPTOSS_PDL = 4u,
  GPTOSS_BULK_STAGE = 8u,
};

#define GPTOSS_MAX_TOPK 8      /* k of the router and of the combine */
#define GPTOSS_MAX_EXPERTS 256 /* E of the router */
#define GPTOSS_RMS_EPS 1e-5f   /* the reference hard-codes this (run.cpp:327) */

/* Library version, "major.minor.patch". */
GPTOSS_API const char *gptoss_version(void);
/* Text for a status code. */
GPTOSS_API const char *gptoss_status_string(int status);
/* The cudaError_t (as int) of the last failed CUDA call made by this thread in
 * this library, 0 if none. */
GPTOSS_API int gptoss_last_cuda_error(void);
/* How many times, on the current device since the library was loaded, a kernel gave up a
 * bounded wait for one of its own bulk copies (about half a second without the copy
 * arriving) and stopped early instead of hanging the GPU; the output of that launch is
 * incomplete.  0 in normal operation; -1 if the counter cannot be read.  Synchronises with
 * the device.  No counterpart in the reference, whose kernels never wait in software on this
 * path (its expert-parallel ep_wait_kernel spins without a limit, kernels/moe_ep.hpp). */
GPTOSS_API long gptoss_wait_giveups(void);
/* The checked build of the library (compiled with -DGPTOSS_BOUNDS; build.py makes it as
 * libgptoss_b200_bounds.so) stands in for a memory checker: it knows the device allocations
 * made through gptoss_device_alloc and the chain, refuses (GPTOSS_ERR_BAD_ARG, nothing
 * launched) a call whose shape arguments would walk a pointer past the end of its allocation,
 * and has the kernels skip and count any row or expert number read from device data that
 * points outside the array it indexes.  gptoss_bounds_enabled: 1 in that build, 0 otherwise.
 * gptoss_bounds_violations: refused calls plus skipped accesses so far (0 in the ordinary
 * build; -1 if the device counter cannot be read).  gptoss_bounds_checked_spans: how many
 * pointer arguments have been checked against a known allocation.  The reference has no
 * counterpart; its tests rely on canaries around outputs (tests/small_kernels_test.cpp). */
GPTOSS_API int gptoss_bounds_enabled(void);
GPTOSS_API long gptoss_bounds_violations(void);
GPTOSS_API long gptoss_bounds_checked_spans(void);
/* How many launches this thread has made so far that fell back to a scalar kernel
 * (sizes that are not multiples of 8 elements, bases that are not 16-byte aligned,
 * rows too wide for the vector kernels).  Results are the same; the speed is not.  A
 * caller that expects the fast path reads it before and after. */
GPTOSS_API long gptoss_generic_launch_count(void);

/*
 * Token-embedding gather: x[t,:] = table[ids[t],:].
 * Replaces embed_kernel (kernels/misc.hpp:16-23; launch gpu_engine.hpp:461-464)
 * and the CPU's memcpy (run.cpp:544-545).  A bf16 table may be widened to fp32
 * (bits << 16) or copied as bf16; an fp32 table is copied as fp32.  Rows are
 * copied bit for bit.  An id outside [0, V) yields a row of zeros.
 */
GPTOSS_API int gptoss_embed(gptoss_stream_t stream, int T, const void *table,
                            gptoss_dtype_t table_dtype, int V, const int *ids, void *x,
                            gptoss_dtype_t x_dtype, int H, unsigned flags);

/*
 * The gather and the first layer's norm in one launch:
 *     x[t,:] = table[ids[t],:] (as fp32);   out[t,:] = weight * x[t,:] / sqrt(mean(x^2) + eps)
 * Replaces the pair embed_kernel + rmsnorm_bf16_kernel / rmsnorm_exact that opens every step
 * (gpu_engine.hpp:461-464 with :479 or :491-492; run.cpp:544-545 and :550 for layer 0).  Results
 * are those of gptoss_embed followed by gptoss_add_rmsnorm(y = NULL) with the same flags, bit for
 * bit; x is not read back in between.  out must not alias x.
 */
GPTOSS_API int gptoss_embed_rmsnorm(gptoss_stream_t stream, int T, const void *table,
                                    gptoss_dtype_t table_dtype, int V, const int *ids, float *x,
                                    const float *weight, void *out, gptoss_dtype_t out_dtype, int H,
                                    unsigned flags);

/*
 * Residual add fused with RMSNorm (eps 1e-5):
 *     if (y) x[t,:] += y[t,:];   out[t,:] = weight * x[t,:] / sqrt(mean(x^2) + eps)
 * With y: replaces add_rmsnorm_bf16 (kernels/fast_misc.hpp:237-267; launch
 * gpu_engine.hpp:503-504) and, with GPTOSS_EXACT, add_inplace_kernel +
 * rmsnorm_exact (kernels/misc.hpp:88-93, 28-50; launches gpu_engine.hpp:507, 519)
 * = run.cpp:653-658.  Without y (NULL): replaces rmsnorm_bf16_kernel
 * (fast_misc.hpp:12-31; launch gpu_engine.hpp:491-492) / rmsnorm_exact
 * (gpu_engine.hpp:479, 615) = rmsnorm() run.cpp:320-333; x is then only read and
 * out may alias x when out_dtype is fp32 (the final norm, run.cpp:751).
 */
GPTOSS_API int gptoss_add_rmsnorm(gptoss_stream_t stream, int T, float *x, const void *y,
                                  gptoss_dtype_t y_dtype, const float *weight, void *out,
                                  gptoss_dtype_t out_dtype, int H, unsigned flags);

/*
 * QKV bias add fused with YaRN RoPE:
 *     row = qkv_in[t,:] (+ bias);  the n_q_heads query heads and the n_kv_heads
 *     key heads are rotated (pairs (i, i + head_dim/2)) by the angles of row
 *     pos[t] of the cos/sin tables; the value heads only get the bias.
 * Replaces the bias add of the QKV GEMM epilogue (kernels/fast_gemm.hpp:295-300,
 * 338-354; run.cpp:568-570) plus rope_exact (kernels/misc.hpp:55-70; launch
 * gpu_engine.hpp:481) and the rotation of rope_kv_bf16 / rope_pair
 * (kernels/fast_misc.hpp:48-127, kernels/fast_common.hpp:25-28; launch
 * gpu_engine.hpp:495-496) = apply_rotary_emb run.cpp:506-526, 591-592.
 * cos_tab / sin_tab: [n_pos, head_dim/2] fp32, built on the host (the engine
 * does so with compute_cos_sin, gpu_engine.hpp:388-396; see
 * gptoss_build_rope_tables).  pos: one position per row; NULL means every row
 * is at position pos_scalar (the engine's one position per step,
 * gpu_engine.hpp:476).  Positions are clamped into [0, n_pos).  bias may be
 * NULL.  qkv_out may be qkv_in (same dtype and stride) for in-place use.  Row
 * strides are in elements.  head_dim must be a multiple of 16.
 */
GPTOSS_API int gptoss_qkv_bias_rope(gptoss_stream_t stream, int T, const void *qkv_in,
                                    gptoss_dtype_t in_dtype, long in_row_stride,
                                    const float *bias, const int *pos, int pos_scalar,
                                    const float *cos_tab, const float *sin_tab, int n_pos,
                                    int n_q_heads, int n_kv_heads, int head_dim, void *qkv_out,
                                    gptoss_dtype_t out_dtype, long out_row_stride,
                                    unsigned flags);

/*
 * Router: the k largest of each row's E logits in descending order (equal
 * values: lower expert first; -0 equals +0), then softmax over those k.
 * Replaces router_topk_wave_kernel / router_topk_exact (kernels/moe.hpp:64-136,
 * 15-52; launch gpu_engine.hpp:524-529) = topk() + softmax() run.cpp:387-420,
 * 335-353, 671-674.  The softmax always follows the CPU's rounding sequence
 * (the reference uses one kernel for both of its paths).  done (may be NULL):
 * rows with done[t] != 0 get expert -1 and weight 0 for all k choices.
 * slot_of (may be NULL): topk_e receives slot_of[e] instead of e.
 * E <= GPTOSS_MAX_EXPERTS, 1 <= k <= min(E, GPTOSS_MAX_TOPK).  A NaN logit is
 * never selected ahead of a number.  k = 4 with E = 32 or 128 (the model
 * family's shapes) runs a kernel of its own with a shorter dependent chain;
 * every other shape, and scores that do not start on a lane's vector boundary
 * (E / 32 elements), the general one: same results.
 */
GPTOSS_API int gptoss_router_topk(gptoss_stream_t stream, int T, const void *logits,
                                  gptoss_dtype_t logits_dtype, int E, int k, float *topk_w,
                                  int *topk_e, const int *done, const int *slot_of,
                                  unsigned flags);

/*
 * Clamped SwiGLU on R rows of interleaved gate/up values:
 *     g = min(Y[r,2j], limit); u = clamp(Y[r,2j+1], -limit, limit);
 *     G[r,j] = g * sigmoid(1.702 g) * (u + 1)
 * Replaces swiglu_bf16_kernel (kernels/fast_misc.hpp:130-141; launch
 * gpu_engine.hpp:571-572), the same arithmetic in the mlp1 GEMM epilogue
 * (kernels/fast_moe_gemm.hpp:546-571) and, with GPTOSS_EXACT, swiglu_exact
 * (kernels/moe.hpp:186-205; launch gpu_engine.hpp:554) = run.cpp:701-724.
 */
GPTOSS_API int gptoss_swiglu(gptoss_stream_t stream, const void *Y, gptoss_dtype_t y_dtype,
                             void *G, gptoss_dtype_t g_dtype, size_t R, int I, float limit,
                             unsigned flags);

/*
 * Weighted expert combine fused with the residual, optionally with the next
 * RMSNorm:
 *     x[t,:] += sum_j topk_w[t,j] * Z[own_row[t*k+j],:];
 *     if (norm_w) out[t,:] = RMSNorm(x[t,:]) * norm_w
 * Replaces moe_combine_rmsnorm (kernels/moe_ep.hpp:479-515, 571-580; launch
 * gpu_engine.hpp:596-603), moe_combine_kernel (kernels/fast_misc.hpp:154-166)
 * and, with GPTOSS_EXACT, moe_combine_exact / moe_combine_ep_kernel<true>
 * (kernels/moe.hpp:210-236, kernels/moe_ep.hpp:286-332; launch
 * gpu_engine.hpp:590-593) = run.cpp:677-748.  Default mode adds the choices in
 * choice order j = 0..k-1 with fused multiply-adds; GPTOSS_EXACT adds them in
 * increasing expert number (phys_of, may be NULL, maps renumbered experts back
 * for that order).  A row whose first expert is negative is a finished request:
 * x is left as it is, but the row still gets its norm.  own_row NULL means row
 * t*k+j; a negative own_row entry (what gptoss_moe_group writes for a pair
 * whose expert is outside its range) means "no row here": the pair is skipped,
 * nothing is read for it (moe_combine_ep_kernel's range test,
 * kernels/moe_ep.hpp:286-332).  norm_w NULL skips the norm (out is then
 * ignored).
 */
GPTOSS_API int gptoss_moe_combine(gptoss_stream_t stream, int T, float *x, const void *Z,
                                  gptoss_dtype_t z_dtype, const int *own_row,
                                  const float *topk_w, const int *topk_e, int k, int H,
                                  const int *phys_of, const float *norm_w, void *out,
                                  gptoss_dtype_t out_dtype, unsigned flags);

/*
 * Greedy pick: out[t] = index of the largest of logits[t, 0..V), the lowest
 * index on ties (-0 equals +0), exactly as sample_argmax (run.cpp:778-789)
 * decides: a NaN is never picked over a number, and a row whose element 0 is
 * NaN, or that holds no number above -inf, gives 0.
 * Replaces argmax_kernel (kernels/misc.hpp:97-129; launch gpu_engine.hpp:617)
 * and the key merge of gemm_bf16_argmax (kernels/fast_gemm.hpp:94-104, 706-714,
 * 901-926; launch gpu_engine.hpp:619).  Each row may be scanned by several
 * thread blocks that merge through 64-bit keys (order-preserving value bits,
 * then ~index) with atomicMax: keys is scratch of T 64-bit words that must be
 * zero on entry and is left zero, like the reference's `keys` argument.  keys
 * may be NULL: each row is then scanned by a single block.  row_stride in
 * elements.
 */
GPTOSS_API int gptoss_argmax(gptoss_stream_t stream, int T, const void *logits,
                             gptoss_dtype_t logits_dtype, long V, long row_stride,
                             unsigned long long *keys, int *out, unsigned flags);

/*
 * Grouping of the n_pairs (token, choice) pairs by expert, for the local
 * experts e_begin .. e_begin + e_count - 1: rows offsets[e] .. offsets[e+1]
 * (offsets has e_count + 1 entries) hold the pairs that chose local expert e,
 * in pair order; counts[e] is their number; row_pair[row] is the pair index
 * (token * k + choice) and own_row[pair] its row, or -1 when the pair's expert
 * is not local or the token is finished (expert -1).  own_row is the row map
 * gptoss_moe_combine reads through.
 * Replaces moe_group_ep without a partner (kernels/moe_ep.hpp:44-257; launch
 * gpu_engine.hpp:542) and moe_group_kernel (kernels/moe.hpp:138-171).  Integer
 * results, reproduced exactly.  A step beside the path the fused kernels sit
 * on (it feeds the expert GEMMs), provided so that a caller gets own_row from
 * the same library.
 */
GPTOSS_API int gptoss_moe_group(gptoss_stream_t stream, const int *topk_e, int n_pairs,
                                int e_begin, int e_count, int *counts, int *offsets,
                                int *row_pair, int *own_row, unsigned flags);

/*
 * Row gather for the expert GEMM input: Xg[row,:] = t[row_pair[row] / k, :] for
 * R rows, bit for bit (same element type on both sides, fp32 or bf16).
 * Replaces moe_gather_kernel (kernels/moe.hpp:175-182), gather_bf16_kernel
 * (kernels/fast_misc.hpp:144-151) and moe_gather_ep_bf16 without a partner
 * (kernels/moe_ep.hpp:337-368; launch gpu_engine.hpp:567-568).  n_tokens bounds
 * the source rows: a row_pair entry outside [0, n_tokens * k) yields zeros.
 */
GPTOSS_API int gptoss_moe_gather(gptoss_stream_t stream, int R, const void *t,
                                 gptoss_dtype_t dtype, int n_tokens, const int *row_pair, int k,
                                 void *Xg, int H, unsigned flags);

/*
 * gptoss_qkv_bias_rope and gptoss_kv_cache_write in one launch, which is what the
 * reference's rope_kv_bf16 is (kernels/fast_misc.hpp:48-127; launch gpu_engine.hpp:495-496):
 * the row is biased and rotated and written to qkv_out as by gptoss_qkv_bias_rope, and
 * its key heads (bf16) and value heads (int8 codes + scale) also go to the caches as by
 * gptoss_kv_cache_write (arguments kc .. slot_scalar as there), taken from the fp32 values
 * before they are rounded to out_dtype -- the reference's order, and the same bits as the
 * two calls when out_dtype is fp32.  head_dim must be 64 and slots a multiple of 64.
 * Shapes or alignments the one-launch kernel does not take (rows or caches not 16-byte
 * aligned, more than 16,384 elements per row) are served by two launches that store the
 * same bits: the cache is written first, from the input rows with the bias and the
 * rotation redone in fp32, then the rows are rotated.
 */
GPTOSS_API int gptoss_qkv_bias_rope_kv(gptoss_stream_t stream, int T, const void *qkv_in,
                                       gptoss_dtype_t in_dtype, long in_row_stride, const float *bias,
                                       const int *pos, int pos_scalar, const float *cos_tab,
                                       const float *sin_tab, int n_pos, int n_q_heads, int n_kv_heads,
                                       int head_dim, void *qkv_out, gptoss_dtype_t out_dtype,
                                       long out_row_stride, uint16_t *kc, int8_t *vq, float *vs, int slots,
                                       const int *slot_of_row, int slot_scalar, unsigned flags);

/*
 * KV-cache write of one decode step, the half of rope_kv_bf16 that follows the
 * rotation (kernels/fast_misc.hpp:48-127; launch gpu_engine.hpp:495-496): from
 * each row of the biased, rotated qkv tensor (gptoss_qkv_bias_rope's output)
 *   - the n_kv_heads key heads go to kc as bf16 (round to nearest even), at
 *     (row, slot, head g, dim i) ->
 *       (row * slots + (slot & ~63)) * kv_dim + g * 4096 + (slot & 63) * 64 + i
 *     with kv_dim = n_kv_heads * 64 (kv_index_chunk64, fast_attention.hpp:558);
 *   - the value heads go to vq as int8 codes c = round(v * 127 / max|v|)
 *     clamped to +-127, at the byte offset of vq_index_chunk64
 *     (fast_attention.hpp:591), and one fp32 scale max|v| / 127 per (slot, head)
 *     to vs at vs_index_chunk64 (:597); an all-zero value vector gives codes 0
 *     and scale 0.
 * slot_of_row: the cache slot of each row (NULL: slot_scalar for every row, the
 * engine's one slot per step); a slot outside [0, slots) skips the row.  slots
 * must be a multiple of 64 and head_dim 64 (the layouts are defined for that).
 * The row index doubles as the sequence index, as in the engine's decode step.
 * Beside the path the fused kernels sit on (it feeds the attention kernel).
 */
GPTOSS_API int gptoss_kv_cache_write(gptoss_stream_t stream, int T, const void *qkv,
                                     gptoss_dtype_t qkv_dtype, long row_stride, int n_q_heads,
                                     int n_kv_heads, int head_dim, uint16_t *kc, int8_t *vq, float *vs,
                                     int slots, const int *slot_of_row, int slot_scalar,
                                     unsigned flags);

/*
 * The second half of a greedy pick fused into a logits producer: out[t] = the
 * column named by keys[t] (0 if nothing was folded in), then keys[t] = 0.
 * The producer folds its values into keys with the device functions of
 * gptoss_argmax_key.cuh and never stores the logits.  Replaces
 * argmax_keys_kernel (kernels/fast_gemm.hpp:706-714; launch :925) of
 * gemm_bf16_argmax (gpu_engine.hpp:619).  Unlike gptoss_argmax, which sees the
 * logits, this cannot reproduce sample_argmax's answer for a row whose
 * element 0 is NaN (the CPU then returns 0); a NaN simply never wins.
 */
GPTOSS_API int gptoss_argmax_keys_finish(gptoss_stream_t stream, int T, unsigned long long *keys,
                                         int *out, unsigned flags);

/* How many slices (thread blocks) gptoss_argmax cuts each row into for T rows
 * of V logits on the current device; has_keys = 0 describes a call with
 * keys == NULL (always 1).  More than one slice means a second, tiny launch
 * decodes the merged keys. */
GPTOSS_API int gptoss_argmax_slices(int T, long V, gptoss_dtype_t logits_dtype, int has_keys);

/*
 * gptoss_argmax for callers that cannot hand over scratch memory.  It has no
 * counterpart in the reference (whose launcher always receives `keys` from
 * the engine); it exists for hosts that have no device allocator to call at
 * this point -- for example a plug-in inside a serving process whose memory
 * pool already owns the whole GPU, or a decode loop that must stay clear of
 * cudaMalloc because an allocation stalls all streams of the device.
 *
 * Same result as gptoss_argmax, bit for bit.  The per-row merge words live in
 * a fixed array inside the library (GPTOSS_ARGMAX_NOALLOC_MAX_ROWS words of 8
 * bytes = 128 KB, resident on every GPU that loads the library until the
 * process ends), so:
 *   - T above GPTOSS_ARGMAX_NOALLOC_MAX_ROWS is refused with
 *     GPTOSS_ERR_UNSUPPORTED and a line on stderr saying so (split the batch,
 *     or use gptoss_argmax);
 *   - all calls on one GPU share that array: the call clears the words it
 *     needs before it starts, but two calls whose work overlaps in time on the
 *     same GPU (different streams or threads) would corrupt each other --
 *     keep them on one stream or order them yourself;
 *   - the first call on each GPU looks up the array's device address; make
 *     that first call before any stream capture begins.
 * The call itself allocates nothing, on the device or in the CUDA runtime.
 */
#define GPTOSS_ARGMAX_NOALLOC_MAX_ROWS 16384
GPTOSS_API int gptoss_argmax_noalloc(gptoss_stream_t stream, int T, const void *logits,
                                     gptoss_dtype_t logits_dtype, long V, long row_stride,
                                     int *out);

#ifdef __cplusplus
}
#endif
#endif /* GPTOSS_KERNELS_H */
