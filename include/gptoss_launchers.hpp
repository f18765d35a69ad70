// gptoss_launchers.hpp -- the reference engine's launcher names on top of the C ABI.
//
// The reference (n30nd/Optimize_Inference_GPT-OSS) calls its small kernels through
// `static` launchers and raw `<<<>>>` launches in getp-csrc/engine/gpu_engine.hpp:461-621.
// This header gives a CUDA port of that engine the same names with the same argument
// order and meaning, each forwarding to one entry point of gptoss_kernels.h.  Like the
// reference's HIP_CHECK (gpu_engine.hpp:41-49) a failed call prints and exits.
//
// Plain C++ (no CUDA headers needed): a stream is passed as the opaque gptoss_stream_t,
// i.e. the cudaStream_t itself.  bf16 tensors are raw 16-bit patterns, as in the
// reference (kernels/fast_common.hpp:7).
#ifndef GPTOSS_LAUNCHERS_HPP
#define GPTOSS_LAUNCHERS_HPP

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "gptoss_kernels.h"

#define GPTOSS_CHECK(call)                                                                       \
  do {                                                                                           \
    const int gptoss_st_ = (call);                                                               \
    if (gptoss_st_ != GPTOSS_OK) {                                                               \
      fprintf(stderr, "gptoss error: %s (cudaError %d) at %s:%d\n", gptoss_status_string(gptoss_st_), \
              gptoss_last_cuda_error(), __FILE__, __LINE__);                                     \
      exit(EXIT_FAILURE);                                                                        \
    }                                                                                            \
  } while (0)

namespace gptoss_ref_names {

typedef uint16_t bf16_t;

// gpu_engine.hpp:463  embed_kernel<<<B,256,0,s>>>(emb, tokens, x, H); V bounds the ids.
static inline void embed(gptoss_stream_t s, int B, const bf16_t *emb, int V, const int *tokens, float *x,
                         int H) {
  GPTOSS_CHECK(gptoss_embed(s, B, emb, GPTOSS_BF16, V, tokens, x, GPTOSS_F32, H, 0));
}

// :492  rmsnorm_bf16_kernel<<<B,256,0,s>>>(x, weight, out, H)
static inline void rmsnorm_bf16(gptoss_stream_t s, int B, float *x, const float *weight, bf16_t *out,
                                int H) {
  GPTOSS_CHECK(gptoss_add_rmsnorm(s, B, x, nullptr, GPTOSS_F32, weight, out, GPTOSS_BF16, H, 0));
}

// :479, :519, :615  rmsnorm_exact<<<B,256,H*4,s>>>(x, weight, out, H)
static inline void rmsnorm_exact(gptoss_stream_t s, int B, float *x, const float *weight, float *out,
                                 int H) {
  GPTOSS_CHECK(gptoss_add_rmsnorm(s, B, x, nullptr, GPTOSS_F32, weight, out, GPTOSS_F32, H, GPTOSS_EXACT));
}

// :503  add_rmsnorm_bf16(s, B, x, y, weight, out, H)          (out2, the partner GCD's copy, has no use here)
static inline void add_rmsnorm_bf16(gptoss_stream_t s, int B, float *x, const float *y, const float *weight,
                                    bf16_t *out, int H) {
  GPTOSS_CHECK(gptoss_add_rmsnorm(s, B, x, y, GPTOSS_F32, weight, out, GPTOSS_BF16, H, 0));
}

// :507 + :519  add_inplace_kernel followed by rmsnorm_exact, as one call
static inline void add_inplace_rmsnorm_exact(gptoss_stream_t s, int B, float *x, const float *y,
                                             const float *weight, float *out, int H) {
  GPTOSS_CHECK(gptoss_add_rmsnorm(s, B, x, y, GPTOSS_F32, weight, out, GPTOSS_F32, H, GPTOSS_EXACT));
}

// :481  rope_exact<<<B,256,0,s>>>(qkv, row_stride, cosv, sinv, n_heads, head_dim): cosv / sinv are the
// rows of the step's position; n_heads = query + key heads.  The value heads are not touched, so the
// row is described to the kernel as n_heads rotated heads and no value heads.  Rounds like the
// reference's kernel (fused multiply-adds).
static inline void rope_exact(gptoss_stream_t s, int B, float *qkv, int row_stride, const float *cosv,
                              const float *sinv, int n_heads, int head_dim) {
  GPTOSS_CHECK(gptoss_qkv_bias_rope(s, B, qkv, GPTOSS_F32, row_stride, nullptr, nullptr, 0, cosv, sinv, 1,
                                    n_heads, 0, head_dim, qkv, GPTOSS_F32, row_stride,
                                    GPTOSS_EXACT | GPTOSS_FMA));
}

// :495  rope_kv_bf16(s, B, qkv, row_stride, cosv, sinv, n_q_heads, n_kv_heads, kc, vq, vs, slots, slot,
// rotate_q): rotation (of the keys, and of the queries with rotate_q) and the cache write, one launch.
// One difference: the rotated keys are also left in qkv (the reference writes them to the cache only).
static inline void rope_kv_bf16(gptoss_stream_t s, int B, float *qkv, int row_stride, const float *cosv,
                                const float *sinv, int n_q_heads, int n_kv_heads, bf16_t *kc, int8_t *vq,
                                float *vs, int slots, int slot, bool rotate_q = true) {
  // without rotate_q the row is described from its first key head on: no query heads at all
  float *first = rotate_q ? qkv : qkv + (size_t)n_q_heads * 64;
  GPTOSS_CHECK(gptoss_qkv_bias_rope_kv(s, B, first, GPTOSS_F32, row_stride, nullptr, nullptr, 0, cosv, sinv, 1,
                                       rotate_q ? n_q_heads : 0, n_kv_heads, 64, first, GPTOSS_F32, row_stride,
                                       kc, vq, vs, slots, nullptr, slot, 0));
}

// :525  router_topk_wave_kernel<<<...>>>(logits, E, k, topk_w, topk_e, B, done, slot_of)
static inline void router_topk_wave(gptoss_stream_t s, const float *logits, int E, int k, float *topk_w,
                                    int *topk_e, int B, const int *done, const int *slot_of) {
  GPTOSS_CHECK(gptoss_router_topk(s, B, logits, GPTOSS_F32, E, k, topk_w, topk_e, done, slot_of, 0));
}

// :529  router_topk_exact<<<...>>>(logits, E, k, topk_w, topk_e, B)
static inline void router_topk_exact(gptoss_stream_t s, const float *logits, int E, int k, float *topk_w,
                                     int *topk_e, int B) {
  GPTOSS_CHECK(gptoss_router_topk(s, B, logits, GPTOSS_F32, E, k, topk_w, topk_e, nullptr, nullptr, 0));
}

// :542  moe_group_ep without a partner: counts, offsets, row_pair, own_row for experts e_begin..+e_count
static inline void moe_group(gptoss_stream_t s, const int *topk_e, int n_pairs, int e_begin, int e_count,
                             int *counts, int *offsets, int *row_pair, int *own_row) {
  GPTOSS_CHECK(gptoss_moe_group(s, topk_e, n_pairs, e_begin, e_count, counts, offsets, row_pair, own_row, 0));
}

// :567  moe_gather_ep_bf16 without a partner: Xg16[row,:] = t16[row_pair[row] / k, :]
static inline void moe_gather_bf16(gptoss_stream_t s, int R, const bf16_t *t16, int n_tokens,
                                   const int *row_pair, int k, bf16_t *Xg16, int H) {
  GPTOSS_CHECK(gptoss_moe_gather(s, R, t16, GPTOSS_BF16, n_tokens, row_pair, k, Xg16, H, 0));
}

// :554  swiglu_exact<<<...>>>(Y, G, R, I, limit)
static inline void swiglu_exact(gptoss_stream_t s, const float *Y, float *G, size_t R, int I, float limit) {
  GPTOSS_CHECK(gptoss_swiglu(s, Y, GPTOSS_F32, G, GPTOSS_F32, R, I, limit, GPTOSS_EXACT));
}

// :571  swiglu_bf16_kernel<<<...>>>(Y, G, R, I, limit)
static inline void swiglu_bf16(gptoss_stream_t s, const float *Y, bf16_t *G, size_t R, int I, float limit) {
  GPTOSS_CHECK(gptoss_swiglu(s, Y, GPTOSS_F32, G, GPTOSS_BF16, R, I, limit, 0));
}

// :591  moe_combine_ep_kernel<true> without a partner (= moe_combine_exact): experts in increasing order
static inline void moe_combine_exact(gptoss_stream_t s, int B, float *x, const float *Z, const int *own_row,
                                     const float *topk_w, const int *topk_e, int k, int H,
                                     const int *phys_of) {
  GPTOSS_CHECK(gptoss_moe_combine(s, B, x, Z, GPTOSS_F32, own_row, topk_w, topk_e, k, H, phys_of, nullptr,
                                  nullptr, GPTOSS_F32, GPTOSS_EXACT | GPTOSS_FMA));
}

// :602  moe_combine_rmsnorm(s, B, x, Z, own_row, topk_w, topk_e, k, H, norm_w, out)
static inline void moe_combine_rmsnorm(gptoss_stream_t s, int B, float *x, const float *Z, const int *own_row,
                                       const float *topk_w, const int *topk_e, int k, int H,
                                       const float *norm_w, bf16_t *out) {
  GPTOSS_CHECK(gptoss_moe_combine(s, B, x, Z, GPTOSS_F32, own_row, topk_w, topk_e, k, H, nullptr, norm_w, out,
                                  GPTOSS_BF16, 0));
}

// :617  argmax_kernel<<<B,256,0,s>>>(logits, V, out)   (keys: B zeroed 64-bit words, or nullptr)
static inline void argmax(gptoss_stream_t s, int B, const float *logits, int V, unsigned long long *keys,
                          int *out) {
  GPTOSS_CHECK(gptoss_argmax(s, B, logits, GPTOSS_F32, V, V, keys, out, 0));
}

// :619  the decode half of gemm_bf16_argmax: the GEMM folds into keys (gptoss_argmax_key.cuh)
static inline void argmax_keys(gptoss_stream_t s, unsigned long long *keys, int M, int *out) {
  GPTOSS_CHECK(gptoss_argmax_keys_finish(s, M, keys, out, 0));
}

} // namespace gptoss_ref_names

#endif // GPTOSS_LAUNCHERS_HPP
