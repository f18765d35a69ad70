// C entry points around the reference's own CPU functions.
//
// TEST INFRASTRUCTURE ONLY.  This file holds no arithmetic of its own: it
// includes the CPU half of the reference's run.cpp (everything before the
// point where that file pulls in its GPU engine), which the Makefile cuts out
// of the reference checkout into a temporary file at build time and names in
// REF_CPU_PART, and forwards each call to the reference's function.  The
// resulting library, oracle/_ref/libgptoss_ref.so, is what the restated oracle
// (gptoss_oracle.c) is pinned against and what produced tests/golden/.
//
// The row-batched entry points loop the reference's per-token functions over
// the rows; with threads > 1 the loop is an OpenMP parallel-for over tokens
// (the reference's functions are re-entrant: they only use local mallocs).
#include REF_CPU_PART

#include <omp.h>

#define REF_API extern "C" __attribute__((visibility("default")))

static int ref_threads(int requested) { return requested > 0 ? requested : omp_get_max_threads(); }

REF_API int ref_max_threads(void) { return omp_get_max_threads(); }

REF_API void ref_rmsnorm(float *o, float *x, float *w, int n) { rmsnorm(o, x, w, n); }
REF_API void ref_softmax(float *x, int n) { softmax(x, n); }
REF_API void ref_topk(float *v, int *idx, float *scores, int n_experts, int k) {
  topk(v, idx, scores, n_experts, k);
}
REF_API void ref_yarn_inv_freq(float theta, int head_dim, float factor, float orig_ctx,
                               float beta_fast, float beta_slow, float *conc, float *inv_freq) {
  compute_concentration_and_inv_freq(theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, conc,
                                     inv_freq);
}
REF_API void ref_yarn_cos_sin(int pos, float theta, int head_dim, float factor, float orig_ctx,
                              float beta_fast, float beta_slow, float *c, float *s) {
  compute_cos_sin(pos, theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, c, s);
}
REF_API void ref_rotate_heads(float *x, float *c, float *s, int n_heads, int head_dim) {
  apply_rotary_emb(x, c, s, n_heads, head_dim);
}
REF_API int ref_argmax(float *p, int n) { return sample_argmax(p, n); }

// ---- row-batched forms (same shapes as the oracle's orc_*_rows) -------------

REF_API void ref_add_rmsnorm_rows(float *x, const float *delta, float *gain, float *normed, int T,
                                  int H, int threads) {
#pragma omp parallel for num_threads(ref_threads(threads)) schedule(static)
  for (int t = 0; t < T; t++) {
    float *xr = x + (size_t)t * H;
    if (delta)
      for (int i = 0; i < H; i++)
        xr[i] += delta[(size_t)t * H + i];
    rmsnorm(normed + (size_t)t * H, xr, gain, H);
  }
}

REF_API void ref_bias_rope_rows(float *qkv, const float *bias, const int *pos, int T, int n_q,
                                int n_kv, int head_dim, float theta, float factor, float orig_ctx,
                                float beta_fast, float beta_slow, int threads) {
  const int row = (n_q + 2 * n_kv) * head_dim;
#pragma omp parallel for num_threads(ref_threads(threads)) schedule(static)
  for (int t = 0; t < T; t++) {
    float *r = qkv + (size_t)t * row;
    if (bias)
      for (int i = 0; i < row; i++)
        r[i] += bias[i];
    float cs[256], sn[256];
    compute_cos_sin(pos[t], theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, cs, sn);
    apply_rotary_emb(r, cs, sn, n_q, head_dim);
    apply_rotary_emb(r + (size_t)n_q * head_dim, cs, sn, n_kv, head_dim);
  }
}

REF_API void ref_router_rows(float *weights, int *experts, float *scores, int T, int n_experts,
                             int k, int threads) {
#pragma omp parallel for num_threads(ref_threads(threads)) schedule(static)
  for (int t = 0; t < T; t++) {
    topk(weights + (size_t)t * k, experts + (size_t)t * k, scores + (size_t)t * n_experts,
         n_experts, k);
    softmax(weights + (size_t)t * k, k);
  }
}

REF_API void ref_argmax_rows(int *out, float *logits, int T, long V, int threads) {
#pragma omp parallel for num_threads(ref_threads(threads)) schedule(static)
  for (int t = 0; t < T; t++)
    out[t] = sample_argmax(logits + (size_t)t * V, (int)V);
}

// ---- the whole forward(), for the loops that only exist inline in it --------

// config_image: the bytes of a Config (run.cpp:25-45).  flat_weights: laid out
// as memory_map_weights() expects.  Runs token i at position i and copies each
// step's logits out.
REF_API int ref_forward_seq(const void *config_image, float *flat_weights, const int *tokens,
                            int n_tokens, float *logits_out) {
  Transformer tr;
  memset(&tr, 0, sizeof tr);
  memcpy(&tr.config, config_image, sizeof(Config));
  memory_map_weights(&tr.weights, &tr.config, flat_weights);
  malloc_run_state(&tr.state, &tr.config);
  for (int i = 0; i < n_tokens; i++) {
    float *lg = forward(&tr, tokens[i], i);
    memcpy(logits_out + (size_t)i * tr.config.vocab_size, lg,
           (size_t)tr.config.vocab_size * sizeof(float));
  }
  free_run_state(&tr.state);
  return 0;
}

REF_API int ref_config_size(void) { return (int)sizeof(Config); }

// ---- the KV-cache layout and the bf16 rounding rule of the reference's kernels ----------
// Four small functions that the reference defines in its HIP headers in host-callable
// form; the Makefile copies their definitions (and nothing else) out of
// kernels/fast_attention.hpp and kernels/fast_common.hpp into REF_CACHE_PART.  The
// qualifiers and the one intrinsic they use are given plain C++ meanings here.
#ifdef REF_CACHE_PART
#include <stdint.h>
#include <string.h>
#define __host__
#define __device__
typedef uint16_t bf16_t;
static inline uint32_t __float_as_uint(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
#include REF_CACHE_PART

REF_API int ref_has_cache_layout(void) { return 1; }
// For n (b, slot, g, i) tuples: where a key element, a value code and the value scale go.
REF_API void ref_cache_indices(long n, const int *b, const int *slot, const int *g, const int *i, int slots,
                               int kv_dim, long long *k_at, long long *vq_at, long long *vs_at) {
  for (long t = 0; t < n; t++) {
    k_at[t] = (long long)kv_index_chunk64(b[t], slot[t], g[t], i[t], slots, kv_dim);
    vq_at[t] = (long long)vq_index_chunk64(b[t], slot[t], g[t], i[t], slots, kv_dim);
    vs_at[t] = (long long)vs_index_chunk64(b[t], slot[t], g[t], slots, kv_dim);
  }
}
REF_API void ref_f32_to_bf16(long n, const float *in, uint16_t *out) {
  for (long t = 0; t < n; t++)
    out[t] = f32_to_bf16(in[t]);
}
#else
REF_API int ref_has_cache_layout(void) { return 0; }
#endif
