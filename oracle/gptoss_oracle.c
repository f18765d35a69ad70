/*
 * CPU oracle for the fused per-layer ops of the gpt-oss engine.
 *
 * THIS FILE IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, in plain C,
 * the arithmetic of the reference's CPU program (run.cpp of
 * n30nd/Optimize_Inference_GPT-OSS) for every op on the hot path, so that the
 * CUDA kernels can be compared with it on identical inputs.  Only the test
 * suite, the smoke check and the bench's CPU-baseline legs may load it.  The
 * shipped library never links or calls anything defined here.
 *
 * Parity status: PINNED.  Every function below is compared bit for bit with
 * the reference's own compiled functions (rmsnorm, softmax, topk,
 * compute_cos_sin, apply_rotary_emb, sample_argmax) and, for the loops that
 * only exist inline in forward() (bias add, SwiGLU, expert combine, residual),
 * through a whole tiny-model forward() run of the reference against
 * orc_forward_seq() here.  The steps on either side of the path, which the CPU
 * program does not have, are held to the reference's GPU kernels, whose bodies
 * the reference library compiles as host code and runs on host threads: pair
 * grouping and the row gather (moe_group_kernel, moe_gather_kernel,
 * moe_count_ep_kernel + moe_place_ep_kernel), the KV-cache write (the index
 * functions, f32_to_bf16, quantize_v of the attention test, and
 * rope_kv_bf16_kernel as a whole), the contracted rotation and combine
 * (rope_exact, moe_combine_exact), and the wave bookkeeping (the host statements
 * of gpu_run_wave).  The golden vectors under tests/golden/ were produced by the
 * reference's code and are checked against this file on every run.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -fPIC -shared (no -ffast-math, no
 * -march=native: the reference baseline build is "-O3 -fopenmp", which on
 * x86-64 has no fused multiply-add, and the restatement keeps every rounding
 * step of that build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* single-row primitives                                                      */
/* ------------------------------------------------------------------------ */

/* RMSNorm of one row.  Follows run.cpp:320-333: the squares are float
 * products, their sum is kept in double in index order, eps is the float
 * constant 1e-5f, the reciprocal root is computed in float and the two
 * scalings are done in double and rounded once. */
ORC_API void orc_rmsnorm(float *out, const float *x, const float *gain, int n) {
  double acc = 0.0;
  for (int j = 0; j < n; j++) {
    float sq = x[j] * x[j];
    acc += (double)sq;
  }
  acc /= (double)n;
  acc += (double)1e-5f;
  float root = sqrtf((float)acc);
  double inv = (double)(1.0f / root);
  for (int j = 0; j < n; j++) {
    double scaled = inv * (double)x[j];
    out[j] = (float)((double)gain[j] * scaled);
  }
}

/* Softmax in place.  Follows run.cpp:335-353: the maximum and the sum are
 * doubles, each exponent argument is (double)x - max narrowed to float, the
 * division is done in double and narrowed. */
ORC_API void orc_softmax(float *x, int n) {
  double top = (double)x[0];
  for (int i = 1; i < n; i++)
    if ((double)x[i] > top)
      top = (double)x[i];
  double total = 0.0;
  for (int i = 0; i < n; i++) {
    float arg = (float)((double)x[i] - top);
    x[i] = expf(arg);
    total += (double)x[i];
  }
  for (int i = 0; i < n; i++)
    x[i] = (float)((double)x[i] / total);
}

typedef struct {
  float score;
  int expert;
} orc_scored_t;

/* Descending by score; equal scores compare equal (run.cpp:377-384), so their
 * order is whatever the C library's qsort leaves: glibc 2.39's qsort is a
 * stable merge sort, which keeps equal scores in increasing expert order. */
static int orc_by_score_desc(const void *pa, const void *pb) {
  float d = ((const orc_scored_t *)pb)->score - ((const orc_scored_t *)pa)->score;
  return d > 0 ? 1 : (d < 0 ? -1 : 0);
}

/* The k best experts of one row of router scores (run.cpp:387-420): qsort of
 * (score, index) pairs, then the first k.  Returns 0, or -1 on the argument
 * errors the reference only prints. */
ORC_API int orc_topk(float *best_scores, int *best_experts, const float *scores,
                     int n_experts, int k) {
  if (n_experts <= 0 || k <= 0 || k > n_experts)
    return -1;
  if (!best_scores || !best_experts || !scores)
    return -1;
  orc_scored_t *tmp = (orc_scored_t *)malloc((size_t)n_experts * sizeof *tmp);
  if (!tmp)
    return -1;
  for (int e = 0; e < n_experts; e++) {
    tmp[e].score = scores[e];
    tmp[e].expert = e;
  }
  qsort(tmp, (size_t)n_experts, sizeof *tmp, orc_by_score_desc);
  for (int j = 0; j < k; j++) {
    best_scores[j] = tmp[j].score;
    best_experts[j] = tmp[j].expert;
  }
  free(tmp);
  return 0;
}

/* YaRN concentration and per-pair inverse frequencies (run.cpp:422-477).
 * All float arithmetic except the division by (beta * 2 * pi), which the
 * reference does in double because M_PI is a double. */
ORC_API void orc_yarn_inv_freq(float theta, int head_dim, float factor, float orig_ctx,
                               float beta_fast, float beta_slow, float *concentration,
                               float *inv_freq) {
  const int half = head_dim / 2;
  if (!(factor > 1.0f)) {
    *concentration = 1.0f;
    for (int i = 0; i < half; i++)
      inv_freq[i] = 1.0f / powf(theta, ((float)(2 * i)) / (float)head_dim);
    return;
  }
  *concentration = 0.1f * logf(factor) + 1.0f;
  const float ln_theta = logf(theta);
  const float lo = (float)half * logf((float)((double)orig_ctx / ((double)(beta_fast * 2.0f) * M_PI))) / ln_theta;
  const float hi = (float)half * logf((float)((double)orig_ctx / ((double)(beta_slow * 2.0f) * M_PI))) / ln_theta;
  for (int i = 0; i < half; i++) {
    const float f = powf(theta, ((float)(2 * i)) / (float)head_dim);
    const float interp = 1.0f / (factor * f);
    const float extrap = 1.0f / f;
    float ramp = ((float)i - lo) / (hi - lo);
    if (ramp < 0)
      ramp = 0;
    if (ramp > 1)
      ramp = 1;
    const float keep = 1.0f - ramp;
    inv_freq[i] = interp * (1.0f - keep) + extrap * keep;
  }
}

/* cos/sin row of one position (run.cpp:479-504). */
ORC_API void orc_yarn_cos_sin(int pos, float theta, int head_dim, float factor, float orig_ctx,
                              float beta_fast, float beta_slow, float *cos_row, float *sin_row) {
  const int half = head_dim / 2;
  float conc;
  float *inv_freq = (float *)malloc((size_t)half * sizeof(float));
  orc_yarn_inv_freq(theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, &conc, inv_freq);
  for (int j = 0; j < half; j++) {
    const float angle = (float)pos * inv_freq[j];
    cos_row[j] = cosf(angle) * conc;
    sin_row[j] = sinf(angle) * conc;
  }
  free(inv_freq);
}

/* Half-split rotation of n_heads heads in place (run.cpp:506-526): pair
 * (i, i + head_dim/2); two products and one add or subtract, each rounded. */
ORC_API void orc_rotate_heads(float *v, const float *cos_row, const float *sin_row, int n_heads,
                              int head_dim) {
  const int half = head_dim / 2;
  for (int h = 0; h < n_heads; h++) {
    float *head = v + (size_t)h * head_dim;
    for (int i = 0; i < half; i++) {
      const float a = head[i], b = head[half + i];
      const float c = cos_row[i], s = sin_row[i];
      const float ac = a * c, bs = b * s, bc = b * c, as = a * s;
      head[i] = ac - bs;
      head[half + i] = bc + as;
    }
  }
}

/* The same rotation as the reference's GPU engine rounds it in its exact path (rope_exact,
 * kernels/misc.hpp:55-70; rope_pair, kernels/fast_common.hpp:25-28), which is also what a CPU
 * build with FMA contraction computes: the first product of each line is fused into the
 * add, the second is rounded on its own. */
ORC_API void orc_rotate_heads_fma(float *v, const float *cos_row, const float *sin_row, int n_heads,
                                  int head_dim) {
  const int half = head_dim / 2;
  for (int h = 0; h < n_heads; h++) {
    float *head = v + (size_t)h * head_dim;
    for (int i = 0; i < half; i++) {
      const float a = head[i], b = head[half + i];
      const float c = cos_row[i], s = sin_row[i];
      const float bs = b * s, as = a * s;
      head[i] = fmaf(a, c, -bs);
      head[half + i] = fmaf(b, c, as);
    }
  }
}

/* Clamped SwiGLU of one interleaved gate/up row (run.cpp:701-724). */
ORC_API void orc_swiglu_row(float *out, const float *gate_up, int n_inter, float limit) {
  const float alpha = 1.702f;
  for (int j = 0; j < n_inter; j++) {
    float g = gate_up[2 * j];
    float u = gate_up[2 * j + 1];
    if (g > limit)
      g = limit;
    if (u > limit)
      u = limit;
    if (u < -limit)
      u = -limit;
    const float sig = 1.0f / (1.0f + expf(-alpha * g));
    g = g * sig;
    g = g * (u + 1.0f);
    out[j] = g;
  }
}

/* Greedy pick (run.cpp:778-789): strict '>' from element 0, so the first
 * maximum wins, a NaN never replaces the running maximum, and a NaN in
 * element 0 is never replaced. */
ORC_API int orc_argmax(const float *p, int n) {
  int best = 0;
  float top = p[0];
  for (int i = 1; i < n; i++)
    if (p[i] > top) {
      best = i;
      top = p[i];
    }
  return best;
}

/* ------------------------------------------------------------------------ */
/* row-batched forms: the shapes the GPU entry points take                    */
/* ------------------------------------------------------------------------ */

static int orc_threads(int requested) {
#ifdef _OPENMP
  return requested > 0 ? requested : omp_get_max_threads();
#else
  (void)requested;
  return 1;
#endif
}

ORC_API int orc_max_threads(void) { return orc_threads(0); }

/* x[t,:] = table[ids[t],:] (run.cpp:544-545). */
ORC_API void orc_embed_rows(float *x, const float *table, const int *ids, int T, int H,
                            int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++)
    memcpy(x + (size_t)t * H, table + (size_t)ids[t] * H, (size_t)H * sizeof(float));
}

/* x += delta (run.cpp:653-655) when delta is not NULL, then
 * normed = RMSNorm(x) * gain (run.cpp:658).  normed may alias x (run.cpp:751). */
ORC_API void orc_add_rmsnorm_rows(float *x, const float *delta, const float *gain,
                                  float *normed, int T, int H, int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    float *xr = x + (size_t)t * H;
    if (delta) {
      const float *dr = delta + (size_t)t * H;
      for (int i = 0; i < H; i++)
        xr[i] += dr[i];
    }
    orc_rmsnorm(normed + (size_t)t * H, xr, gain, H);
  }
}

/* qkv[t,:] += bias (run.cpp:568-570), then the q heads and the k heads of the
 * row are rotated by the angles of pos[t] (run.cpp:588-592; the reference
 * recomputes the cos/sin row for every token and layer, and so does this). */
ORC_API void orc_bias_rope_rows(float *qkv, const float *bias, const int *pos, int T,
                                int n_q_heads, int n_kv_heads, int head_dim, float theta,
                                float factor, float orig_ctx, float beta_fast, float beta_slow,
                                int threads) {
  const int row = (n_q_heads + 2 * n_kv_heads) * head_dim;
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    float *r = qkv + (size_t)t * row;
    if (bias)
      for (int i = 0; i < row; i++)
        r[i] += bias[i];
    float cs[256], sn[256]; /* head_dim <= 512 */
    orc_yarn_cos_sin(pos[t], theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, cs, sn);
    orc_rotate_heads(r, cs, sn, n_q_heads, head_dim);
    orc_rotate_heads(r + (size_t)n_q_heads * head_dim, cs, sn, n_kv_heads, head_dim);
  }
}

/* Rotation with a ready cos/sin table indexed by position, the form the GPU
 * engine uses (gpu_engine.hpp:388-396, 476). */
ORC_API void orc_bias_rope_rows_table(float *qkv, const float *bias, const int *pos, int T,
                                      int n_q_heads, int n_kv_heads, int head_dim,
                                      const float *cos_tab, const float *sin_tab, int threads) {
  const int row = (n_q_heads + 2 * n_kv_heads) * head_dim, half = head_dim / 2;
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    float *r = qkv + (size_t)t * row;
    if (bias)
      for (int i = 0; i < row; i++)
        r[i] += bias[i];
    const float *cs = cos_tab + (size_t)pos[t] * half, *sn = sin_tab + (size_t)pos[t] * half;
    orc_rotate_heads(r, cs, sn, n_q_heads, head_dim);
    orc_rotate_heads(r + (size_t)n_q_heads * head_dim, cs, sn, n_kv_heads, head_dim);
  }
}

/* The same with the contracted rotation (orc_rotate_heads_fma). */
ORC_API void orc_bias_rope_rows_table_fma(float *qkv, const float *bias, const int *pos, int T,
                                          int n_q_heads, int n_kv_heads, int head_dim,
                                          const float *cos_tab, const float *sin_tab, int threads) {
  const int row = (n_q_heads + 2 * n_kv_heads) * head_dim, half = head_dim / 2;
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    float *r = qkv + (size_t)t * row;
    if (bias)
      for (int i = 0; i < row; i++)
        r[i] += bias[i];
    const float *cs = cos_tab + (size_t)pos[t] * half, *sn = sin_tab + (size_t)pos[t] * half;
    orc_rotate_heads_fma(r, cs, sn, n_q_heads + n_kv_heads, head_dim);
  }
}

/* Build the cos/sin table for positions 0..n_pos-1. */
ORC_API void orc_yarn_table(float *cos_tab, float *sin_tab, int n_pos, float theta, int head_dim,
                            float factor, float orig_ctx, float beta_fast, float beta_slow,
                            int threads) {
  const int half = head_dim / 2;
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int p = 0; p < n_pos; p++)
    orc_yarn_cos_sin(p, theta, head_dim, factor, orig_ctx, beta_fast, beta_slow,
                     cos_tab + (size_t)p * half, sin_tab + (size_t)p * half);
}

/* Top-k then softmax of each row of router scores (run.cpp:671-674). */
ORC_API void orc_router_rows(float *weights, int *experts, const float *scores, int T,
                             int n_experts, int k, int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    orc_topk(weights + (size_t)t * k, experts + (size_t)t * k, scores + (size_t)t * n_experts,
             n_experts, k);
    orc_softmax(weights + (size_t)t * k, k);
  }
}

ORC_API void orc_swiglu_rows(float *out, const float *gate_up, long R, int n_inter, float limit,
                             int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (long r = 0; r < R; r++)
    orc_swiglu_row(out + (size_t)r * n_inter, gate_up + (size_t)r * 2 * n_inter, n_inter, limit);
}

/* x[t,:] += sum over the token's k experts of weight * Z[row,:], the experts
 * taken in increasing expert number as forward() visits them
 * (run.cpp:677-748): agg starts at zero, each expert adds product-then-sum,
 * and agg is added to x at the end.  row_of[t*k+j] is the row of Z holding
 * the output of choice j of token t.  A token whose first expert is negative
 * is a finished request and is left untouched (gpu_engine's convention).  A
 * pair whose row_of entry is negative has no expert row on this device (the
 * grouping step's -1 for an expert outside its range) and adds nothing, as in
 * moe_combine_ep_kernel's `e >= e_begin && e < e_begin + e_count` test
 * (kernels/moe_ep.hpp:286-332). */
ORC_API void orc_combine_rows(float *x, const float *Z, const int *row_of, const float *weights,
                              const int *experts, int T, int k, int H, int n_experts,
                              int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    const int *ex = experts + (size_t)t * k;
    if (ex[0] < 0)
      continue;
    float *agg = (float *)calloc((size_t)H, sizeof(float));
    for (int e = 0; e < n_experts; e++) {
      int hit = -1;
      for (int j = 0; j < k; j++)
        if (ex[j] == e) {
          hit = j;
          break;
        }
      if (hit < 0 || row_of[(size_t)t * k + hit] < 0)
        continue;
      const float w = weights[(size_t)t * k + hit];
      const float *z = Z + (size_t)row_of[(size_t)t * k + hit] * H;
      for (int i = 0; i < H; i++) {
        const float prod = z[i] * w;
        agg[i] += prod;
      }
    }
    float *xr = x + (size_t)t * H;
    for (int i = 0; i < H; i++)
      xr[i] += agg[i];
    free(agg);
  }
}

ORC_API void orc_argmax_rows(int *out, const float *logits, int T, long V, int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++)
    out[t] = orc_argmax(logits + (size_t)t * V, (int)V);
}

/* The combine as the reference's GPU engine rounds it in its exact path (moe_combine_exact,
 * kernels/moe.hpp:210-236): the token's experts in increasing expert number, a chain of fused
 * multiply-adds from zero, one add into x.  Equal expert numbers keep their choice order (the
 * kernel's insertion sort is stable).  Finished tokens (expert -1) are left alone, as by
 * orc_combine_rows. */
ORC_API void orc_combine_rows_fma(float *x, const float *Z, const int *row_of, const float *weights,
                                  const int *experts, int T, int k, int H, int threads) {
  const int nt = orc_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static)
  for (int t = 0; t < T; t++) {
    const int *ex = experts + (size_t)t * k;
    if (ex[0] < 0 || k > 64)
      continue;
    int order[64];
    for (int j = 0; j < k; j++)
      order[j] = j;
    for (int i = 1; i < k; i++)
      for (int j = i; j > 0 && ex[order[j]] < ex[order[j - 1]]; j--) {
        const int tmp = order[j];
        order[j] = order[j - 1];
        order[j - 1] = tmp;
      }
    float *xr = x + (size_t)t * H;
    for (int i = 0; i < H; i++) {
      float acc = 0.0f;
      for (int j = 0; j < k; j++) {
        const size_t p = (size_t)t * k + order[j];
        if (row_of[p] >= 0)
          acc = fmaf(Z[(size_t)row_of[p] * H + i], weights[p], acc);
      }
      xr[i] += acc;
    }
  }
}

/* Grouping of (token, choice) pairs by expert, the contract of the reference's
 * moe_group_kernel / moe_group_ep (kernels/moe.hpp:138-171, kernels/moe_ep.hpp:44-49):
 * rows offsets[e] .. offsets[e+1] belong to local expert e_begin + e, in pair
 * order; row_pair[row] is the pair (token * k + choice) in that row and
 * own_row[pair] its inverse, -1 for a pair whose expert is not local (or -1,
 * a finished token).  The reference's forward() loops over experts instead, so
 * the pins are its GPU kernels, run on host threads by the reference library
 * (one per GPU thread, a barrier for __syncthreads, 64 threads to a wavefront
 * for ballot and shuffle): moe_group_kernel over all experts, and
 * moe_count_ep_kernel + moe_place_ep_kernel (kernels/moe_ep.hpp:55-127) with
 * no partner for part of them; tests/test_oracle_pins.py holds this function
 * to both. */
ORC_API void orc_moe_group(const int *topk_e, int n_pairs, int e_begin, int e_count, int *counts,
                           int *offsets, int *row_pair, int *own_row) {
  int row = 0;
  for (int e = 0; e < e_count; e++) {
    offsets[e] = row;
    for (int p = 0; p < n_pairs; p++)
      if (topk_e[p] == e_begin + e) {
        row_pair[row] = p;
        own_row[p] = row;
        row++;
      }
    counts[e] = row - offsets[e];
  }
  offsets[e_count] = row;
  for (int p = 0; p < n_pairs; p++)
    if (topk_e[p] < e_begin || topk_e[p] >= e_begin + e_count)
      own_row[p] = -1;
}

/* Xg[row,:] = t[row_pair[row] / k, :] (moe_gather_kernel, kernels/moe.hpp:175-182). */
ORC_API void orc_moe_gather(float *Xg, const float *t, const int *row_pair, int R, int k, int H) {
  for (int r = 0; r < R; r++)
    memcpy(Xg + (size_t)r * H, t + (size_t)(row_pair[r] / k) * H, (size_t)H * sizeof(float));
}

/* KV-cache write of one decode step: the cache half of the reference's
 * rope_kv_bf16_kernel (kernels/fast_misc.hpp:48-108) with the chunk64 index
 * functions of kernels/fast_attention.hpp:558-600.  qkv rows are already biased
 * and rotated.  Keys: bf16 round-to-nearest-even.  Values: amax = max|v| over
 * the head's 64 numbers, inv = amax > 0 ? 127/amax : 0, code =
 * clamp(rintf(v*inv), +-127), scale = amax/127, all in fp32.  The kernel itself
 * has no CPU form in the reference, but its three parts do, and
 * tests/test_oracle_pins.py holds each against them: the layout (the three index
 * functions) and the bf16 rounding rule are host-callable in the reference's
 * headers, the value rule is quantize_v of its attention test. */
static size_t orc_chunk64(int b, int slot, int g, int i, int slots, int kv_dim) {
  return ((size_t)b * slots + (size_t)(slot & ~63)) * kv_dim + (size_t)g * 64 * 64 +
         (size_t)(slot & 63) * 64 + i;
}
static uint16_t orc_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u)
    return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
/* The three index functions and the rounding rule on their own, so that they can be
 * held against the reference's (which, unlike the kernel around them, are callable on
 * the host). */
ORC_API void orc_cache_indices(long n, const int *b, const int *slot, const int *g, const int *i, int slots,
                               int kv_dim, long long *k_at, long long *vq_at, long long *vs_at) {
  for (long t = 0; t < n; t++) {
    k_at[t] = (long long)orc_chunk64(b[t], slot[t], g[t], i[t], slots, kv_dim);
    vq_at[t] = (long long)(orc_chunk64(b[t], slot[t] & ~15, g[t], 0, slots, kv_dim) + ((slot[t] >> 2) & 3) * 256 +
                           (i[t] >> 2) * 16 + (i[t] & 3) * 4 + (slot[t] & 3));
    vs_at[t] = (long long)(orc_chunk64(b[t], slot[t], g[t], 0, slots, kv_dim) / 64);
  }
}
ORC_API void orc_f32_to_bf16(long n, const float *in, uint16_t *out) {
  for (long t = 0; t < n; t++)
    out[t] = orc_bf16(in[t]);
}

/* The int8 form of one 64-wide value head (kernels/fast_misc.hpp:79-87; in host code,
 * quantize_v of tests/attn_test.cpp:218-226): scale = max|v| / 127, code = v * (127 / max|v|)
 * rounded to the nearest integer, ties to even, and held to [-127, 127]; a head of zeros
 * gives zero codes and a zero scale. */
static void orc_value_head(const float *v, int8_t *codes, float *scale) {
  float amax = 0.0f;
  for (int i = 0; i < 64; i++)
    amax = fmaxf(amax, fabsf(v[i]));
  const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
  for (int i = 0; i < 64; i++) {
    float c = rintf(v[i] * inv);
    c = fminf(fmaxf(c, -127.0f), 127.0f);
    codes[i] = (int8_t)c;
  }
  *scale = amax / 127.0f;
}
ORC_API void orc_value_codes(long n_heads, const float *v, int8_t *codes, float *scales) {
  for (long h = 0; h < n_heads; h++)
    orc_value_head(v + h * 64, codes + h * 64, scales + h);
}

ORC_API void orc_kv_cache_write(const float *qkv, long row_stride, int T, int n_q_heads, int n_kv_heads,
                                uint16_t *kc, int8_t *vq, float *vs, int slots, const int *slot_of_row) {
  const int kv_dim = n_kv_heads * 64;
  for (int b = 0; b < T; b++) {
    const int slot = slot_of_row[b];
    if (slot < 0 || slot >= slots)
      continue;
    const float *k = qkv + (size_t)b * row_stride + (size_t)n_q_heads * 64, *v = k + kv_dim;
    for (int g = 0; g < n_kv_heads; g++) {
      int8_t codes[64];
      float scale;
      for (int i = 0; i < 64; i++)
        kc[orc_chunk64(b, slot, g, i, slots, kv_dim)] = orc_bf16(k[g * 64 + i]);
      orc_value_head(v + g * 64, codes, &scale);
      for (int i = 0; i < 64; i++) {
        const size_t at = orc_chunk64(b, slot & ~15, g, 0, slots, kv_dim) + ((slot >> 2) & 3) * 256 +
                          (i >> 2) * 16 + (i & 3) * 4 + (slot & 3);
        vq[at] = codes[i];
      }
      vs[orc_chunk64(b, slot, g, 0, slots, kv_dim) / 64] = scale;
    }
  }
}

/* What a wave of requests looks like from outside, given the tokens each step picked
 * (engine/gpu_engine.hpp:761-841, the host statements between its GPU calls).  Stated row
 * by row instead of step by step, since rows do not interact except through when the wave
 * ends.  A row with np prompt tokens is fed prompt[p] in step p while p < np and afterwards
 * the token its previous step picked, picked[(p - 1) * n_rows + b]; tokens fed from the
 * model are recorded at out[p - np]; the first end token (199999 or 200002) fed at p >= 1
 * finishes the row at f = p.  The wave runs P = min(steps, latest finish) steps, or `steps`
 * when some row never finishes.  A finished row gets a -1 behind its tokens at f - np + 1
 * and counts f - np + 1 generated tokens; an unfinished one the same with P for f (the
 * count may be negative for a prompt longer than the wave, and is added as it is).
 * fed[s * n_rows + b]: the token row b was given in step s (a finished row keeps its last).
 * mask[s * n_rows + b]: whether the device saw row b as finished during step s (f <= s).
 * out_rows is [n_rows, width] and only the entries named above are written. */
ORC_API long long orc_wave_bookkeeping(int n_rows, const int *prompt_tokens, const int *prompt_offsets,
                                       int steps, const int *picked, int width, int *out_rows,
                                       int *done_out, int *steps_run, int *fed, int *mask) {
  int *finish = (int *)malloc((size_t)(n_rows > 0 ? n_rows : 1) * sizeof(int));
  int latest = 0, all_finish = 1;
  for (int b = 0; b < n_rows; b++) {
    const int *prompt = prompt_tokens + prompt_offsets[b];
    const int np = prompt_offsets[b + 1] - prompt_offsets[b];
    finish[b] = -1;
    for (int p = 1; p <= steps; p++) {
      const int token = p < np ? prompt[p] : picked[(size_t)(p - 1) * n_rows + b];
      if (token == 199999 || token == 200002) {
        finish[b] = p;
        break;
      }
    }
    if (finish[b] < 0)
      all_finish = 0;
    else if (finish[b] > latest)
      latest = finish[b];
  }
  const int P = (all_finish && n_rows > 0) ? (latest < steps ? latest : steps) : (n_rows > 0 ? steps : 0);
  long long count = 0;
  for (int b = 0; b < n_rows; b++) {
    const int *prompt = prompt_tokens + prompt_offsets[b];
    const int np = prompt_offsets[b + 1] - prompt_offsets[b];
    int *out = out_rows + (size_t)b * width;
    const int f = (finish[b] >= 0 && finish[b] <= P) ? finish[b] : -1;
    const int last = f >= 0 ? f : P;
    int token = prompt[0];
    for (int s = 0; s < P; s++) {
      if (s >= 1 && s <= last) {
        token = s < np ? prompt[s] : picked[(size_t)(s - 1) * n_rows + b];
        if (s >= np)
          out[s - np] = token;
      }
      fed[(size_t)s * n_rows + b] = token;
      mask[(size_t)s * n_rows + b] = f >= 0 && f <= s;
    }
    if (last >= 1 && last == P && last >= np) /* the token fed to a step that never ran */
      out[last - np] = picked[(size_t)(last - 1) * n_rows + b];
    if (last - np + 1 >= 0)
      out[last - np + 1] = -1;
    count += last - np + 1;
    done_out[b] = f >= 0;
  }
  free(finish);
  *steps_run = P;
  return count;
}

/* Host expf, exported so tests can compare a device exponential with the C
 * library's on chosen inputs. */
ORC_API void orc_expf_array(float *out, const float *in, long n) {
  for (long i = 0; i < n; i++)
    out[i] = expf(in[i]);
}

/* ------------------------------------------------------------------------ */
/* whole-model forward, used only to pin this file against the reference      */
/* ------------------------------------------------------------------------ */

typedef struct {
  int vocab, hidden, n_experts, top_k, inter, n_layers, head_dim, n_q_heads, n_kv_heads, seq_len,
      orig_ctx;
  float theta, factor;
  int window;
  float limit;
} orc_config_t; /* same field order as run.cpp:25-45, so one byte image serves both */

/* out[d] = W[d,n] . x[n] with a double accumulator over float products
 * (run.cpp:355-368). */
static void orc_matvec(float *out, const float *x, const float *W, int n, int d) {
  for (int i = 0; i < d; i++) {
    double acc = 0.0;
    for (int j = 0; j < n; j++) {
      const float prod = W[(size_t)i * n + j] * x[j];
      acc += (double)prod;
    }
    out[i] = (float)acc;
  }
}

/* Runs n_tokens decode steps (token i at position i) and writes each step's
 * logits.  flat_weights is laid out as memory_map_weights() expects
 * (run.cpp:207-247).  Restates forward() (run.cpp:528-756) using the row
 * primitives above.  Returns 0. */
ORC_API int orc_forward_seq(const orc_config_t *c, const float *flat_weights, const int *tokens,
                            int n_tokens, float *logits_out) {
  const int H = c->hidden, D = c->head_dim, NQ = c->n_q_heads, NKV = c->n_kv_heads;
  const int QKV = (NQ + 2 * NKV) * D, KVD = NKV * D, E = c->n_experts, K = c->top_k,
            I = c->inter, L = c->n_layers, S = c->seq_len, V = c->vocab;
  const float *p = flat_weights;
  const float *emb = p;        p += (size_t)V * H;
  const float *unemb = p;      p += (size_t)V * H;
  const float *g_attn = p;     p += (size_t)L * H;
  const float *g_ffn = p;      p += (size_t)L * H;
  const float *g_out = p;      p += (size_t)H;
  const float *w_qkv = p;      p += (size_t)L * H * QKV;
  const float *b_qkv = p;      p += (size_t)L * QKV;
  const float *w_o = p;        p += (size_t)L * NQ * D * H;
  const float *b_o = p;        p += (size_t)L * H;
  const float *sinks = p;      p += (size_t)L * NQ;
  const float *w_router = p;   p += (size_t)L * H * E;
  const float *b_router = p;   p += (size_t)L * E;
  const float *w_mlp1 = p;     p += (size_t)L * E * 2 * I * H;
  const float *b_mlp1 = p;     p += (size_t)L * E * 2 * I;
  const float *w_mlp2 = p;     p += (size_t)L * E * H * I;
  const float *b_mlp2 = p;

  float *x = calloc(H, 4), *t = calloc(H, 4), *qkv = calloc(QKV, 4), *attn = calloc(NQ * D, 4);
  float *proj = calloc(H, 4), *router = calloc(E, 4), *tw = calloc(K, 4);
  int *te = calloc(K, sizeof(int));
  float *y = calloc(2 * I, 4), *act = calloc(I, 4), *agg = calloc(H, 4);
  float *kc = calloc((size_t)L * S * KVD, 4), *vc = calloc((size_t)L * S * KVD, 4);
  float *score = calloc((size_t)S + 2, 4);
  float cs[256], sn[256];

  for (int step = 0; step < n_tokens; step++) {
    const int pos = step;
    memcpy(x, emb + (size_t)tokens[step] * H, (size_t)H * 4);
    for (int l = 0; l < L; l++) {
      orc_rmsnorm(t, x, g_attn + (size_t)l * H, H);
      orc_matvec(qkv, t, w_qkv + (size_t)l * H * QKV, H, QKV);
      for (int i = 0; i < QKV; i++)
        qkv[i] += b_qkv[(size_t)l * QKV + i];
      orc_yarn_cos_sin(pos, c->theta, D, c->factor, (float)c->orig_ctx, 32.0f, 1.0f, cs, sn);
      orc_rotate_heads(qkv, cs, sn, NQ, D);
      orc_rotate_heads(qkv + NQ * D, cs, sn, NKV, D);
      float *kl = kc + (size_t)l * S * KVD, *vl = vc + (size_t)l * S * KVD;
      memcpy(kl + (size_t)pos * KVD, qkv + NQ * D, (size_t)KVD * 4);
      memcpy(vl + (size_t)pos * KVD, qkv + NQ * D + KVD, (size_t)KVD * 4);
      const int group = NQ / NKV;
      for (int h = 0; h < NQ; h++) {
        const float *q = qkv + h * D;
        for (int u = 0; u <= pos; u++) {
          const float *k = kl + (size_t)u * KVD + (h / group) * D;
          double dot = 0.0;
          for (int i = 0; i < D; i++) {
            const float prod = q[i] * k[i];
            dot += (double)prod;
          }
          dot /= (double)sqrtf((float)D);
          if (c->window > 0 && (l % 2 == 0)) {
            const float m = (pos - u >= c->window) ? -INFINITY : 0.0f;
            dot += (double)m;
          }
          score[u] = (float)dot;
        }
        score[pos + 1] = sinks[(size_t)l * NQ + h];
        orc_softmax(score, pos + 2);
        float *o = attn + h * D;
        memset(o, 0, (size_t)D * 4);
        for (int u = 0; u <= pos; u++) {
          const float *v = vl + (size_t)u * KVD + (h / group) * D;
          const float a = score[u];
          for (int i = 0; i < D; i++) {
            const float prod = a * v[i];
            o[i] += prod;
          }
        }
      }
      orc_matvec(proj, attn, w_o + (size_t)l * NQ * D * H, NQ * D, H);
      for (int i = 0; i < H; i++)
        proj[i] += b_o[(size_t)l * H + i];
      for (int i = 0; i < H; i++)
        x[i] += proj[i];
      orc_rmsnorm(t, x, g_ffn + (size_t)l * H, H);
      orc_matvec(router, t, w_router + (size_t)l * H * E, H, E);
      for (int i = 0; i < E; i++)
        router[i] += b_router[(size_t)l * E + i];
      orc_topk(tw, te, router, E, K);
      orc_softmax(tw, K);
      memset(agg, 0, (size_t)H * 4);
      for (int e = 0; e < E; e++) {
        int hit = -1;
        for (int j = 0; j < K; j++)
          if (te[j] == e) {
            hit = j;
            break;
          }
        if (hit < 0)
          continue;
        const size_t le = (size_t)l * E + e;
        orc_matvec(y, t, w_mlp1 + le * 2 * I * H, H, 2 * I);
        for (int i = 0; i < 2 * I; i++)
          y[i] += b_mlp1[le * 2 * I + i];
        orc_swiglu_row(act, y, I, c->limit);
        orc_matvec(proj, act, w_mlp2 + le * H * I, I, H);
        for (int i = 0; i < H; i++)
          proj[i] += b_mlp2[le * H + i];
        for (int i = 0; i < H; i++) {
          const float prod = proj[i] * tw[hit];
          agg[i] += prod;
        }
      }
      for (int i = 0; i < H; i++)
        x[i] += agg[i];
    }
    orc_rmsnorm(x, x, g_out, H);
    orc_matvec(logits_out + (size_t)step * V, x, unemb, H, V);
  }
  free(x); free(t); free(qkv); free(attn); free(proj); free(router); free(tw); free(te);
  free(y); free(act); free(agg); free(kc); free(vc); free(score);
  return 0;
}
