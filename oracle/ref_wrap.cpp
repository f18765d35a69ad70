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

// ---- the int8 value rule of the KV cache -------------------------------------------------
// quantize_v of the reference's attention test (tests/attn_test.cpp:218-226): the host form
// of what rope_kv_bf16_kernel does per value head (kernels/fast_misc.hpp:79-87).  It works
// on D values; the test's D is 64, the head width of both models.
#ifdef REF_VALUE_PART
#include <algorithm>
#include <cmath>
namespace ref_value {
constexpr int D = 64;
#include REF_VALUE_PART
} // namespace ref_value
REF_API int ref_has_value_codes(void) { return 1; }
REF_API void ref_value_codes(long n_heads, const float *v, int8_t *codes, float *scales) {
  for (long h = 0; h < n_heads; h++)
    ref_value::quantize_v(v + h * 64, codes + h * 64, scales + h);
}
#else
REF_API int ref_has_value_codes(void) { return 0; }
#endif

// ---- the between-steps bookkeeping of gpu_run_wave ----------------------------------------
// engine/gpu_engine.hpp:696-701 (WaveSlot), :802-826 (after each step) and :828-838 (after
// the loop), included here as they stand, with the Requests struct and get_tok_gen_ptr of
// getp_eval.cpp:9-15, 39-41 (that file as a whole calls into the GPU runner).  What the reference does on
// the GPU between two bookkeeping passes is replaced by recorded tokens: picked[step * n_rows
// + b] is what the step's argmax returned for row b.  fed[step * n_rows + b] receives the
// token the row was fed in that step and mask[step * n_rows + b] the finished-row mask the
// device held during it (copied only when it changed, as the reference copies it).
#if defined(REF_WAVE_TYPES) && defined(REF_WAVE_STEP) && defined(REF_WAVE_TAIL)
#include <vector>
#include REF_WAVE_TYPES
REF_API int ref_has_wave(void) { return 1; }
REF_API long long ref_wave_bookkeeping(int n_rows, const int *prompt_tokens, const int *prompt_offsets,
                                       int steps, const int *picked, int width, int *out_rows,
                                       int *done_out, int *steps_run, int *fed, int *mask) {
  Requests requests;
  memset(&requests, 0, sizeof requests);
  requests.num_reqs = n_rows;
  requests.max_seq_len = width - 1; // rows of get_tok_gen_ptr are max_seq_len + 1 apart
  requests.tok_gens = out_rows;
  Requests *req = &requests;
  std::vector<WaveSlot> slots(1);
  {
    WaveSlot &ws = slots[0];
    ws.first = 0;
    ws.n = n_rows;
    ws.prompts.assign(n_rows, {});
    for (int b = 0; b < n_rows; b++)
      ws.prompts[b].assign(prompt_tokens + prompt_offsets[b], prompt_tokens + prompt_offsets[b + 1]);
    ws.cur.resize(n_rows);
    ws.next.resize(n_rows);
    ws.done.assign(n_rows, 0);
    for (int b = 0; b < n_rows; b++) // wave_slot_init, gpu_engine.hpp:726-727
      ws.cur[b] = ws.prompts[b][0];
  }
  const int n = 1; // one member in the group
  int active = n_rows;
  long long generated = 0;
  int pos = 0;
  std::vector<int> device_mask(n_rows, 0); // hipMemset(row_done, 0), gpu_engine.hpp:773
  while (pos < steps && active > 0) {
    if (slots[0].done_changed) { // :784-788
      device_mask = slots[0].done;
      slots[0].done_changed = false;
    }
    for (int b = 0; b < n_rows; b++) {
      fed[(size_t)pos * n_rows + b] = slots[0].cur[b];
      mask[(size_t)pos * n_rows + b] = device_mask[b];
      slots[0].next[b] = picked[(size_t)pos * n_rows + b];
    }
#include REF_WAVE_STEP
  }
#include REF_WAVE_TAIL
  for (int b = 0; b < n_rows; b++)
    done_out[b] = slots[0].done[b];
  *steps_run = pos;
  return generated;
}
#else
REF_API int ref_has_wave(void) { return 0; }
#endif

// ---- the grouping of (token, choice) pairs by expert, and the row gather --------------------
// moe_group_kernel and moe_gather_kernel (kernels/moe.hpp:142-171, 175-182) as they stand.
// Their bodies are plain C per GPU thread -- a loop over the pairs, a __shared__ array, two
// __syncthreads() -- so a block is run here as host threads: threadIdx is a thread-local, the
// shared array a function-local static, the barrier a pthread barrier.  One block at a time
// (a mutex), as the shared array is one per process.
#ifdef REF_GROUP_PART
#include <pthread.h>

#include <functional>
#include <mutex>
#include <thread>
#include <vector>
namespace ref_group {
struct Index {
  int x;
};
static thread_local Index threadIdx, blockIdx;
static Index blockDim;
static pthread_barrier_t block_barrier;
static std::mutex one_block_at_a_time;
// A 64-wide wavefront's collectives, for the kernels that group for part of the experts
// (kernels/moe_ep.hpp): every lane of the wave calls them together, as on the GPU.
static pthread_barrier_t wave_barrier[16];
static long long wave_slot[16][64];
static inline long long wave_read(long long mine, int src_lane) {
  const int wave = threadIdx.x / 64, lane = threadIdx.x % 64;
  wave_slot[wave][lane] = mine;
  pthread_barrier_wait(&wave_barrier[wave]);
  const long long got = wave_slot[wave][src_lane >= 0 && src_lane < 64 ? src_lane : lane];
  pthread_barrier_wait(&wave_barrier[wave]);
  return got;
}
static inline long long bits_of(float v) {
  int u;
  memcpy(&u, &v, 4);
  return u;
}
static inline float float_of(long long bits) {
  const int u = (int)bits;
  float v;
  memcpy(&v, &u, 4);
  return v;
}
static inline int __shfl_down(int v, int offset) { return (int)wave_read(v, threadIdx.x % 64 + offset); }
static inline int __shfl_xor(int v, int mask) { return (int)wave_read(v, (threadIdx.x % 64) ^ mask); }
static inline float __shfl_xor(float v, int mask) { return float_of(wave_read(bits_of(v), (threadIdx.x % 64) ^ mask)); }
static inline int __shfl(int v, int lane) { return (int)wave_read(v, lane); }
static inline float __shfl(float v, int lane) { return float_of(wave_read(bits_of(v), lane)); }
static inline unsigned long long __ballot(int pred) {
  const int wave = threadIdx.x / 64, lane = threadIdx.x % 64;
  wave_slot[wave][lane] = pred != 0;
  pthread_barrier_wait(&wave_barrier[wave]);
  unsigned long long mask = 0;
  for (int i = 0; i < 64; i++)
    mask |= (unsigned long long)(wave_slot[wave][i] != 0) << i;
  pthread_barrier_wait(&wave_barrier[wave]);
  (void)lane;
  return mask;
}
#define __popcll __builtin_popcountll
#define __launch_bounds__(...)
#define __device__
#define __global__
#define __shared__ static
#define __syncthreads() pthread_barrier_wait(&ref_group::block_barrier)
#include REF_GROUP_PART
#ifdef REF_EXACT_PART
// rope_exact and moe_combine_exact, the GPU engine's bit-exact rotation and combine: plain C per
// thread with the rounding of every step spelled out (__fmaf_rn, __fmul_rn, __fadd_rn); here
// fmaf() and the plain operators (the build targets baseline x86-64, which has no fused
// instruction for the compiler to contract them into; ref_has_exact_kernels() checks it).
static inline float __fmaf_rn(float a, float b, float c) { return fmaf(a, b, c); }
static inline float __fmul_rn(float a, float b) { return a * b; }
static inline float __fadd_rn(float a, float b) { return a + b; }
#include REF_EXACT_PART
#endif
#ifdef REF_GROUP_EP_PART
#include REF_GROUP_EP_PART
#endif
static inline int min(int a, int b) { return a < b ? a : b; }
#if defined(REF_FUSED_PART) && defined(REF_CACHE_PART) && defined(REF_EXACT_PART)
// add_rmsnorm_bf16_kernel (kernels/fast_misc.hpp:237-256, with block_sum256, row_has, load_row256,
// rms_inv_row and rmsnorm_store_bf16 before it) and moe_combine_rmsnorm_kernel
// (kernels/moe_ep.hpp:479-515): the fast path's fused row kernels.  Their row sum meets at a block
// barrier and finishes inside each 64-wide wave with shuffles.
static inline float __shfl_down(float v, int offset) { return float_of(wave_read(bits_of(v), threadIdx.x % 64 + offset)); }
#include REF_FUSED_PART
#define REF_HAS_FUSED 1
#endif
#if defined(REF_FAST_PART) && defined(REF_CACHE_PART)
// Three kernels of the engine's fast (bf16-activation) path: rmsnorm_bf16_kernel, swiglu_bf16_kernel,
// moe_combine_kernel (kernels/fast_misc.hpp:11-30, 130-141, 154-166).  The device's approximate
// __expf has no host twin; the C library's expf stands in (the two differ by a few units in the
// last place of an fp32 value that is then rounded to bf16).
static inline float __expf(float x) { return expf(x); }
#include REF_FAST_PART
#define REF_HAS_FAST 1
#endif
#ifdef REF_ARGMAX_KEY_PART
// argmax_key (kernels/fast_gemm.hpp:94-104): the 64-bit word the LM-head epilogue folds with atomicMax.
#include REF_ARGMAX_KEY_PART
#endif
#if defined(REF_ROPE_KV_PART) && defined(REF_EXACT_PART) && defined(REF_CACHE_PART)
// rope_pair (kernels/fast_common.hpp:25-28) and rope_kv_bf16_kernel (kernels/fast_misc.hpp:48-108):
// the engine's rotation + KV-cache write in one launch.  It calls the index functions and the
// rounding rule included above, and one wave-wide maximum per value head.
#include REF_ROPE_KV_PART
#define REF_HAS_ROPE_KV 1
#endif
#ifdef REF_ROUTER_PART
// router_topk_wave_kernel (kernels/moe.hpp:64-136) with the expf_cpu it calls
// (kernels/exact_math.hpp:12-52): the device's correctly rounded double operations are the
// host's plain ones.
static inline uint32_t __float_as_uint(float v) { return (uint32_t)bits_of(v); }
static inline long long __double_as_longlong(double v) {
  long long u;
  memcpy(&u, &v, 8);
  return u;
}
static inline double __longlong_as_double(long long u) {
  double v;
  memcpy(&v, &u, 8);
  return v;
}
static inline double __dmul_rn(double a, double b) { return a * b; }
static inline double __dadd_rn(double a, double b) { return a + b; }
static inline double __dsub_rn(double a, double b) { return a - b; }
static inline double __ddiv_rn(double a, double b) { return a / b; }
static inline double __fma_rn(double a, double b, double c) { return fma(a, b, c); }
#include REF_ROUTER_PART
#endif
#if defined(REF_EXACT_ROWS_PART) && defined(REF_ROUTER_PART) && defined(REF_EXACT_PART)
// The rest of the GPU engine's bit-exact path: embed_kernel, add_inplace_kernel, argmax_kernel
// (kernels/misc.hpp:10-23, 86-93, 95-129), router_topk_exact and swiglu_exact
// (kernels/moe.hpp:15-52, 186-205; expf_cpu is already in from the router's cut).
static inline float __uint_as_float(uint32_t u) { return float_of((long long)u); }
static inline float __fdiv_rn(float a, float b) { return a / b; }
#include REF_EXACT_ROWS_PART
#define REF_HAS_EXACT_ROWS 1
#endif
#undef __syncthreads
#undef __shared__
#undef __global__
#undef __device__
#undef __launch_bounds__
#undef __popcll
} // namespace ref_group

REF_API int ref_has_group(void) { return 1; }
// One block of E threads, as the reference launches it (E <= 1024).  pair_row keeps the
// caller's fill for pairs of finished tokens (expert -1), which no thread owns.
REF_API void ref_moe_group(const int *topk_e, int n_pairs, int E, int *offsets, int *row_pair, int *pair_row) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  pthread_barrier_init(&ref_group::block_barrier, nullptr, (unsigned)E);
  ref_group::blockDim.x = E;
  std::vector<std::thread> block;
  for (int e = 0; e < E; e++)
    block.emplace_back([=] {
      ref_group::threadIdx.x = e;
      ref_group::blockIdx.x = 0;
      ref_group::moe_group_kernel(topk_e, n_pairs, E, offsets, row_pair, pair_row);
    });
  for (auto &t : block)
    t.join();
  pthread_barrier_destroy(&ref_group::block_barrier);
}
// One block per row, 256 threads each; no barrier inside, so the threads of a block are a loop.
REF_API void ref_moe_gather(const float *x, const int *row_pair, int R, int k, float *Xg, int H) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int row = 0; row < R; row++)
    for (int t = 0; t < 256; t++) {
      ref_group::blockIdx.x = row;
      ref_group::threadIdx.x = t;
      ref_group::moe_gather_kernel(x, row_pair, k, Xg, H);
    }
}

#ifdef REF_EXACT_PART
// 1 if a * b + c written with plain operators rounds twice in this build, as the kernels' spelled-out
// steps require; 0 (and the pin is skipped) if the compiler fused it.
REF_API int ref_has_exact_kernels(void) {
  volatile float a = 1.0f + 0x1p-12f, b = 1.0f + 0x1p-12f, c = -1.0f;
  const float twice = ref_group::__fadd_rn(ref_group::__fmul_rn(a, b), c);
  return twice != fmaf(a, b, c);
}
// No barrier in either kernel: a block's threads are a loop.
REF_API void ref_rope_exact(float *qkv, int B, int row_stride, const float *cosv, const float *sinv, int n_heads,
                            int head_dim) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int b = 0; b < B; b++)
    for (int t = 0; t < 256; t++) {
      ref_group::blockIdx.x = b;
      ref_group::threadIdx.x = t;
      ref_group::rope_exact(qkv, row_stride, cosv, sinv, n_heads, head_dim);
    }
}
REF_API void ref_moe_combine_exact(float *x, int B, const float *Z, const int *pair_row, const float *topk_w,
                                   const int *topk_e, int k, int H) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int b = 0; b < B; b++)
    for (int t = 0; t < 256; t++) {
      ref_group::blockIdx.x = b;
      ref_group::threadIdx.x = t;
      ref_group::moe_combine_exact(x, Z, pair_row, topk_w, topk_e, k, H);
    }
}
#else
REF_API int ref_has_exact_kernels(void) { return 0; }
#endif

#ifdef REF_HAS_EXACT_ROWS
REF_API int ref_has_exact_rows(void) { return 1; }
// Runs `kernel` for every (block, thread) of a launch whose blocks have no barrier.
template <class K> static void run_flat(long blocks, int threads, K kernel) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = threads;
  for (long b = 0; b < blocks; b++)
    for (int t = 0; t < threads; t++) {
      ref_group::blockIdx.x = (int)b;
      ref_group::threadIdx.x = t;
      kernel();
    }
}
REF_API void ref_embed(int B, const uint16_t *emb, const int *tokens, float *x, int H) {
  run_flat(B, 256, [=] { ref_group::embed_kernel(emb, tokens, x, H); });
}
REF_API void ref_add_inplace(float *x, const float *y, long n) {
  run_flat((n + 255) / 256, 256, [=] { ref_group::add_inplace_kernel(x, y, (size_t)n); });
}
REF_API void ref_router_topk_exact(const float *logits, int E, int k, float *topk_w, int *topk_e, int B) {
  run_flat((B + 63) / 64, 64, [=] { ref_group::router_topk_exact(logits, E, k, topk_w, topk_e, B); });
}
REF_API void ref_swiglu_exact(const float *Y, float *G, long R, int I, float limit) {
  run_flat((R * I + 255) / 256, 256, [=] { ref_group::swiglu_exact(Y, G, (size_t)R, I, limit); });
}
// argmax_kernel merges through shared arrays with a block barrier per level: 256 host threads per row.
REF_API void ref_argmax_kernel(int B, const float *logits, int V, int *out) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int block = 0; block < B; block++) {
    pthread_barrier_init(&ref_group::block_barrier, nullptr, 256);
    std::vector<std::thread> pool;
    for (int t = 0; t < 256; t++)
      pool.emplace_back([=] {
        ref_group::threadIdx.x = t;
        ref_group::blockIdx.x = block;
        ref_group::argmax_kernel(logits, V, out);
      });
    for (auto &t : pool)
      t.join();
    pthread_barrier_destroy(&ref_group::block_barrier);
  }
}
#else
REF_API int ref_has_exact_rows(void) { return 0; }
#endif

#ifdef REF_HAS_FUSED
REF_API int ref_has_fused_kernels(void) { return 1; }
// A block of 256 host threads with the block barrier and four wave barriers set up.
template <class K> static void run_blocks_256(int blocks, K kernel) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int block = 0; block < blocks; block++) {
    pthread_barrier_init(&ref_group::block_barrier, nullptr, 256);
    for (int w = 0; w < 4; w++)
      pthread_barrier_init(&ref_group::wave_barrier[w], nullptr, 64);
    std::vector<std::thread> pool;
    for (int t = 0; t < 256; t++)
      pool.emplace_back([=] {
        ref_group::threadIdx.x = t;
        ref_group::blockIdx.x = block;
        kernel();
      });
    for (auto &t : pool)
      t.join();
    for (int w = 0; w < 4; w++)
      pthread_barrier_destroy(&ref_group::wave_barrier[w]);
    pthread_barrier_destroy(&ref_group::block_barrier);
  }
}
// Instantiated as the launchers do (kernels/fast_misc.hpp:259-267, kernels/moe_ep.hpp:563-573).
REF_API void ref_add_rmsnorm_bf16(int B, float *x, const float *y, const float *weight, uint16_t *out, int H) {
  if ((H + 255) / 256 == 12)
    run_blocks_256(B, [=] { ref_group::add_rmsnorm_bf16_kernel<12>(x, y, weight, out, H, nullptr); });
  else
    run_blocks_256(B, [=] { ref_group::add_rmsnorm_bf16_kernel<FUSED_ROW_MAX>(x, y, weight, out, H, nullptr); });
}
REF_API void ref_moe_combine_rmsnorm(int B, float *x, const float *Z, const int *own_row, const float *topk_w,
                                     const int *topk_e, int k, int H, const float *norm_w, uint16_t *out) {
  if (k <= 4 && (H + 255) / 256 == 12)
    run_blocks_256(B, [=] { ref_group::moe_combine_rmsnorm_kernel<4, 12>(x, Z, own_row, topk_w, topk_e, k, H, norm_w, out); });
  else
    run_blocks_256(B, [=] {
      ref_group::moe_combine_rmsnorm_kernel<MOE_MAX_TOPK, FUSED_ROW_MAX>(x, Z, own_row, topk_w, topk_e, k, H, norm_w, out);
    });
}
#else
REF_API int ref_has_fused_kernels(void) { return 0; }
#endif

#ifdef REF_HAS_FAST
REF_API int ref_has_fast_kernels(void) { return 1; }
// One block of 256 threads per row; the halving tree has a block barrier per level.
REF_API void ref_rmsnorm_bf16(int B, const float *x, const float *weight, uint16_t *out, int H) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int block = 0; block < B; block++) {
    pthread_barrier_init(&ref_group::block_barrier, nullptr, 256);
    std::vector<std::thread> pool;
    for (int t = 0; t < 256; t++)
      pool.emplace_back([=] {
        ref_group::threadIdx.x = t;
        ref_group::blockIdx.x = block;
        ref_group::rmsnorm_bf16_kernel(x, weight, out, H);
      });
    for (auto &t : pool)
      t.join();
    pthread_barrier_destroy(&ref_group::block_barrier);
  }
}
// No barrier in these two: a block's threads are a loop.
REF_API void ref_swiglu_bf16(const float *Y, uint16_t *G, long R, int I, float limit) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  const long blocks = (R * I + 255) / 256;
  for (long block = 0; block < blocks; block++)
    for (int t = 0; t < 256; t++) {
      ref_group::blockIdx.x = (int)block;
      ref_group::threadIdx.x = t;
      ref_group::swiglu_bf16_kernel(Y, G, (size_t)R, I, limit);
    }
}
REF_API void ref_moe_combine_fast(int B, float *x, const float *Z, const int *pair_row, const float *topk_w, int k,
                                  int H) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  ref_group::blockDim.x = 256;
  for (int block = 0; block < B; block++)
    for (int t = 0; t < 256; t++) {
      ref_group::blockIdx.x = block;
      ref_group::threadIdx.x = t;
      ref_group::moe_combine_kernel(x, Z, pair_row, topk_w, k, H);
    }
}
#else
REF_API int ref_has_fast_kernels(void) { return 0; }
#endif

#ifdef REF_ARGMAX_KEY_PART
REF_API int ref_has_argmax_key(void) { return 1; }
REF_API void ref_argmax_keys(long n, const float *x, const int *col, unsigned long long *keys) {
  for (long i = 0; i < n; i++)
    keys[i] = ref_group::argmax_key(x[i], col[i]);
}
#else
REF_API int ref_has_argmax_key(void) { return 0; }
#endif

#ifdef REF_HAS_ROPE_KV
REF_API int ref_has_rope_kv(void) { return 1; }
// B blocks of 256 threads (four 64-wide waves, no block barrier), instantiated as the launcher
// rope_kv_bf16 chooses (kernels/fast_misc.hpp:110-127): rotate_q = 0 starts at the first key head.
REF_API void ref_rope_kv_bf16(int B, float *qkv, int row_stride, const float *cosv, const float *sinv, int n_q_heads,
                              int n_kv_heads, uint16_t *kc, int8_t *vq, float *vs, int slots, int slot, int rotate_q) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  const int h0 = rotate_q ? 0 : n_q_heads;
  const int ns = (n_q_heads + n_kv_heads - h0 + 7) / 8, nv = (n_kv_heads * 64 + 255) / 256;
  ref_group::blockDim.x = 256;
  for (int block = 0; block < B; block++) {
    for (int w = 0; w < 4; w++)
      pthread_barrier_init(&ref_group::wave_barrier[w], nullptr, 64);
    std::vector<std::thread> pool;
    for (int t = 0; t < 256; t++)
      pool.emplace_back([=] {
        ref_group::threadIdx.x = t;
        ref_group::blockIdx.x = block;
        if (ns == 1 && nv == 2)
          ref_group::rope_kv_bf16_kernel<1, 2>(qkv, row_stride, cosv, sinv, n_q_heads, n_kv_heads, h0, kc, vq, vs, slots, slot);
        else if (ns == 9 && nv == 2)
          ref_group::rope_kv_bf16_kernel<9, 2>(qkv, row_stride, cosv, sinv, n_q_heads, n_kv_heads, h0, kc, vq, vs, slots, slot);
        else
          ref_group::rope_kv_bf16_kernel<16, 4>(qkv, row_stride, cosv, sinv, n_q_heads, n_kv_heads, h0, kc, vq, vs, slots, slot);
      });
    for (auto &t : pool)
      t.join();
    for (int w = 0; w < 4; w++)
      pthread_barrier_destroy(&ref_group::wave_barrier[w]);
  }
}
#else
REF_API int ref_has_rope_kv(void) { return 0; }
#endif

#ifdef REF_ROUTER_PART
REF_API int ref_has_router_wave(void) { return 1; }
// One 64-lane wave per row, TOPK_WAVES rows per block, as the engine launches it
// (engine/gpu_engine.hpp:524-527).  No block barrier in the kernel: a wave whose row is past the
// end leaves at once, the others only meet inside their own wave.
REF_API void ref_router_topk_wave(const float *logits, int E, int k, float *topk_w, int *topk_e, int B, const int *done,
                                  const int *slot_of) {
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  const int threads = 64 * TOPK_WAVES;
  ref_group::blockDim.x = threads;
  for (int block = 0; block < (B + TOPK_WAVES - 1) / TOPK_WAVES; block++) {
    for (int w = 0; w < TOPK_WAVES; w++)
      pthread_barrier_init(&ref_group::wave_barrier[w], nullptr, 64);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; t++)
      pool.emplace_back([=] {
        ref_group::threadIdx.x = t;
        ref_group::blockIdx.x = block;
        ref_group::router_topk_wave_kernel(logits, E, k, topk_w, topk_e, B, done, slot_of);
      });
    for (auto &t : pool)
      t.join();
    for (int w = 0; w < TOPK_WAVES; w++)
      pthread_barrier_destroy(&ref_group::wave_barrier[w]);
  }
}
#else
REF_API int ref_has_router_wave(void) { return 0; }
#endif

#ifdef REF_GROUP_EP_PART
REF_API int ref_has_group_ep(void) { return 1; }
// moe_count_ep_kernel then moe_place_ep_kernel (kernels/moe_ep.hpp:55-127), the pair that
// moe_group_ep launches for shapes its fused kernel does not take (:250-254), with no partner
// (n_peer = 0): e_count blocks of MOE_GROUP_THREADS threads each, one block at a time, a host
// thread per GPU thread, four 64-wide waves per block.
static void run_block_ep(int block, const std::function<void()> &kernel) {
  pthread_barrier_init(&ref_group::block_barrier, nullptr, MOE_GROUP_THREADS);
  for (int w = 0; w < MOE_GROUP_THREADS / 64; w++)
    pthread_barrier_init(&ref_group::wave_barrier[w], nullptr, 64);
  ref_group::blockDim.x = MOE_GROUP_THREADS;
  std::vector<std::thread> threads;
  for (int t = 0; t < MOE_GROUP_THREADS; t++)
    threads.emplace_back([=, &kernel] {
      ref_group::threadIdx.x = t;
      ref_group::blockIdx.x = block;
      kernel();
    });
  for (auto &t : threads)
    t.join();
  for (int w = 0; w < MOE_GROUP_THREADS / 64; w++)
    pthread_barrier_destroy(&ref_group::wave_barrier[w]);
  pthread_barrier_destroy(&ref_group::block_barrier);
}
REF_API void ref_moe_group_ep(const int *topk_own, int n_own, int e_begin, int e_count, int *counts, int *offsets,
                              int *row_pair, int *own_row) {
  static_assert(MOE_GROUP_THREADS % 64 == 0 && MOE_GROUP_THREADS / 64 <= 16, "waves per block");
  std::lock_guard<std::mutex> lock(ref_group::one_block_at_a_time);
  for (int e = 0; e < e_count; e++)
    run_block_ep(e, [=] { ref_group::moe_count_ep_kernel(topk_own, n_own, nullptr, 0, e_begin, counts); });
  for (int e = 0; e < e_count; e++)
    run_block_ep(e, [=] {
      ref_group::moe_place_ep_kernel(topk_own, n_own, nullptr, 0, n_own, e_begin, e_count, counts, offsets, row_pair,
                                     own_row, nullptr);
    });
}
#else
REF_API int ref_has_group_ep(void) { return 0; }
#endif
#else
REF_API int ref_has_group(void) { return 0; }
REF_API int ref_has_group_ep(void) { return 0; }
REF_API int ref_has_exact_kernels(void) { return 0; }
REF_API int ref_has_router_wave(void) { return 0; }
REF_API int ref_has_rope_kv(void) { return 0; }
REF_API int ref_has_argmax_key(void) { return 0; }
REF_API int ref_has_fast_kernels(void) { return 0; }
REF_API int ref_has_exact_rows(void) { return 0; }
REF_API int ref_has_fused_kernels(void) { return 0; }
#endif
