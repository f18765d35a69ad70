// The layer-chain driver (include/gptoss_engine.h): owns the device buffers of
// one GPU and issues the fused kernels in the order of the reference engine's
// decode step (step_embed, layer_attention, layer_route, layer_experts,
// layer_combine, step_logits: getp-csrc/engine/gpu_engine.hpp:461-621), with a
// caller-filled stand-in tensor wherever that engine runs a GEMM or attention.
#include <string.h>

#include <map>
#include <new>
#include <vector>

#include "../../include/gptoss_engine.h"
#include "common.cuh"

namespace gptoss {
int cuda_status(cudaError_t e);
}
using namespace gptoss;

struct gptoss_chain {
  gptoss_chain_config_t cfg;
  int max_tokens = 0, n_sets = 0, device = 0;
  cudaStream_t stream = nullptr;
  size_t total_bytes = 0;
  std::vector<void *> allocs;
  // weights
  void *embedding = nullptr;
  float *gain_attn = nullptr, *gain_ffn = nullptr, *gain_out = nullptr, *qkv_bias = nullptr;
  float *cos_tab = nullptr, *sin_tab = nullptr;
  // stand-ins, n_sets of each (logits: one)
  void *attn_proj = nullptr, *qkv = nullptr, *router = nullptr, *mlp1 = nullptr, *expert = nullptr,
       *logits = nullptr;
  // state
  int *tokens = nullptr, *pos = nullptr, *next = nullptr, *topk_e = nullptr, *own_row = nullptr, *row_done = nullptr;
  float *x = nullptr, *topk_w = nullptr;
  void *normed = nullptr, *qkv_out = nullptr, *swiglu = nullptr;
  // second copies of the three write-only activations, made when the per-kind profile first
  // runs: a kind's launches replayed back to back then alternate between two output buffers,
  // so that a launch does not find its output lines still dirty in L2 from the one before
  // (in the whole step ~600 MB of other kernels' traffic passes between them)
  void *normed_alt = nullptr, *qkv_out_alt = nullptr, *swiglu_alt = nullptr;
  bool alternate_outputs = false; // only while a per-kind profiling graph is being captured
  unsigned long long *keys = nullptr;
  void *flush = nullptr;
  size_t flush_bytes = 0;
  std::map<int, cudaGraphExec_t> graphs;                       // whole step, per T
  std::map<int, cudaGraphExec_t> io_graphs;                    // the step between its host<->device copies, per T
  // the wave loop kept on the device (gptoss_chain_run_wave_on_device)
  std::map<int, cudaGraphExec_t> wave_graphs; // one step followed by the bookkeeping kernel, per T
  int *wave_prompts = nullptr, *wave_offsets = nullptr, *wave_generated = nullptr;
  size_t wave_prompts_cap = 0, wave_generated_cap = 0; // in ints
  struct WaveState *wave_state = nullptr;              // device
  struct WaveState *wave_state_host = nullptr;         // pinned
  int *io_host = nullptr; // pinned staging of gptoss_chain_step: tokens | positions | picked tokens, max_tokens each
  std::map<std::pair<int, int>, cudaGraphExec_t> kind_graphs; // one kernel kind's launches, per (T, kind)
  std::vector<cudaEvent_t> events;

  size_t act() const { return cfg.act_dtype == GPTOSS_F32 ? 4 : 2; }
  int qkv_dim() const { return (cfg.n_q_heads + 2 * cfg.n_kv_heads) * cfg.head_dim; }
};

// Counters of a wave served without the host in the loop.
struct WaveState {
  int active;          // rows not finished
  int steps_run;       // positions completed while any row was active
  int width;           // row pitch of `generated` (steps + 2)
  unsigned arrived;    // blocks of the running bookkeeping launch that are through; 0 between launches
  long long generated; // the reference's count over the rows that finished on an end token
  const int *prompts;  // device: the wave's prompts back to back
  int *out_rows;       // device: [n, width] generated tokens
  // (the two buffers are named here, not in the kernel's arguments, so that a captured
  // graph stays valid when a later wave needs larger ones)
  int finished_now;    // rows that finished in the running launch, until its last block takes them off `active`
  int pad;
};

namespace {

constexpr int kWaveThreads = 256;

// The per-step bookkeeping of gpu_run_wave (gpu_engine.hpp:800-826) as a kernel that
// runs behind the step's argmax: the row takes its next prompt token while it has one
// and the picked token afterwards, records generated tokens, and finishes on an end
// token.  One thread per row, so the four dependent reads of a row (position, offsets,
// token, output slot) are paid once for the batch and not once per 1024 rows.  "Was
// anybody still active when this step began" must be the same answer in every block:
// `active` is only written by the launch's last block (the one that finds every other
// block through), after all of them have read it.  Once nobody is active the kernel
// leaves everything as it is, and the steps the host had already queued change nothing.
__global__ void __launch_bounds__(kWaveThreads)
    wave_advance(int n, const int *__restrict__ offsets, const int *__restrict__ next,
                 int *__restrict__ tokens, int *__restrict__ pos, int *__restrict__ done, WaveState *state) {
  pdl_prologue();
  __shared__ int s_active, s_finished, s_width;
  __shared__ long long s_count;
  __shared__ const int *s_prompts;
  __shared__ int *s_out_rows;
  if (threadIdx.x == 0) {
    s_active = *reinterpret_cast<volatile int *>(&state->active);
    s_width = state->width;
    s_prompts = state->prompts;
    s_out_rows = state->out_rows;
    s_finished = 0;
    s_count = 0;
  }
  __syncthreads();
  const int b = blockIdx.x * kWaveThreads + threadIdx.x;
  if (s_active > 0 && b < n) {
    const int p = pos[b] + 1; // every row sits at the same position
    pos[b] = p;
    if (!done[b]) {
      const int first = offsets[b], np = offsets[b + 1] - first;
      int *out = s_out_rows + (size_t)b * s_width;
      int token;
      if (p < np) {
        token = s_prompts[first + p];
      } else {
        token = next[b];
        out[p - np] = token;
      }
      if (token == 199999 || token == 200002) {
        done[b] = 1;
        if (p - np + 1 >= 0)
          out[p - np + 1] = -1;
        atomicAdd(&s_finished, 1);
        atomicAdd(reinterpret_cast<unsigned long long *>(&s_count), (unsigned long long)(long long)(p - np + 1));
      }
      tokens[b] = token;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_finished)
      atomicAdd(&state->finished_now, s_finished);
    if (s_count)
      atomicAdd(reinterpret_cast<unsigned long long *>(&state->generated), (unsigned long long)s_count);
    __threadfence();
    if (atomicAdd(&state->arrived, 1u) == gridDim.x - 1) { // every other block is through
      __threadfence();
      if (s_active > 0) {
        state->active = s_active - atomicExch(&state->finished_now, 0);
        state->steps_run += 1;
      }
      state->arrived = 0u;
    }
  }
}

template <typename P> int dev_alloc(gptoss_chain *c, P **p, size_t bytes) {
  void *q = nullptr;
  const int st = cuda_status(cudaMalloc(&q, bytes ? bytes : 16));
  if (st != GPTOSS_OK)
    return st;
  c->allocs.push_back(q);
  bounds_register(q, bytes ? bytes : 16);
  c->total_bytes += bytes;
  *p = static_cast<P *>(q);
  return GPTOSS_OK;
}

struct BufInfo {
  void *base;
  size_t bytes_per_layer; // size of one layer's (or the only) instance
  int layered;            // 0: single, 1: per model layer, 2: per stand-in set
};

BufInfo buf_info(const gptoss_chain *c, gptoss_chain_buffer_t which) {
  const gptoss_chain_config_t &g = c->cfg;
  const size_t T = (size_t)c->max_tokens, H = (size_t)g.hidden, a = c->act(), K = (size_t)g.top_k;
  const size_t half = (size_t)g.head_dim / 2;
  switch (which) {
  case GPTOSS_BUF_EMBEDDING: return {c->embedding, (size_t)g.vocab * H * a, 0};
  case GPTOSS_BUF_GAIN_ATTN: return {c->gain_attn, H * 4, 1};
  case GPTOSS_BUF_GAIN_FFN: return {c->gain_ffn, H * 4, 1};
  case GPTOSS_BUF_GAIN_OUT: return {c->gain_out, H * 4, 0};
  case GPTOSS_BUF_QKV_BIAS: return {c->qkv_bias, (size_t)c->qkv_dim() * 4, 1};
  case GPTOSS_BUF_COS: return {c->cos_tab, (size_t)g.max_pos * half * 4, 0};
  case GPTOSS_BUF_SIN: return {c->sin_tab, (size_t)g.max_pos * half * 4, 0};
  case GPTOSS_BUF_ATTN_PROJ: return {c->attn_proj, T * H * a, 2};
  case GPTOSS_BUF_QKV: return {c->qkv, T * (size_t)c->qkv_dim() * a, 2};
  case GPTOSS_BUF_ROUTER: return {c->router, T * (size_t)g.n_experts * a, 2};
  case GPTOSS_BUF_MLP1: return {c->mlp1, K * T * 2 * (size_t)g.inter * a, 2};
  case GPTOSS_BUF_EXPERT: return {c->expert, K * T * H * a, 2};
  case GPTOSS_BUF_LOGITS: return {c->logits, T * (size_t)g.vocab * a, 0};
  case GPTOSS_BUF_TOKENS: return {c->tokens, T * 4, 0};
  case GPTOSS_BUF_POS: return {c->pos, T * 4, 0};
  case GPTOSS_BUF_X: return {c->x, T * H * 4, 0};
  case GPTOSS_BUF_NORMED: return {c->normed, T * H * a, 0};
  case GPTOSS_BUF_QKV_OUT: return {c->qkv_out, T * (size_t)c->qkv_dim() * a, 0};
  case GPTOSS_BUF_TOPK_W: return {c->topk_w, T * K * 4, 0};
  case GPTOSS_BUF_TOPK_E: return {c->topk_e, T * K * 4, 0};
  case GPTOSS_BUF_SWIGLU: return {c->swiglu, K * T * (size_t)g.inter * a, 0};
  case GPTOSS_BUF_NEXT: return {c->next, T * 4, 0};
  case GPTOSS_BUF_ROW_DONE: return {c->row_done, T * 4, 0};
  default: return {nullptr, 0, 0};
  }
}

char *layer_ptr(const gptoss_chain *c, gptoss_chain_buffer_t which, int layer) {
  const BufInfo b = buf_info(c, which);
  size_t idx = 0;
  if (b.layered == 1)
    idx = (size_t)layer;
  else if (b.layered == 2)
    idx = (size_t)(layer % c->n_sets);
  return static_cast<char *>(b.base) + idx * b.bytes_per_layer;
}

// Called around every launch of a step; used by the profiler.
struct Hook {
  virtual void before(gptoss_chain_kernel_t) {}
  virtual void after(gptoss_chain_kernel_t) {}
  virtual ~Hook() {}
};

#define STEP(kind, call)                                                                          \
  do {                                                                                            \
    if (only >= 0 && only != (int)(kind))                                                         \
      break;                                                                                      \
    if (hook)                                                                                     \
      hook->before(kind);                                                                         \
    const int st_ = (call);                                                                       \
    if (hook)                                                                                     \
      hook->after(kind);                                                                          \
    if (st_ != GPTOSS_OK)                                                                         \
      return st_;                                                                                 \
  } while (0)

// Issues every kernel of one step for T rows on s; with only >= 0, just the
// launches of that kernel kind (all layers, in layer order).
int issue_step(gptoss_chain *c, int T, cudaStream_t s, Hook *hook, int only = -1) {
  const gptoss_chain_config_t &g = c->cfg;
  const gptoss_dtype_t a = (gptoss_dtype_t)g.act_dtype;
  const int H = g.hidden, L = g.n_layers, K = g.top_k, QKV = c->qkv_dim();
  gptoss_stream_t gs = s;
  if (g.flags & GPTOSS_CHAIN_SPLIT_EMBED_NORM) {
    // step_embed: x = embedding[tokens]
    STEP(GPTOSS_K_EMBED, gptoss_embed(gs, T, c->embedding, a, g.vocab, c->tokens, c->x, GPTOSS_F32, H, g.flags));
    // layer 0's attention norm; later layers get theirs from the previous combine
    STEP(GPTOSS_K_NORM, gptoss_add_rmsnorm(gs, T, c->x, nullptr, a, c->gain_attn, c->normed, a, H, g.flags));
  } else {
    // both in one launch
    STEP(GPTOSS_K_EMBED, gptoss_embed_rmsnorm(gs, T, c->embedding, a, g.vocab, c->tokens, c->x, c->gain_attn,
                                              c->normed, a, H, g.flags));
  }
  for (int l = 0; l < L; l++) {
    const bool alt = c->alternate_outputs && (l & 1);
    void *normed_l = alt ? c->normed_alt : c->normed, *qkv_out_l = alt ? c->qkv_out_alt : c->qkv_out;
    void *swiglu_l = alt ? c->swiglu_alt : c->swiglu;
    // [QKV GEMM of `normed`] -> stand-in qkv; bias + RoPE
    STEP(GPTOSS_K_ROPE,
         gptoss_qkv_bias_rope(gs, T, layer_ptr(c, GPTOSS_BUF_QKV, l), a, QKV,
                              (const float *)layer_ptr(c, GPTOSS_BUF_QKV_BIAS, l), c->pos, 0,
                              c->cos_tab, c->sin_tab, g.max_pos, g.n_q_heads, g.n_kv_heads,
                              g.head_dim, qkv_out_l, a, QKV, g.flags));
    // [attention + output GEMM] -> stand-in projection; residual add + MoE norm
    STEP(GPTOSS_K_ADD_NORM,
         gptoss_add_rmsnorm(gs, T, c->x, layer_ptr(c, GPTOSS_BUF_ATTN_PROJ, l), a,
                            (const float *)layer_ptr(c, GPTOSS_BUF_GAIN_FFN, l), normed_l, a, H,
                            g.flags));
    // [router GEMM] -> stand-in logits; top-k + softmax
    STEP(GPTOSS_K_ROUTER, gptoss_router_topk(gs, T, layer_ptr(c, GPTOSS_BUF_ROUTER, l), a,
                                             g.n_experts, K, c->topk_w, c->topk_e, c->row_done, nullptr, g.flags));
    // [mlp1 GEMM] -> stand-in gate/up rows; SwiGLU
    STEP(GPTOSS_K_SWIGLU, gptoss_swiglu(gs, layer_ptr(c, GPTOSS_BUF_MLP1, l), a, swiglu_l, a,
                                        (size_t)K * T, g.inter, g.swiglu_limit, g.flags));
    // [mlp2 GEMM] -> stand-in expert rows; combine + residual + next norm
    const float *next_gain = l + 1 < L ? (const float *)layer_ptr(c, GPTOSS_BUF_GAIN_ATTN, l + 1)
                                       : c->gain_out;
    STEP(GPTOSS_K_COMBINE,
         gptoss_moe_combine(gs, T, c->x, layer_ptr(c, GPTOSS_BUF_EXPERT, l), a, c->own_row, c->topk_w,
                            c->topk_e, K, H, nullptr, next_gain, normed_l, a, g.flags));
  }
  // [LM-head GEMM of `normed`] -> stand-in logits; greedy pick
  STEP(GPTOSS_K_ARGMAX, gptoss_argmax(gs, T, c->logits, a, g.vocab, g.vocab, c->keys, c->next, g.flags));
  return GPTOSS_OK;
}

struct ProfileHook : Hook {
  gptoss_chain *c;
  cudaStream_t s;
  bool flush;
  size_t n = 0;
  std::vector<gptoss_chain_kernel_t> kinds;
  ProfileHook(gptoss_chain *c_, cudaStream_t s_, bool f) : c(c_), s(s_), flush(f) {}
  cudaEvent_t event(size_t i) {
    while (c->events.size() <= i) {
      cudaEvent_t e = nullptr;
      cudaEventCreate(&e);
      c->events.push_back(e);
    }
    return c->events[i];
  }
  void before(gptoss_chain_kernel_t k) override {
    if (flush)
      gptoss_flush_l2(c->flush, c->flush_bytes, s);
    kinds.push_back(k);
    cudaEventRecord(event(2 * n), s);
  }
  void after(gptoss_chain_kernel_t) override {
    cudaEventRecord(event(2 * n + 1), s);
    n++;
  }
};

} // namespace

extern "C" {

int gptoss_chain_config_gpt_oss(int which, gptoss_dtype_t act_dtype, int max_pos,
                                gptoss_chain_config_t *cfg) {
  if (!cfg || (which != 20 && which != 120) || !valid_dtype(act_dtype) || max_pos <= 0)
    return GPTOSS_ERR_BAD_ARG;
  memset(cfg, 0, sizeof *cfg);
  cfg->vocab = 201088;
  cfg->hidden = 2880;
  cfg->n_experts = which == 20 ? 32 : 128;
  cfg->top_k = 4;
  cfg->inter = 2880;
  cfg->n_layers = which == 20 ? 24 : 36;
  cfg->head_dim = 64;
  cfg->n_q_heads = 64;
  cfg->n_kv_heads = 8;
  cfg->max_pos = max_pos;
  cfg->orig_ctx = 4096.0f;
  cfg->theta = 150000.0f;
  cfg->factor = 32.0f;
  cfg->beta_fast = 32.0f;
  cfg->beta_slow = 1.0f;
  cfg->swiglu_limit = 7.0f;
  cfg->act_dtype = act_dtype;
  // Programmatic launch between the chain's kernels is on: every kernel waits for its predecessor
  // before it reads anything, so results do not change, and a step of 123 launches measured
  // 2 % shorter at 4096 tokens and 11 % shorter at 512.
  cfg->flags = (act_dtype == GPTOSS_F32 ? (unsigned)GPTOSS_EXACT : 0u) | (unsigned)GPTOSS_PDL;
  return GPTOSS_OK;
}

int gptoss_chain_create(const gptoss_chain_config_t *cfg, int max_tokens, int n_standin_layers,
                        gptoss_chain_t **out) {
  if (!cfg || !out || max_tokens <= 0 || cfg->n_layers <= 0 || n_standin_layers <= 0 ||
      n_standin_layers > cfg->n_layers || cfg->hidden <= 0 || cfg->vocab <= 0 || cfg->inter <= 0 ||
      cfg->top_k <= 0 || cfg->top_k > GPTOSS_MAX_TOPK || cfg->n_experts < cfg->top_k ||
      cfg->n_experts > GPTOSS_MAX_EXPERTS || cfg->head_dim <= 0 || cfg->head_dim % 2 != 0 ||
      cfg->max_pos <= 0 || !valid_dtype((gptoss_dtype_t)cfg->act_dtype))
    return GPTOSS_ERR_BAD_ARG;
  *out = nullptr;
  gptoss_chain *c = new (std::nothrow) gptoss_chain;
  if (!c)
    return GPTOSS_ERR_BAD_ARG;
  c->cfg = *cfg;
  c->max_tokens = max_tokens;
  c->n_sets = n_standin_layers;
  int st = cuda_status(cudaGetDevice(&c->device));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  const size_t T = (size_t)max_tokens, H = (size_t)cfg->hidden, a = c->act(), K = (size_t)cfg->top_k;
  const size_t L = (size_t)cfg->n_layers, S = (size_t)c->n_sets, QKV = (size_t)c->qkv_dim();
  const size_t half = (size_t)cfg->head_dim / 2;
#define ALLOC(field, bytes)                                                                       \
  if (st == GPTOSS_OK)                                                                            \
  st = dev_alloc(c, &c->field, (bytes))
  ALLOC(embedding, (size_t)cfg->vocab * H * a);
  ALLOC(gain_attn, L * H * 4);
  ALLOC(gain_ffn, L * H * 4);
  ALLOC(gain_out, H * 4);
  ALLOC(qkv_bias, L * QKV * 4);
  ALLOC(cos_tab, (size_t)cfg->max_pos * half * 4);
  ALLOC(sin_tab, (size_t)cfg->max_pos * half * 4);
  ALLOC(attn_proj, S * T * H * a);
  ALLOC(qkv, S * T * QKV * a);
  ALLOC(router, S * T * (size_t)cfg->n_experts * a);
  ALLOC(mlp1, S * K * T * 2 * (size_t)cfg->inter * a);
  ALLOC(expert, S * K * T * H * a);
  ALLOC(logits, T * (size_t)cfg->vocab * a);
  ALLOC(tokens, T * 4);
  ALLOC(pos, T * 4);
  ALLOC(next, T * 4);
  ALLOC(x, T * H * 4);
  ALLOC(normed, T * H * a);
  ALLOC(qkv_out, T * QKV * a);
  ALLOC(topk_w, T * K * 4);
  ALLOC(topk_e, T * K * 4);
  ALLOC(swiglu, K * T * (size_t)cfg->inter * a);
  ALLOC(keys, T * 8);
  ALLOC(own_row, T * K * 4);
  ALLOC(row_done, T * 4);
  c->flush_bytes = (size_t)256 << 20;
  ALLOC(flush, c->flush_bytes);
#undef ALLOC
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMallocHost(reinterpret_cast<void **>(&c->io_host), 3 * T * 4));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->keys, 0, T * 8, c->stream));
  if (st == GPTOSS_OK) {
    // The engine's grouping step decides where each (token, choice) pair's expert output
    // lands; with the stand-in tensors that map is the identity, passed explicitly so the
    // combine goes through the indirection exactly as it does behind a real grouping.
    std::vector<int> ident(T * K);
    for (size_t i = 0; i < ident.size(); i++)
      ident[i] = (int)i;
    st = cuda_status(cudaMemcpy(c->own_row, ident.data(), ident.size() * 4, cudaMemcpyHostToDevice));
  }
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->row_done, 0, T * 4, c->stream));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->tokens, 0, T * 4, c->stream));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->pos, 0, T * 4, c->stream));
  if (st == GPTOSS_OK) {
    std::vector<float> cs((size_t)cfg->max_pos * half), sn((size_t)cfg->max_pos * half);
    st = gptoss_build_rope_tables(cfg->max_pos, cfg->head_dim, cfg->theta, cfg->factor,
                                  cfg->orig_ctx, cfg->beta_fast, cfg->beta_slow, cs.data(),
                                  sn.data());
    if (st == GPTOSS_OK)
      st = cuda_status(cudaMemcpy(c->cos_tab, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
    if (st == GPTOSS_OK)
      st = cuda_status(cudaMemcpy(c->sin_tab, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
  }
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(c->stream));
  if (st != GPTOSS_OK) {
    gptoss_chain_destroy(c);
    return st;
  }
  *out = c;
  return GPTOSS_OK;
}

int gptoss_chain_destroy(gptoss_chain_t *c) {
  if (!c)
    return GPTOSS_OK;
  if (c->stream)
    (void)cudaStreamSynchronize(c->stream);
  for (auto &kv : c->graphs)
    (void)cudaGraphExecDestroy(kv.second);
  for (auto &kv : c->kind_graphs)
    (void)cudaGraphExecDestroy(kv.second);
  for (auto &kv : c->io_graphs)
    (void)cudaGraphExecDestroy(kv.second);
  for (auto &kv : c->wave_graphs)
    (void)cudaGraphExecDestroy(kv.second);
  if (c->wave_state_host)
    (void)cudaFreeHost(c->wave_state_host);
  // wave_prompts / wave_generated are not in `allocs`: they are replaced when a wave needs more room
  bounds_unregister(c->wave_prompts);
  bounds_unregister(c->wave_generated);
  if (c->wave_prompts)
    (void)cudaFree(c->wave_prompts);
  if (c->wave_generated)
    (void)cudaFree(c->wave_generated);
  if (c->io_host)
    (void)cudaFreeHost(c->io_host);
  for (cudaEvent_t e : c->events)
    (void)cudaEventDestroy(e);
  for (void *p : c->allocs) {
    bounds_unregister(p);
    (void)cudaFree(p);
  }
  if (c->stream)
    (void)cudaStreamDestroy(c->stream);
  delete c;
  return GPTOSS_OK;
}

size_t gptoss_chain_device_bytes(const gptoss_chain_t *c) { return c ? c->total_bytes : 0; }

gptoss_stream_t gptoss_chain_stream(const gptoss_chain_t *c) { return c ? c->stream : nullptr; }

int gptoss_chain_buffer(const gptoss_chain_t *c, gptoss_chain_buffer_t which, int layer,
                        void **device_ptr, size_t *bytes) {
  if (!c || which < 0 || which >= GPTOSS_BUF_COUNT || layer < 0 || layer >= c->cfg.n_layers)
    return GPTOSS_ERR_BAD_ARG;
  const BufInfo b = buf_info(c, which);
  if (device_ptr)
    *device_ptr = layer_ptr(c, which, layer);
  if (bytes)
    *bytes = b.bytes_per_layer;
  return GPTOSS_OK;
}

int gptoss_chain_fill_synthetic(gptoss_chain_t *c, int T, uint64_t seed, int threads) {
  if (!c || T <= 0 || T > c->max_tokens)
    return GPTOSS_ERR_BAD_ARG;
  const gptoss_chain_config_t &g = c->cfg;
  const gptoss_dtype_t a = (gptoss_dtype_t)g.act_dtype;
  const size_t H = (size_t)g.hidden, K = (size_t)g.top_k, QKV = (size_t)c->qkv_dim(), el = c->act();
  // One host staging buffer, reused for every tensor, cut into pieces so the
  // host generates piece i+1 while piece i is on its way to the device.
  const size_t piece_elems = (size_t)32 << 20;
  void *stage[2] = {nullptr, nullptr};
  int st = cuda_status(cudaMallocHost(&stage[0], piece_elems * 4));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMallocHost(&stage[1], piece_elems * 4));
  cudaEvent_t done[2] = {nullptr, nullptr};
  if (st == GPTOSS_OK)
    st = cuda_status(cudaEventCreate(&done[0]));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaEventCreate(&done[1]));
  int turn = 0;
  uint64_t stream_id = 0;
  // Rows of a stand-in are generated for T rows although the buffer holds
  // max_tokens: the chain indexes rows, so a prefix is all a T-row step reads.
  auto fill = [&](void *dev, gptoss_dtype_t dt, size_t count, float mean, float sd) {
    const size_t esz = dt == GPTOSS_F32 ? 4 : 2;
    const uint64_t sid = stream_id++;
    for (size_t off = 0; off < count && st == GPTOSS_OK; off += piece_elems) {
      const size_t n = count - off < piece_elems ? count - off : piece_elems;
      st = cuda_status(cudaEventSynchronize(done[turn]));
      if (st != GPTOSS_OK)
        break;
      // a piece is its own sub-stream so pieces are independent of piece size
      st = gptoss_synth_normal(stage[turn], dt, n, seed, sid * 4096 + off / piece_elems, mean, sd,
                               threads);
      if (st != GPTOSS_OK)
        break;
      st = cuda_status(cudaMemcpyAsync((char *)dev + off * esz, stage[turn], n * esz,
                                       cudaMemcpyHostToDevice, c->stream));
      if (st == GPTOSS_OK)
        st = cuda_status(cudaEventRecord(done[turn], c->stream));
      turn ^= 1;
    }
  };
  if (st == GPTOSS_OK) {
    fill(c->embedding, a, (size_t)g.vocab * H, 0.0f, 0.02f);
    fill(c->gain_attn, GPTOSS_F32, (size_t)g.n_layers * H, 1.0f, 0.1f);
    fill(c->gain_ffn, GPTOSS_F32, (size_t)g.n_layers * H, 1.0f, 0.1f);
    fill(c->gain_out, GPTOSS_F32, H, 1.0f, 0.1f);
    fill(c->qkv_bias, GPTOSS_F32, (size_t)g.n_layers * QKV, 0.0f, 0.02f);
    for (int l = 0; l < c->n_sets; l++) {
      fill(layer_ptr(c, GPTOSS_BUF_ATTN_PROJ, l), a, (size_t)T * H, 0.0f, 1.0f);
      fill(layer_ptr(c, GPTOSS_BUF_QKV, l), a, (size_t)T * QKV, 0.0f, 1.0f);
      fill(layer_ptr(c, GPTOSS_BUF_ROUTER, l), a, (size_t)T * g.n_experts, 0.0f, 1.0f);
      fill(layer_ptr(c, GPTOSS_BUF_MLP1, l), a, K * T * 2 * (size_t)g.inter, 0.0f, 2.0f);
      fill(layer_ptr(c, GPTOSS_BUF_EXPERT, l), a, K * T * H, 0.0f, 1.0f);
    }
    fill(c->logits, a, (size_t)T * g.vocab, 0.0f, 3.0f);
  }
  (void)el;
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(c->stream));
  if (done[0])
    (void)cudaEventDestroy(done[0]);
  if (done[1])
    (void)cudaEventDestroy(done[1]);
  if (stage[0])
    (void)cudaFreeHost(stage[0]);
  if (stage[1])
    (void)cudaFreeHost(stage[1]);
  return st;
}

// Captures the launches of one step (only < 0) or of one kernel kind into a graph; with
// lead_flush an L2 flush goes first (only == GPTOSS_K_COUNT then gives the flush alone).
static int capture_step(gptoss_chain *c, int T, int only, cudaGraphExec_t *exec_out, bool lead_flush = false,
                        bool with_io = false, bool with_wave_advance = false) {
  // Warm every kernel once outside capture (occupancy queries, lazy module load).
  int st = lead_flush ? gptoss_flush_l2(c->flush, c->flush_bytes, c->stream) : GPTOSS_OK;
  if (st == GPTOSS_OK)
    st = issue_step(c, T, c->stream, nullptr, only);
  if (st != GPTOSS_OK)
    return st;
  st = cuda_status(cudaStreamSynchronize(c->stream));
  if (st != GPTOSS_OK)
    return st;
  st = cuda_status(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  if (st != GPTOSS_OK)
    return st;
  int issued = lead_flush ? gptoss_flush_l2(c->flush, c->flush_bytes, c->stream) : GPTOSS_OK;
  const size_t io_bytes = (size_t)T * 4, io_stride = (size_t)c->max_tokens;
  if (with_io && issued == GPTOSS_OK)
    issued = cuda_status(cudaMemcpyAsync(c->tokens, c->io_host, io_bytes, cudaMemcpyHostToDevice, c->stream));
  if (with_io && issued == GPTOSS_OK)
    issued = cuda_status(cudaMemcpyAsync(c->pos, c->io_host + io_stride, io_bytes, cudaMemcpyHostToDevice, c->stream));
  if (issued == GPTOSS_OK)
    issued = issue_step(c, T, c->stream, nullptr, only);
  if (with_io && issued == GPTOSS_OK)
    issued = cuda_status(cudaMemcpyAsync(c->io_host + 2 * io_stride, c->next, io_bytes, cudaMemcpyDeviceToHost, c->stream));
  if (with_wave_advance && issued == GPTOSS_OK) {
    const PdlScope pdl(c->cfg.flags);
    launch_kernel(wave_advance, dim3((T + kWaveThreads - 1) / kWaveThreads), dim3(kWaveThreads), 0, c->stream, T,
                  static_cast<const int *>(c->wave_offsets), static_cast<const int *>(c->next), c->tokens, c->pos,
                  c->row_done, c->wave_state);
    issued = launch_status();
  }
  cudaGraph_t graph = nullptr;
  st = cuda_status(cudaStreamEndCapture(c->stream, &graph));
  if (issued != GPTOSS_OK || st != GPTOSS_OK) {
    if (graph)
      (void)cudaGraphDestroy(graph);
    return issued != GPTOSS_OK ? issued : st;
  }
  st = cuda_status(cudaGraphInstantiate(exec_out, graph, 0));
  (void)cudaGraphDestroy(graph);
  return st;
}

int gptoss_chain_enqueue(gptoss_chain_t *c, int T, int use_graph) {
  if (!c || T < 0 || T > c->max_tokens)
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  if (!use_graph)
    return issue_step(c, T, c->stream, nullptr);
  auto it = c->graphs.find(T);
  if (it == c->graphs.end()) {
    cudaGraphExec_t exec = nullptr;
    const int st = capture_step(c, T, -1, &exec);
    if (st != GPTOSS_OK)
      return st;
    it = c->graphs.emplace(T, exec).first;
  }
  return cuda_status(cudaGraphLaunch(it->second, c->stream));
}

int gptoss_chain_step(gptoss_chain_t *c, int T, const int *tokens_host, const int *pos_host,
                      int *next_host) {
  if (!c || T < 0 || T > c->max_tokens || (T > 0 && (!tokens_host || !pos_host || !next_host)))
    return GPTOSS_ERR_BAD_ARG;
  if (T == 0)
    return GPTOSS_OK;
  // One graph launch per step: the two copies in, every kernel, the copy out.  The caller's
  // arrays pass through the chain's pinned staging block, whose addresses the graph holds.
  auto it = c->io_graphs.find(T);
  if (it == c->io_graphs.end()) {
    cudaGraphExec_t exec = nullptr;
    const int st = capture_step(c, T, -1, &exec, false, true);
    if (st != GPTOSS_OK)
      return st;
    it = c->io_graphs.emplace(T, exec).first;
  }
  const size_t stride = (size_t)c->max_tokens;
  memcpy(c->io_host, tokens_host, (size_t)T * 4);
  memcpy(c->io_host + stride, pos_host, (size_t)T * 4);
  int st = cuda_status(cudaGraphLaunch(it->second, c->stream));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(c->stream));
  if (st == GPTOSS_OK)
    memcpy(next_host, c->io_host + 2 * stride, (size_t)T * 4);
  return st;
}

int gptoss_chain_run_wave(gptoss_chain_t *c, const int *prompt_tokens, const int *prompt_offsets,
                          int n_requests, int steps, int *generated, long long *n_generated,
                          int *steps_run) {
  if (!c || n_requests < 0 || n_requests > c->max_tokens || steps < 0 || steps > c->cfg.max_pos)
    return GPTOSS_ERR_BAD_ARG;
  if (n_generated)
    *n_generated = 0;
  if (steps_run)
    *steps_run = 0;
  if (n_requests == 0)
    return GPTOSS_OK;
  if (!prompt_tokens || !prompt_offsets || !generated)
    return GPTOSS_ERR_BAD_ARG;
  const int n = n_requests, width = steps + 2;
  for (int b = 0; b < n; b++)
    if (prompt_offsets[b + 1] - prompt_offsets[b] < 1)
      return GPTOSS_ERR_BAD_ARG; // every request needs at least one prompt token
  const int eos_a = 199999, eos_b = 200002; // the two end tokens of the gpt-oss vocabulary
  std::vector<int> cur(n), next(n), done(n, 0), position(n, 0);
  for (int b = 0; b < n; b++)
    cur[b] = prompt_tokens[prompt_offsets[b]];
  for (size_t i = 0; i < (size_t)n * width; i++)
    generated[i] = -1;
  int st = cuda_status(cudaMemsetAsync(c->row_done, 0, (size_t)n * 4, c->stream));
  bool done_changed = false;
  long long total = 0;
  int active = n, pos = 0;
  while (st == GPTOSS_OK && pos < steps && active > 0) {
    // the host side of a step: tokens in (and the done mask when it changed), ids out
    if (done_changed) {
      st = cuda_status(cudaMemcpyAsync(c->row_done, done.data(), (size_t)n * 4, cudaMemcpyHostToDevice, c->stream));
      done_changed = false;
    }
    for (int b = 0; b < n; b++)
      position[b] = pos; // one position for the whole batch, as in the engine
    if (st == GPTOSS_OK)
      st = gptoss_chain_step(c, n, cur.data(), position.data(), next.data());
    if (st != GPTOSS_OK)
      break;
    pos++;
    for (int b = 0; b < n; b++) {
      if (done[b])
        continue;
      const int np = prompt_offsets[b + 1] - prompt_offsets[b];
      int *out = generated + (size_t)b * width;
      int token;
      if (pos < np) {
        token = prompt_tokens[prompt_offsets[b] + pos];
      } else {
        token = next[b];
        out[pos - np] = token;
      }
      if (token == eos_a || token == eos_b) {
        done[b] = 1;
        done_changed = true;
        active--;
        if (pos - np + 1 >= 0)
          out[pos - np + 1] = -1;
        total += pos - np + 1;
      }
      cur[b] = token;
    }
  }
  for (int b = 0; b < n && st == GPTOSS_OK; b++) {
    if (done[b])
      continue;
    const int np = prompt_offsets[b + 1] - prompt_offsets[b];
    if (pos - np + 1 >= 0)
      generated[(size_t)b * width + (pos - np + 1)] = -1;
    total += pos - np + 1;
  }
  if (st == GPTOSS_OK && done_changed) // leave the mask on the device as the wave ended
    st = cuda_status(cudaMemcpy(c->row_done, done.data(), (size_t)n * 4, cudaMemcpyHostToDevice));
  if (n_generated)
    *n_generated = total;
  if (steps_run)
    *steps_run = pos;
  return st;
}

// Room for a wave's prompts and output rows on the device.
static int wave_reserve(gptoss_chain *c, size_t prompt_ints, size_t generated_ints) {
  int st = GPTOSS_OK;
  if (!c->wave_state) {
    st = dev_alloc(c, &c->wave_offsets, ((size_t)c->max_tokens + 1) * 4);
    if (st == GPTOSS_OK)
      st = dev_alloc(c, &c->wave_state, sizeof(WaveState));
    if (st == GPTOSS_OK)
      st = cuda_status(cudaMallocHost(reinterpret_cast<void **>(&c->wave_state_host), 3 * sizeof(WaveState))); // [0] set-up and result, [1], [2] batch reports
    if (st == GPTOSS_OK)
      st = cuda_status(cudaMemsetAsync(c->wave_state, 0, sizeof(WaveState), c->stream));
    if (st == GPTOSS_OK) {
      // first launch of the bookkeeping kernel outside any capture; with no active row it returns at once
      wave_advance<<<1, kWaveThreads, 0, c->stream>>>(0, nullptr, nullptr, nullptr, nullptr, nullptr, c->wave_state);
      st = cuda_status(cudaGetLastError());
    }
    if (st == GPTOSS_OK)
      st = cuda_status(cudaStreamSynchronize(c->stream));
  }
  auto grow = [&](int **buf, size_t *cap, size_t want) {
    if (st != GPTOSS_OK || want <= *cap)
      return;
    (void)cudaStreamSynchronize(c->stream);
    bounds_unregister(*buf);
    if (*buf)
      (void)cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    void *q = nullptr;
    st = cuda_status(cudaMalloc(&q, want * 4));
    if (st == GPTOSS_OK)
      bounds_register(q, want * 4);
    if (st == GPTOSS_OK) {
      *buf = static_cast<int *>(q);
      *cap = want;
    }
  };
  grow(&c->wave_prompts, &c->wave_prompts_cap, prompt_ints ? prompt_ints : 1);
  grow(&c->wave_generated, &c->wave_generated_cap, generated_ints ? generated_ints : 1);
  return st;
}

int gptoss_chain_run_wave_on_device(gptoss_chain_t *c, const int *prompt_tokens, const int *prompt_offsets,
                                    int n_requests, int steps, int *generated, long long *n_generated,
                                    int *steps_run) {
  if (!c || n_requests < 0 || n_requests > c->max_tokens || steps < 0 || steps > c->cfg.max_pos)
    return GPTOSS_ERR_BAD_ARG;
  if (n_generated)
    *n_generated = 0;
  if (steps_run)
    *steps_run = 0;
  if (n_requests == 0)
    return GPTOSS_OK;
  if (!prompt_tokens || !prompt_offsets || !generated)
    return GPTOSS_ERR_BAD_ARG;
  const int n = n_requests, width = steps + 2;
  for (int b = 0; b < n; b++)
    if (prompt_offsets[b + 1] - prompt_offsets[b] < 1)
      return GPTOSS_ERR_BAD_ARG;
  const size_t n_prompt = (size_t)(prompt_offsets[n] - prompt_offsets[0]);
  int st = wave_reserve(c, n_prompt, (size_t)n * width);
  if (st != GPTOSS_OK)
    return st;

  // the wave's inputs and starting state go to the device once
  std::vector<int> first(n), offsets(n + 1);
  for (int b = 0; b <= n; b++)
    offsets[b] = prompt_offsets[b] - prompt_offsets[0];
  for (int b = 0; b < n; b++)
    first[b] = prompt_tokens[prompt_offsets[b]];
  cudaStream_t s = c->stream;
  st = cuda_status(cudaMemcpyAsync(c->wave_prompts, prompt_tokens + prompt_offsets[0], n_prompt * 4, cudaMemcpyHostToDevice, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemcpyAsync(c->wave_offsets, offsets.data(), ((size_t)n + 1) * 4, cudaMemcpyHostToDevice, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemcpyAsync(c->tokens, first.data(), (size_t)n * 4, cudaMemcpyHostToDevice, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->pos, 0, (size_t)n * 4, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->row_done, 0, (size_t)n * 4, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemsetAsync(c->wave_generated, 0xff, (size_t)n * width * 4, s)); // every entry -1
  WaveState *hs = c->wave_state_host;
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(s)); // the vectors above are pageable, and hs may still be in use
  if (st != GPTOSS_OK)
    return st;
  hs->active = n;
  hs->steps_run = 0;
  hs->width = width;
  hs->arrived = 0u;
  hs->finished_now = 0;
  hs->pad = 0;
  hs->generated = 0;
  hs->prompts = c->wave_prompts;
  hs->out_rows = c->wave_generated;
  st = cuda_status(cudaMemcpyAsync(c->wave_state, hs, sizeof(WaveState), cudaMemcpyHostToDevice, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(s));
  if (st != GPTOSS_OK)
    return st;

  auto it = c->wave_graphs.find(n);
  if (it == c->wave_graphs.end()) {
    cudaGraphExec_t exec = nullptr;
    st = capture_step(c, n, -1, &exec, false, false, true);
    if (st != GPTOSS_OK)
      return st;
    it = c->wave_graphs.emplace(n, exec).first;
  }
  // Steps are queued a batch at a time, and the next batch is queued before the host looks
  // at the counters the previous one left (copied to one of two pinned slots, each with
  // its event), so the GPU never waits for the host.  Once a batch reports every row done,
  // no more are queued; steps already queued past that point run with every row masked
  // and leave the bookkeeping alone.
  const int batch = 16;
  while (c->events.size() < 2 && st == GPTOSS_OK) {
    cudaEvent_t e = nullptr;
    st = cuda_status(cudaEventCreate(&e));
    if (st == GPTOSS_OK)
      c->events.push_back(e);
  }
  int queued = 0, batches = 0;
  auto queue_batch = [&]() {
    const int now = steps - queued < batch ? steps - queued : batch;
    for (int i = 0; i < now && st == GPTOSS_OK; i++)
      st = cuda_status(cudaGraphLaunch(it->second, s));
    queued += now;
    if (st == GPTOSS_OK)
      st = cuda_status(cudaMemcpyAsync(hs + 1 + (batches & 1), c->wave_state, sizeof(WaveState),
                                       cudaMemcpyDeviceToHost, s));
    if (st == GPTOSS_OK)
      st = cuda_status(cudaEventRecord(c->events[batches & 1], s));
    batches++;
  };
  if (steps > 0 && st == GPTOSS_OK)
    queue_batch();
  for (int seen = 0; seen < batches && st == GPTOSS_OK; seen++) {
    if (queued < steps)
      queue_batch(); // keeps the GPU busy while the host waits for the batch before it
    st = cuda_status(cudaEventSynchronize(c->events[seen & 1]));
    if (st == GPTOSS_OK && hs[1 + (seen & 1)].active <= 0)
      break;
  }
  std::vector<int> done(n);
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemcpyAsync(hs, c->wave_state, sizeof(WaveState), cudaMemcpyDeviceToHost, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemcpyAsync(generated, c->wave_generated, (size_t)n * width * 4, cudaMemcpyDeviceToHost, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaMemcpyAsync(done.data(), c->row_done, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
  if (st == GPTOSS_OK)
    st = cuda_status(cudaStreamSynchronize(s));
  if (st != GPTOSS_OK)
    return st;
  // rows still running when the wave ended are closed here, as after the reference's loop (:828-838)
  const int pos = hs->steps_run;
  long long total = hs->generated;
  for (int b = 0; b < n; b++) {
    if (done[b])
      continue;
    const int np = prompt_offsets[b + 1] - prompt_offsets[b];
    if (pos - np + 1 >= 0)
      generated[(size_t)b * width + (pos - np + 1)] = -1;
    total += pos - np + 1;
  }
  if (n_generated)
    *n_generated = total;
  if (steps_run)
    *steps_run = pos;
  return GPTOSS_OK;
}

int gptoss_chain_profile(gptoss_chain_t *c, int T, int steps, int mode, double *ms_per_kind,
                         long *launches_per_kind) {
  if (!c || T <= 0 || T > c->max_tokens || steps <= 0 || !ms_per_kind || !launches_per_kind ||
      mode < 0 || mode > 2)
    return GPTOSS_ERR_BAD_ARG;
  for (int k = 0; k < GPTOSS_K_COUNT; k++) {
    ms_per_kind[k] = 0.0;
    launches_per_kind[k] = 0;
  }
  if (mode == 2) {
    // One event pair around all of a kind's launches of a step, replayed from a graph
    // captured for that kind alone: launches sit as close together as they do in the
    // whole-step graph, and the cost of the two event records is spread over the batch.
    // A kind with a single launch per step has no batch to spread it over (the pair costs
    // about 4 us): it is timed behind an L2 flush in the same graph -- cold, as it is in the
    // chain, where the argmax before it has swept the cache -- and the time of the flush
    // alone, taken between the same kind of event pair in the same pass, is subtracted.
    const bool split = (c->cfg.flags & GPTOSS_CHAIN_SPLIT_EMBED_NORM) != 0;
    const int per_step[GPTOSS_K_COUNT] = {1, split ? 1 : 0, c->cfg.n_layers, c->cfg.n_layers, c->cfg.n_layers,
                                          c->cfg.n_layers, c->cfg.n_layers, 1};
    while (c->events.size() < 2) {
      cudaEvent_t e = nullptr;
      int st = cuda_status(cudaEventCreate(&e));
      if (st != GPTOSS_OK)
        return st;
      c->events.push_back(e);
    }
    if (!c->swiglu_alt) {
      const size_t Tm = (size_t)c->max_tokens, a = c->act();
      int st = dev_alloc(c, &c->normed_alt, Tm * (size_t)c->cfg.hidden * a);
      if (st == GPTOSS_OK)
        st = dev_alloc(c, &c->qkv_out_alt, Tm * (size_t)c->qkv_dim() * a);
      if (st == GPTOSS_OK)
        st = dev_alloc(c, &c->swiglu_alt, (size_t)c->cfg.top_k * Tm * (size_t)c->cfg.inter * a);
      if (st != GPTOSS_OK)
        return st;
    }
    for (int kind = 0; kind <= GPTOSS_K_COUNT; kind++) // GPTOSS_K_COUNT: the flush alone
      if (!c->kind_graphs.count({T, kind})) {
        cudaGraphExec_t exec = nullptr;
        c->alternate_outputs = true;
        const int st = capture_step(c, T, kind, &exec, kind == GPTOSS_K_COUNT || per_step[kind] == 1);
        c->alternate_outputs = false;
        if (st != GPTOSS_OK)
          return st;
        c->kind_graphs[{T, kind}] = exec;
      }
    for (int s = 0; s < steps; s++) {
      double flush_ms = 0.0;
      for (int kind = GPTOSS_K_COUNT; kind >= 0; kind--) { // the flush alone first
        if (kind < GPTOSS_K_COUNT && per_step[kind] == 0)
          continue;
        int st = cuda_status(cudaEventRecord(c->events[0], c->stream));
        if (st == GPTOSS_OK)
          st = cuda_status(cudaGraphLaunch(c->kind_graphs[{T, kind}], c->stream));
        if (st == GPTOSS_OK)
          st = cuda_status(cudaEventRecord(c->events[1], c->stream));
        if (st == GPTOSS_OK)
          st = cuda_status(cudaStreamSynchronize(c->stream));
        float ms = 0.0f;
        if (st == GPTOSS_OK)
          st = cuda_status(cudaEventElapsedTime(&ms, c->events[0], c->events[1]));
        if (st != GPTOSS_OK)
          return st;
        if (kind == GPTOSS_K_COUNT) {
          flush_ms = ms;
          continue;
        }
        ms_per_kind[kind] += per_step[kind] == 1 ? (ms > flush_ms ? ms - flush_ms : 0.0) : ms;
        launches_per_kind[kind] += per_step[kind];
      }
    }
    return GPTOSS_OK;
  }
  for (int s = 0; s < steps; s++) {
    ProfileHook hook(c, c->stream, mode == 1);
    int st = issue_step(c, T, c->stream, &hook);
    if (st != GPTOSS_OK)
      return st;
    st = cuda_status(cudaStreamSynchronize(c->stream));
    if (st != GPTOSS_OK)
      return st;
    for (size_t i = 0; i < hook.n; i++) {
      float ms = 0.0f;
      st = cuda_status(cudaEventElapsedTime(&ms, c->events[2 * i], c->events[2 * i + 1]));
      if (st != GPTOSS_OK)
        return st;
      ms_per_kind[hook.kinds[i]] += ms;
      launches_per_kind[hook.kinds[i]]++;
    }
  }
  return GPTOSS_OK;
}

size_t gptoss_chain_kernel_bytes(const gptoss_chain_t *c, gptoss_chain_kernel_t kind, int T) {
  if (!c || T <= 0)
    return 0;
  const gptoss_chain_config_t &g = c->cfg;
  const size_t t = (size_t)T, H = (size_t)g.hidden, a = c->act(), K = (size_t)g.top_k;
  const size_t QKV = (size_t)c->qkv_dim();
  switch (kind) {
  case GPTOSS_K_EMBED: // id + table row in + fp32 row out (+ normed out, gain once, when fused)
    return (g.flags & GPTOSS_CHAIN_SPLIT_EMBED_NORM) ? t * (4 + H * a + H * 4)
                                                     : t * (4 + H * a + H * 4 + H * a) + H * 4;
  case GPTOSS_K_NORM: // x in, normed out, gain once
    return (g.flags & GPTOSS_CHAIN_SPLIT_EMBED_NORM) ? t * (H * 4 + H * a) + H * 4 : 0;
  case GPTOSS_K_ROPE: // qkv in and out, position; bias once; cos/sin rows stay in cache
    return t * (2 * QKV * a + 4) + QKV * 4;
  case GPTOSS_K_ADD_NORM: // x in/out, delta in, normed out, gain once
    return t * (2 * H * 4 + 2 * H * a) + H * 4;
  case GPTOSS_K_ROUTER: // logits in, k indices and k weights out
    return t * ((size_t)g.n_experts * a + K * 8);
  case GPTOSS_K_SWIGLU: // k rows of 2I in, k rows of I out
    return t * K * 3 * (size_t)g.inter * a;
  case GPTOSS_K_COMBINE: // k expert rows, k indices and weights, x in/out, normed out, gain once
    return t * (K * H * a + K * 8 + 2 * H * 4 + H * a) + H * 4;
  case GPTOSS_K_ARGMAX: // logits in, one index out
    return t * ((size_t)g.vocab * a + 4);
  default:
    return 0;
  }
}

int gptoss_chain_launches_per_step(const gptoss_chain_t *c, int T) {
  if (!c || T <= 0)
    return 0;
  // embed with the first norm (one launch, or two), 5 per layer, argmax scan (+ its key
  // decode when rows are split)
  const int slices = gptoss_argmax_slices(T, c->cfg.vocab, (gptoss_dtype_t)c->cfg.act_dtype, 1);
  const int opening = (c->cfg.flags & GPTOSS_CHAIN_SPLIT_EMBED_NORM) ? 2 : 1;
  return opening + 5 * c->cfg.n_layers + (slices > 1 ? 2 : 1);
}

} // extern "C"
