/*
 * gptoss_engine.h -- host side of the fused-kernel path: device-buffer helpers,
 * the RoPE table builder and the layer-chain driver that strings the kernels of
 * gptoss_kernels.h together in the order the reference engine's decode step
 * launches them (getp-csrc/engine/gpu_engine.hpp:459-690 of
 * n30nd/Optimize_Inference_GPT-OSS).
 *
 * Everything here is host C++ behind a C ABI; nothing is computed on the CPU
 * except the cos/sin tables, which the reference engine also builds on the host
 * (gpu_engine.hpp:388-396).  All functions return a GPTOSS_* status.
 */
#ifndef GPTOSS_ENGINE_H
#define GPTOSS_ENGINE_H

#include "gptoss_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- devices, buffers, streams ----------------------------------------------
 * The engine owns every device buffer (gpu_alloc / gpu_upload,
 * gpu_engine.hpp:119-132); the kernels only borrow pointers.  These are thin
 * wrappers over the CUDA runtime so that a host program needs no other CUDA
 * binding. */
GPTOSS_API int gptoss_device_count(int *count);
GPTOSS_API int gptoss_device_set(int device);
GPTOSS_API int gptoss_device_name(int device, char *buf, int buf_len);
GPTOSS_API int gptoss_device_alloc(void **ptr, size_t bytes);
GPTOSS_API int gptoss_device_free(void *ptr);
GPTOSS_API int gptoss_device_memset(void *ptr, int byte, size_t bytes, gptoss_stream_t stream);
/* Copies are queued on `stream`; host memory must stay valid until the stream
 * has been synchronised (pinned memory makes them truly asynchronous). */
GPTOSS_API int gptoss_upload(void *dst_device, const void *src_host, size_t bytes,
                             gptoss_stream_t stream);
GPTOSS_API int gptoss_download(void *dst_host, const void *src_device, size_t bytes,
                               gptoss_stream_t stream);
GPTOSS_API int gptoss_host_alloc_pinned(void **ptr, size_t bytes);
GPTOSS_API int gptoss_host_free_pinned(void *ptr);
GPTOSS_API int gptoss_stream_create(gptoss_stream_t *stream);
GPTOSS_API int gptoss_stream_destroy(gptoss_stream_t stream);
GPTOSS_API int gptoss_stream_synchronize(gptoss_stream_t stream);
GPTOSS_API int gptoss_device_synchronize(void);

/* CUDA events, for timing on the stream the kernels run on. */
typedef void *gptoss_event_t;
GPTOSS_API int gptoss_event_create(gptoss_event_t *event);
GPTOSS_API int gptoss_event_destroy(gptoss_event_t event);
GPTOSS_API int gptoss_event_record(gptoss_event_t event, gptoss_stream_t stream);
GPTOSS_API int gptoss_event_synchronize(gptoss_event_t event);
GPTOSS_API int gptoss_event_elapsed_ms(gptoss_event_t start, gptoss_event_t stop, float *ms);

/* Overwrites `bytes` of scratch device memory (at least as large as the L2
 * cache) so that the next kernel finds none of its inputs cached. */
GPTOSS_API int gptoss_flush_l2(void *scratch, size_t bytes, gptoss_stream_t stream);

/* Stream capture into a replayable graph, the way the reference engine would batch a step's
 * launches (it has no graphs: HIP launches one kernel at a time, gpu_engine.hpp:459-690).
 * Between gptoss_graph_begin and gptoss_graph_end every launch made by this thread on `stream`
 * is recorded instead of run; a kernel should have been launched once outside capture first.
 * The stream must be one made by gptoss_stream_create (not the default stream). */
typedef void *gptoss_graph_t;
GPTOSS_API int gptoss_graph_begin(gptoss_stream_t stream);
GPTOSS_API int gptoss_graph_end(gptoss_stream_t stream, gptoss_graph_t *graph);
GPTOSS_API int gptoss_graph_launch(gptoss_graph_t graph, gptoss_stream_t stream);
GPTOSS_API int gptoss_graph_destroy(gptoss_graph_t graph);

/* ---- RoPE tables --------------------------------------------------------------
 * cos/sin of every position 0..n_pos-1, [n_pos, head_dim/2] fp32 each, computed
 * on the host with the C library's powf/logf/cosf/sinf exactly as the engine
 * does with run.cpp's compute_cos_sin (run.cpp:422-504; gpu_engine.hpp:388-396):
 * YaRN concentration 0.1 ln(factor) + 1, NTK-by-parts blend between beta_fast
 * and beta_slow.  Host pointers. */
GPTOSS_API int gptoss_build_rope_tables(int n_pos, int head_dim, float theta, float factor,
                                        float orig_ctx, float beta_fast, float beta_slow,
                                        float *cos_host, float *sin_host);

/* ---- seeded synthetic tensors ---------------------------------------------------
 * Counter-based generator: element j of stream (seed, stream_id) is
 * mean + sd * N(0,1), from two splitmix64 hashes of the counter through
 * Box-Muller, so any thread count produces the same bits.  Fills HOST memory
 * as fp32 or as bf16 (round to nearest even); runs on `threads` host threads
 * (0 = all).  Integers: uniform in [lo, hi). */
GPTOSS_API int gptoss_synth_normal(void *dst_host, gptoss_dtype_t dtype, size_t count,
                                   uint64_t seed, uint64_t stream_id, float mean, float sd,
                                   int threads);
GPTOSS_API int gptoss_synth_uniform_int(int *dst_host, size_t count, uint64_t seed,
                                        uint64_t stream_id, int lo, int hi);

/* ---- the layer chain ------------------------------------------------------------
 * One decode step of the engine with the GEMMs and the attention taken out:
 *
 *   embed + norm of layer 0, one launch     (step_embed, gpu_engine.hpp:461; layer_attention, :491)
 *   per layer:  [QKV GEMM]  bias + RoPE     (:493-496)
 *               [attention, out GEMM]  residual add + norm      (:499-504)
 *               [router GEMM]  top-k + softmax                  (layer_route, :522-527)
 *               [mlp1 GEMM]  SwiGLU                             (layer_experts, :563-572)
 *               [mlp2 GEMM]  combine + residual + next norm     (layer_combine, :596-603)
 *   [LM-head GEMM]  greedy argmax                               (step_logits, :615-619)
 *
 * Each bracketed GEMM is replaced by a device-resident stand-in tensor of the
 * GEMM's output shape that the caller fills (per layer: attention projection
 * [T,H], qkv [T,QKV], router logits [T,E], mlp1 output [k T, 2I], expert output
 * [k T, H]; and the logits [T,V]); the chain's own outputs that would feed a
 * GEMM (normalised rows, rotated qkv, SwiGLU rows) are written to scratch.  The
 * residual stream, the routing weights and the picked tokens flow through the
 * chain exactly as in the engine.  A chain owns one stream and is driven by one
 * host thread at a time (the engine has one thread per device too,
 * gpu_engine.hpp:916-945); different chains are independent. */
typedef struct gptoss_chain gptoss_chain_t;

/* Bit of gptoss_chain_config_t.flags that only the chain reads: open the step with the
 * reference's two launches (gptoss_embed, then gptoss_add_rmsnorm) instead of the fused
 * gptoss_embed_rmsnorm.  Kernels ignore it. */
#define GPTOSS_CHAIN_SPLIT_EMBED_NORM 0x100u

typedef struct {
  int vocab, hidden, n_experts, top_k, inter, n_layers, head_dim, n_q_heads, n_kv_heads;
  int max_pos;    /* rows of the cos/sin tables (positions 0..max_pos-1) */
  float orig_ctx; /* initial_context_length */
  float theta, factor, beta_fast, beta_slow, swiglu_limit;
  int act_dtype;  /* gptoss_dtype_t of GEMM-side tensors: F32 = fp32 mode, BF16 = bf16-activation mode */
  unsigned flags; /* GPTOSS_EXACT / GPTOSS_FMA / GPTOSS_PDL, passed to every kernel; GPTOSS_CHAIN_* */
} gptoss_chain_config_t;

/* gpt-oss-20b (24 layers, 32 experts) or gpt-oss-120b (36 layers, 128 experts)
 * shapes (export_model_bin/gpt-oss-20b/config.json and gpt-oss-120b/config.json).
 * which: 20 or 120.  flags come back as GPTOSS_PDL, plus GPTOSS_EXACT for fp32 tensors. */
GPTOSS_API int gptoss_chain_config_gpt_oss(int which, gptoss_dtype_t act_dtype, int max_pos,
                                           gptoss_chain_config_t *cfg);

/* Allocates every buffer for up to max_tokens rows on the current device and
 * builds and uploads the RoPE tables.  n_standin_layers: how many distinct
 * per-layer stand-in sets to keep (1..n_layers; layer l uses set l mod n). */
GPTOSS_API int gptoss_chain_create(const gptoss_chain_config_t *cfg, int max_tokens,
                                   int n_standin_layers, gptoss_chain_t **chain);
GPTOSS_API int gptoss_chain_destroy(gptoss_chain_t *chain);
GPTOSS_API size_t gptoss_chain_device_bytes(const gptoss_chain_t *chain);
GPTOSS_API gptoss_stream_t gptoss_chain_stream(const gptoss_chain_t *chain);

typedef enum {
  /* weights (uploaded once) */
  GPTOSS_BUF_EMBEDDING = 0, /* [vocab, hidden] act_dtype */
  GPTOSS_BUF_GAIN_ATTN,     /* per layer [hidden] fp32: norm before attention */
  GPTOSS_BUF_GAIN_FFN,      /* per layer [hidden] fp32: norm before the MoE */
  GPTOSS_BUF_GAIN_OUT,      /* [hidden] fp32: final norm */
  GPTOSS_BUF_QKV_BIAS,      /* per layer [qkv] fp32 */
  GPTOSS_BUF_COS,           /* [max_pos, head_dim/2] fp32 (built by create) */
  GPTOSS_BUF_SIN,
  /* stand-ins for GEMM / attention outputs (per stand-in layer) */
  GPTOSS_BUF_ATTN_PROJ, /* [T, hidden] act_dtype */
  GPTOSS_BUF_QKV,       /* [T, qkv] act_dtype */
  GPTOSS_BUF_ROUTER,    /* [T, n_experts] act_dtype */
  GPTOSS_BUF_MLP1,      /* [top_k T, 2 inter] act_dtype */
  GPTOSS_BUF_EXPERT,    /* [top_k T, hidden] act_dtype */
  GPTOSS_BUF_LOGITS,    /* [T, vocab] act_dtype */
  /* state */
  GPTOSS_BUF_TOKENS,  /* [T] int32 */
  GPTOSS_BUF_POS,     /* [T] int32 */
  GPTOSS_BUF_X,       /* [T, hidden] fp32 residual stream */
  GPTOSS_BUF_NORMED,  /* [T, hidden] act_dtype: last RMSNorm output */
  GPTOSS_BUF_QKV_OUT, /* [T, qkv] act_dtype: biased, rotated */
  GPTOSS_BUF_TOPK_W,  /* [T, top_k] fp32 */
  GPTOSS_BUF_TOPK_E,  /* [T, top_k] int32 */
  GPTOSS_BUF_SWIGLU,  /* [top_k T, inter] act_dtype */
  GPTOSS_BUF_NEXT,    /* [T] int32: picked tokens */
  GPTOSS_BUF_ROW_DONE, /* [T] int32: non-zero = finished request: no experts, residual frozen */
  GPTOSS_BUF_COUNT
} gptoss_chain_buffer_t;

/* Device address and size of a buffer (layer ignored for non-layered ones). */
GPTOSS_API int gptoss_chain_buffer(const gptoss_chain_t *chain, gptoss_chain_buffer_t which,
                                   int layer, void **device_ptr, size_t *bytes);

/* Fills every weight and stand-in with seeded synthetic values of the
 * distributions the real tensors have (embedding N(0,0.02); gains 1+N(0,0.1);
 * bias N(0,0.02); projections, qkv, router logits N(0,1); mlp1 output N(0,2);
 * expert output N(0,1); logits N(0,3)), generated on the HOST for T rows and
 * uploaded.  threads: host threads (0 = all). */
GPTOSS_API int gptoss_chain_fill_synthetic(gptoss_chain_t *chain, int T, uint64_t seed,
                                           int threads);

/* Queues one step for T rows on the chain's stream using the device-resident
 * tokens and positions (GPTOSS_BUF_TOKENS / _POS); no copies, no sync.  The
 * first call for a given T captures the launches into a CUDA graph; later
 * calls replay it.  use_graph = 0 launches kernel by kernel. */
GPTOSS_API int gptoss_chain_enqueue(gptoss_chain_t *chain, int T, int use_graph);

/* One full engine step as gpu_run_wave does it (gpu_engine.hpp:777-798): copy
 * T tokens and positions from host memory, run the chain, copy the T picked
 * tokens back, synchronise the stream.  The copies are nodes of the same CUDA
 * graph as the kernels (one launch call per step); the caller's arrays, pinned
 * or not, pass through a pinned staging block owned by the chain. */
GPTOSS_API int gptoss_chain_step(gptoss_chain_t *chain, int T, const int *tokens_host,
                                 const int *pos_host, int *next_host);

/* Serves one wave of requests the way the reference engine does (gpu_run_wave,
 * gpu_engine.hpp:761-841): request b starts from the first token of its prompt; every step
 * all rows sit at the same position; after the step a row takes the next prompt token while
 * it has one and the picked token afterwards; a row finishes when it takes one of the two
 * end tokens (199999, 200002), is then marked in GPTOSS_BUF_ROW_DONE (re-uploaded only when
 * it changed) so that the router gives it no experts, and the wave ends after `steps`
 * positions or when every row is done.
 *   prompt_tokens / prompt_offsets: the prompts back to back; request b owns
 *       [prompt_offsets[b], prompt_offsets[b+1]), at least one token each
 *   generated: [n_requests, steps + 2] int32, request b's generated tokens from column 0,
 *       closed with -1 (as the reference's output rows are)
 *   n_generated: the reference's count (for each request, position reached - prompt
 *       length + 1)
 * n_requests <= max_tokens, steps <= max_pos.  Host pointers; synchronous. */
GPTOSS_API int gptoss_chain_run_wave(gptoss_chain_t *chain, const int *prompt_tokens,
                                     const int *prompt_offsets, int n_requests, int steps,
                                     int *generated, long long *n_generated, int *steps_run);

/* The same wave with the bookkeeping on the GPU: prompts, the finished-row mask, the
 * output rows and the counters stay in device memory, a one-block kernel behind each
 * step's argmax does what the reference's host loop does between steps
 * (gpu_engine.hpp:800-826), and the host only queues steps, sixteen at a time, looking at
 * the counters in between to stop once every row is done.  No token crosses the bus
 * during the wave: prompts go in before it, output rows come back after it.  Same
 * arguments and, bit for bit, the same outputs as gptoss_chain_run_wave. */
GPTOSS_API int gptoss_chain_run_wave_on_device(gptoss_chain_t *chain, const int *prompt_tokens,
                                               const int *prompt_offsets, int n_requests, int steps,
                                               int *generated, long long *n_generated, int *steps_run);

typedef enum {
  GPTOSS_K_EMBED = 0, /* gather fused with layer 0's norm; the gather alone with GPTOSS_CHAIN_SPLIT_EMBED_NORM */
  GPTOSS_K_NORM,      /* RMSNorm alone (layer 0): launched only with GPTOSS_CHAIN_SPLIT_EMBED_NORM */
  GPTOSS_K_ROPE,     /* qkv bias + RoPE */
  GPTOSS_K_ADD_NORM, /* residual add + RMSNorm */
  GPTOSS_K_ROUTER,
  GPTOSS_K_SWIGLU,
  GPTOSS_K_COMBINE, /* combine + residual + next norm */
  GPTOSS_K_ARGMAX,
  GPTOSS_K_COUNT
} gptoss_chain_kernel_t;

/* Device time per kernel kind, from CUDA events on the chain's stream, summed
 * over `steps` steps, with the number of launches it covers (arrays of
 * GPTOSS_K_COUNT).
 *   mode 0: the step runs in order with an event pair around every launch;
 *   mode 1: the same, and a 256 MB scratch buffer is overwritten before every
 *           launch (cold L2);
 *   mode 2: per kind, all of its launches of a step (one per layer, each on its
 *           own layer's tensors) run back to back between one event pair, so the
 *           cost of the event records themselves (a few microseconds per pair,
 *           comparable to the shortest kernels) is spread over the batch; the
 *           values the chain computes are meaningless in this mode. */
GPTOSS_API int gptoss_chain_profile(gptoss_chain_t *chain, int T, int steps, int mode,
                                    double *ms_per_kind, long *launches_per_kind);

/* Algorithmic bytes one launch of a kernel kind moves for T rows: compulsory
 * reads plus writes, shared tables (gains, bias, cos/sin rows) counted once. */
GPTOSS_API size_t gptoss_chain_kernel_bytes(const gptoss_chain_t *chain,
                                            gptoss_chain_kernel_t kind, int T);
/* Kernel launches in one step of T rows. */
GPTOSS_API int gptoss_chain_launches_per_step(const gptoss_chain_t *chain, int T);

#ifdef __cplusplus
}
#endif
#endif /* GPTOSS_ENGINE_H */
