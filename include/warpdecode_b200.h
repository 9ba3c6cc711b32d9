/* warpdecode_b200 — C ABI of the B200 (sm_100a) batch-1 MoE decode path.
 *
 * This is the boundary a host engine binds: plain pointers and sizes, int status codes,
 * no C++ or torch types. It stands in for the C++ entry points the reference engine calls
 * for its MoE block (the reference has no C ABI of its own; each function below names the
 * reference interface it replaces, paths relative to the reference project).
 *
 * Conventions
 *   - every function returns 0 on success or a negative WD_E_* code; wd_last_error() gives
 *     the message of the calling thread's most recent failure
 *   - "ggml layout" means the on-disk GGUF block layout, row-major, experts contiguous
 *   - device pointers are CUDA device pointers of the engine's device; `stream` is a
 *     cudaStream_t passed as void* (NULL = the engine's own stream)
 *   - an engine is driven by one host thread at a time (as the reference's is)
 */
#ifndef WARPDECODE_B200_H
#define WARPDECODE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WD_OK 0
#define WD_E_INVALID (-1)     /* bad argument or unsupported geometry */
#define WD_E_CUDA (-2)        /* a CUDA runtime call failed */
#define WD_E_STATE (-3)       /* call order: weights missing, layer out of range, ... */
#define WD_E_DEVICE (-4)      /* the kernel reported an error word (timeout, miss, bad slot) */
#define WD_E_NOMEM (-5)

/* ggml tensor type ids (src/gguf.hpp:26-44). */
#define WD_TYPE_F32 0
#define WD_TYPE_Q4_0 2
#define WD_TYPE_Q8_0 8
#define WD_TYPE_IQ4_NL 20
#define WD_TYPE_IQ3_S 21
#define WD_TYPE_IQ2_S 22

typedef struct wd_engine wd_engine;

/* Geometry of the MoE stack. Replaces the fields load_qwen38_runtime() derives from the
 * GGUF (src/qwen38_runtime.cuh:117-147, src/qwen38_layout.hpp:102-211) and the limits of
 * Qwen38MoeScratch::initialize (src/qwen38_moe.cuh:1709-1714: experts <= 4096, k <= 16). */
/* Two families of kernels serve an engine. The TILED kernels (one launch per layer, per token batch or per stack of
 * layers; slot cache; expert parallelism) take hidden = 256 * 2^n (n <= 5), expert_ffn = 256 * 2^n (n <= 3), IQ3_S or
 * IQ2_S experts with gate and up of one type, and a Q8_0 router. Any other configuration that the reference's
 * ggml-exact path accepts (q38_moe_separate_experts_q8_act_compatible, src/qwen38_moe.cuh:2181-2211: hidden % 256 == 0,
 * expert_ffn % 64 == 0, IQ4_NL down tensors; an F32 router, :2252-2258) - the reference's own 2560 / 640 model among
 * them - runs on the PLAIN-LAYOUT path: tensors stay in ggml layout, one warp per row, every expert resident, one GPU;
 * wd_moe_forward, wd_moe_forward_host, wd_read_tap and wd_stack_step (as a chain of per-layer calls) serve such an
 * engine, the slot cache, expert parallelism, profiling stamps and the device-side generator return WD_E_INVALID. */
typedef struct {
    int32_t hidden;          /* multiple of 256 */
    int32_t expert_ffn;      /* multiple of 256 (IQ3_S / IQ2_S down) or of 64 (IQ4_NL down) */
    int32_t shared_ffn;      /* 0 = no shared expert; else multiple of 128 */
    int32_t n_experts;       /* multiple of 8, <= 1024 */
    int32_t top_k;           /* 1..16 */
    int32_t n_layers;
    int32_t gate_type, up_type, down_type;   /* WD_TYPE_IQ3_S or WD_TYPE_IQ2_S; down also WD_TYPE_IQ4_NL */
    float w_scale;           /* expert_weights_scale; 0 or 1 = none */
    int32_t ep_rank, ep_size;/* this engine owns experts [rank*E/size, (rank+1)*E/size) */
    int32_t max_tokens;      /* tokens per forward call, 1..4 (batch verify) */
    int32_t device;          /* CUDA device ordinal */
    int64_t cache_mib;       /* expert slot pool size; <= 0: size it to hold every owned expert.
                                Same meaning as WARODECODE_EXPERT_CACHE_MIB
                                (src/qwen38_tuning.hpp:113-116). On the plain-layout path: the room
                                the experts may take; they must all fit. */
    float rms_eps;           /* epsilon of the optional fused RMSNorm prologue */
    int32_t router_f32;      /* nonzero: the router is F32 [n_experts][hidden], set with wd_set_router_f32 and applied
                                to the F32 input in ggml_vec_dot_f32 order (src/qwen38_moe.cuh:2252-2258,
                                src/matrix.cuh:218-250); 0: Q8_0, set with wd_set_router */
} wd_config;

/* ---- lifetime ------------------------------------------------------------------------ */
/* Replaces load_qwen38_runtime() + Qwen38DecodeState::initialize() for the MoE part
 * (src/qwen38_runtime.cuh:117, src/qwen38_state.cuh:59-120): allocates the slot pool, the
 * per-layer tables and all scratch once; forward calls allocate nothing. */
int wd_engine_create(const wd_config *cfg, wd_engine **out);
void wd_engine_destroy(wd_engine *e);
const char *wd_last_error(void);
/* Library/ABI version, (major << 16) | minor. */
int wd_version(void);

/* Default slot pool size for a GPU with `memory_mib` of memory:
 * clamp(0.75 * memory_mib - 8192, 512, 65536), overridden by the environment variable
 * WARODECODE_EXPERT_CACHE_MIB when it holds a positive integer
 * (qwen38_tuning_for_gpu, src/qwen38_tuning.hpp:88-116). */
int64_t wd_default_cache_mib(int64_t memory_mib);

/* ---- weights ------------------------------------------------------------------------- */
/* Router of one layer: Q8_0 [n_experts][hidden] in ggml layout, host memory; optional F32
 * per-expert logit bias. Replaces upload_matrix(router) (src/qwen38_runtime.cuh:198). */
int wd_set_router(wd_engine *e, int layer, const void *router_q8_0, const float *bias);
/* Same for an engine created with router_f32: F32 [n_experts][hidden], host memory (launch_matrix_gemv_f32_weights,
 * src/matrix.cuh:257). */
int wd_set_router_f32(wd_engine *e, int layer, const float *router, const float *bias);
/* Shared expert of one layer: F32 gate vector [hidden] and Q8_0 gate/up [shared_ffn][hidden],
 * down [hidden][shared_ffn]. Replaces load_qwen38_shared_expert (src/qwen38_moe.cuh:564-599). */
int wd_set_shared(wd_engine *e, int layer, const float *gate_vec, const void *gate_q8_0,
                  const void *up_q8_0, const void *down_q8_0);
/* RMSNorm weight applied to the block input when the fused prologue is used (may be NULL). */
int wd_set_norm(wd_engine *e, int layer, const float *weight);
/* Routed experts of one layer: three 3-D tensors in ggml layout in HOST memory (typically
 * the GGUF mapping). The pointers are retained: they must stay valid for the engine's
 * lifetime, exactly as the reference requires of its GgufFile (src/qwen38_runtime.cuh:201).
 * Experts this rank owns are uploaded now when the pool holds them all, otherwise on demand. */
int wd_set_experts(wd_engine *e, int layer, const void *gate, const void *up, const void *down);
/* Same with the ggml type of each tensor given per layer (the reference model's routed experts are IQ2_S in every
 * layer but one, which is IQ3_S: src/qwen38_moe.cuh:2185-2190). An engine on the plain-layout path takes any accepted
 * combination per layer; a tiled engine only the types it was created with. */
int wd_set_experts_typed(wd_engine *e, int layer, const void *gate, int gate_type, const void *up, int up_type,
                         const void *down, int down_type);
/* Same from the fused form some files carry: ONE tensor [n_experts][2 * expert_ffn][hidden] per layer, each expert's
 * gate rows followed by its up rows (ffn_gate_up_exps, qwen38_moe_tensors, src/qwen38_moe.cuh:601-612, :2688).
 * Engines on the plain-layout path only. */
int wd_set_experts_fused(wd_engine *e, int layer, const void *gate_up, int gate_up_type, const void *down, int down_type);
/* Same, from ggml-layout tensors already in DEVICE memory (used by the synthetic model
 * generator); needs a pool that holds every owned expert. Nothing is retained. */
int wd_set_experts_device(wd_engine *e, int layer, const void *gate, const void *up, const void *down);

/* ---- expert slot cache (GpuExpertCache, src/expert_cache.cuh:2156-2536) ---------------- */
/* Number of slots in the pool / bytes of one slot (gate + up + down of one expert). */
int64_t wd_cache_slot_count(const wd_engine *e);
int64_t wd_cache_slot_bytes(const wd_engine *e);
/* Makes (layer, expert) resident and returns its slot index; a miss fills the least
 * recently used slot from the host tensors. Replaces GpuExpertCache::acquire (:2252). */
int wd_cache_acquire(wd_engine *e, int layer, int expert, int *slot);
/* hits / misses / evictions since creation (ExpertCacheMonitor counters, :1671). */
int wd_cache_stats(const wd_engine *e, int64_t stats[3]);
/* Miss stream since creation: bytes sent host -> device, nanoseconds of host time spent placing missed experts
 * (reads, enqueueing the copies), number of layers that went through the placement
 * (the per-stage timings of ExpertStagePath, src/expert_cache.cuh:1166-1273). */
int wd_cache_stream_stats(const wd_engine *e, int64_t stats[3]);

/* ---- forward --------------------------------------------------------------------------- */
/* One MoE block on device buffers: x [n_tokens][hidden] F32 -> out [n_tokens][hidden] F32
 * (router select, selected experts, ordered weighted combine, shared expert, finish).
 * Replaces run_qwen38_routed_moe_separate_f32_x + run_qwen38_shared_expert_f32_x +
 * q38_finish_moe_f32 (src/qwen38_moe.cuh:3761, :3963, :2442) and, for n_tokens in 2..max_tokens,
 * Qwen38MoeTokenBatch::run (:2955): pair (t, j) = expert ids[t][j] on the activation of token t, each
 * token combined in its own rank order. Enqueues on `stream` (NULL: the engine's own non-blocking stream,
 * which does not synchronise with the legacy default stream) and returns without synchronising when
 * every selected expert is resident; with a capped cache it synchronises once per token. */
int wd_moe_forward(wd_engine *e, int layer, const float *x_dev, float *out_dev, int n_tokens,
                   void *stream);
/* Same through HOST buffers: copies x in, runs the block, copies out back, synchronises. */
int wd_moe_forward_host(wd_engine *e, int layer, const float *x_host, float *out_host, int n_tokens);
/* One decode token through layers [0, n_layers) of the stack: per layer
 * x = RMSNorm(residual) * norm_weight, residual += moe(x). residual_dev is [hidden] F32,
 * updated in place. The whole token is one kernel launch. */
int wd_stack_step(wd_engine *e, float *residual_dev, void *stream);
int wd_stack_step_host(wd_engine *e, const float *residual_in_host, float *residual_out_host);

/* ---- inspection (parity tests; not on the hot path) ------------------------------------- */
#define WD_TAP_LOGITS 0       /* F32 [n_experts] */
#define WD_TAP_IDS 1          /* I32 [top_k] */
#define WD_TAP_WEIGHTS 2      /* F32 [top_k] */
#define WD_TAP_ACT 3          /* F32 [top_k][expert_ffn]  silu(gate)*up */
#define WD_TAP_EXPERT_OUT 4   /* F32 [top_k][hidden] */
#define WD_TAP_ROUTED 5       /* F32 [hidden] */
#define WD_TAP_SHARED 6       /* F32 [hidden] shared expert before its gate */
#define WD_TAP_SHARED_GATE 7  /* F32 [1] */
#define WD_TAP_SHARED_ACT 8   /* F32 [shared_ffn] */
#define WD_TAP_STAMPS 9       /* U64 [sm_count][32] phase timestamps (ns), see wd_set_profiling */
#define WD_TAP_FALLBACKS 10   /* U32 [1] rows so far whose ids came from the exact rungs because the proof of the
                               * threshold pick failed (0 for engines created with WD_THRESHOLD_SELECT=0) */
/* Copies a tap of the most recent forward of token `token` to host memory (synchronises).
 * token = -1 means the last token of that call. After a batch of several tokens, ids and weights
 * are kept for every token; the other taps show the last token only (earlier ones: WD_E_STATE).
 * The post-conditions the reference's callers read from Qwen38MoeScratch
 * (d_logits/h_ids/h_weights/d_accum/down_f32/d_shared_gate, src/qwen38_moe.cuh:1804-1830). */
int wd_read_tap(wd_engine *e, int tap, int token, void *dst, size_t bytes);
/* Per-phase device timestamps (the role of the reference's Q38MoeKernelProfiler sites,
 * src/qwen38_moe.cuh:296-535): when on, every CTA of the layer kernel records the global timer at
 * its phase boundaries (0 start, 1 table, 2 x quantised, 3 rows done, 4 barrier, 5 selection,
 * 6 copies issued, 7 gate/up done, 8 barrier, 9 activations quantised, 10 end). Off by default. */
int wd_set_profiling(wd_engine *e, int on);
/* Number of SMs = CTAs of the layer kernel. */
int wd_sm_count(const wd_engine *e);
/* Name of the kernel a stack step of this engine launches (for bench records). */
const char *wd_kernel_name(const wd_engine *e);
/* ---- The plain (dense) Q4_0 decoder: the Llama-style per-token step of the reference's dense path
 * (Model / Runtime / emit_step, src/warodecode.cu:1211-2150): embedding row, per layer RMSNorm -> fused QKV product ->
 * rotary embedding (GPT-NeoX pairing) + cache store -> decode attention -> output product -> RMSNorm -> gate/up
 * product -> SiLU(g) * u -> down product, output norm, output head, greedy arg-max. Every 2-D tensor is Q4_0 in ggml
 * block layout ([rows][cols / 32] blocks of 18 bytes); activations are quantised to Q8_0 for the products, as the
 * reference does (:1504-1562). One CUDA-graph replay per token; token and position stay on the device. ---- */
typedef struct wd_dense_config {
    int hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, n_layers, max_ctx;
    float rms_eps, rope_theta;
    int device;
} wd_dense_config;
typedef struct wd_dense_decoder wd_dense_decoder;
#define WD_DT_TOKEN_EMBD 0   /* Q4_0 [vocab][hidden] */
#define WD_DT_OUTPUT_NORM 1  /* F32  [hidden] */
#define WD_DT_OUTPUT 2       /* Q4_0 [vocab][hidden] */
#define WD_DT_ATTN_NORM 3    /* F32  [hidden], per layer */
#define WD_DT_WQKV 4         /* Q4_0 [(n_heads + 2 n_kv_heads) * head_dim][hidden]: q rows, k rows, v rows (Layer::qkv) */
#define WD_DT_WO 5           /* Q4_0 [hidden][n_heads * head_dim] */
#define WD_DT_FFN_NORM 6     /* F32  [hidden] */
#define WD_DT_W_GATE_UP 7    /* Q4_0 [2 * ffn][hidden]: gate rows, then up rows (Layer::gate_up) */
#define WD_DT_W_DOWN 8       /* Q4_0 [hidden][ffn] */
#define WD_DT_BQKV 9         /* F32  [(n_heads + 2 n_kv_heads) * head_dim], optional: q, k, v biases (Qwen2 files) */
#define WD_DT_Q_NORM 10      /* F32  [head_dim], optional: RMSNorm weight of every q head before the rotary embedding (Qwen3) */
#define WD_DT_K_NORM 11      /* F32  [head_dim], optional: the same for the k heads */
int wd_dense_decoder_create(const wd_dense_config *cfg, wd_dense_decoder **out);
/* Decoder with the geometry and every tensor of a Llama-style Q4_0 model file (architectures llama, qwen2, qwen3), read
 * the way load_model does (src/warodecode.cu:1255-1345): q/k/v and gate/up joined row-wise, an absent output.weight tied
 * to the embedding table; Q8_0 and Q6_K matrices (the output head and some ffn_down tensors of the Q4_0 files llama.cpp
 * writes) requantised to Q8_0 on the host by ggml_requantize_row_to_q8_0 (src/ggml_dequant.hpp:362-392); q/k/v biases
 * (Qwen2) and q/k head norms (Qwen3) read. Files with partial or scaled rotary embeddings or 2-D tensors of other types
 * are refused by name. The file may be closed afterwards (wd_gguf is declared further down). */
struct wd_gguf;
int wd_dense_decoder_load_gguf(const struct wd_gguf *g, int max_ctx, int device, wd_dense_decoder **out);
/* The configuration a decoder was created with. */
int wd_dense_decoder_config(const wd_dense_decoder *d, wd_dense_config *cfg);
void wd_dense_decoder_destroy(wd_dense_decoder *d);
/* What a token runs on: a CUDA graph of per-operation kernels (the default, and the faster of the two as measured), or
 * with WD_DENSE_TOKEN_KERNEL=1 and a geometry that fits it one persistent launch of the token kernel. Same results. */
const char *wd_dense_decoder_kernel_name(const wd_dense_decoder *d);
/* `layer` is ignored for the three model-level tensors. The bytes are copied; the pointer is not kept. */
int wd_dense_decoder_set_tensor(wd_dense_decoder *d, int layer, int which, const void *host);
/* Same for a 2-D tensor given as WD_TYPE_Q4_0 or WD_TYPE_Q8_0 blocks (34 bytes per 32 values): the reference's dense
 * loader turns every 2-D tensor that is not Q4_0 into Q8_0 and multiplies with it as such (planarize_q4,
 * src/warodecode.cu:1027-1075). A tensor keeps its type once the first token has been decoded. */
int wd_dense_decoder_set_tensor_typed(wd_dense_decoder *d, int layer, int which, int type, const void *host);
/* ggml type of a tensor as the decoder holds it (WD_TYPE_F32 for the norms), or a negative error code. */
int wd_dense_decoder_tensor_type(wd_dense_decoder *d, int layer, int which);
int wd_dense_decoder_get_tensor(wd_dense_decoder *d, int layer, int which, void *host_out, size_t bytes);
/* Every 2-D tensor drawn N(0, sigma) and quantised to Q4_0 on the device, norms 1 (synthetic models for measurements). */
int wd_dense_decoder_synth(wd_dense_decoder *d, unsigned long long seed, float sigma);
/* Greedy decode from position 0: the prompt is fed token by token, then n_gen tokens are generated (Runtime::run,
 * src/warodecode.cu:2120-2150). out_tokens [n_prompt + n_gen] receives the prompt followed by the generated tokens;
 * ms_total (optional) the device time of the n_prompt + n_gen - 1 steps. */
int wd_dense_decoder_decode(wd_dense_decoder *d, const int *prompt, int n_prompt, int n_gen, int *out_tokens, float *ms_total);
/* Profiling of the token kernel: when WD_DENSE_STAMPS was set at creation, the SM clock counter of one CTA at the twelve
 * steps of layer 1 of the last token (residual gathered, norm, QKV rows, attention, attention output gathered, O rows,
 * residual gathered, norm, gate/up rows, activations gathered, down rows). */
int wd_dense_decoder_stamps(wd_dense_decoder *d, unsigned long long *out12);
/* Logits of the last step [vocab] and the residual stream before the output norm [hidden]; either may be null. */
int wd_dense_decoder_read(wd_dense_decoder *d, float *logits_host, float *hidden_host);

/* Measurement, no counterpart in the reference: SM clock cycles one SM of `device` needs to decode a round of `warps`
 * IQ3_S tiles (32 blocks = 8192 weights each, one per warp) that already sit in shared memory, against Q8_K activations
 * of nsb superblocks, with the layer kernels' own decoder (unroll 1: as the single-token kernel runs it; 8: as the batch
 * kernel does). Median over the SMs. This is the instruction-issue bound of the expert GEMVs. */
int wd_measure_tile_decoder(int device, int nsb, int warps, int unroll, double *cycles_per_round);
/* Name of the kernel a token batch (wd_moe_forward with n_tokens > 1) runs on: the batch kernel when the engine has
 * every expert resident on one GPU and the geometry fits it, else the kernel above walking the tokens. */
const char *wd_batch_kernel_name(const wd_engine *e);
/* Name of the kernel the LAST forward call ran on. One-token calls of wd_moe_forward take the batch kernel too where it
 * is available (it is the faster one for a single layer); WD_BATCH_SINGLE=0 keeps them on the layer kernel. */
const char *wd_last_kernel_name(const wd_engine *e);
/* Device error word of the last forward (0 = none) and a reset of the barrier state. */
int wd_device_status(wd_engine *e, int *status);

/* ---- stand-alone pieces (unit parity tests) ---------------------------------------------- */
/* Router chain on given logits: softmax over all experts, top-k, renormalised weights
 * (q38_launch_topk_softmax, src/qwen38_moe.cuh:1065-1083). Host in, host out. */
int wd_router_topk_host(const float *logits, int n_experts, int k, float w_scale, int *ids,
                        float *weights, float *probs);
/* Activation quantisers on host buffers, output in ggml block layout (Q8_0: 34-byte blocks;
 * Q8_K: 292-byte blocks d/qs/bsums) (src/qwen38_hc.cuh:368, src/lowbit.cuh:815). */
int wd_quantize_q8_0_host(const float *x, int n, void *blocks);
int wd_quantize_q8_K_host(const float *x, int n, void *blocks);
/* y = W x for one low-bit matrix in ggml layout (host), through the same repack + decode the
 * engine uses. `partials`, if not NULL, receives the int32 sums [rows][cols/256][8] (IQ types). */
int wd_matvec_host(int type, const void *w, int rows, int cols, const float *x, float *y,
                   int32_t *partials);
/* ---- model load from GGUF ------------------------------------------------------------------ */
/* Read-only mapping of a GGUF file (v2/v3) with its metadata and tensor directory parsed: the part of
 * GgufFile (src/gguf.hpp) and load_qwen38_runtime (src/qwen38_runtime.cuh:117-265) that the MoE path
 * needs. wd_gguf_config fills the geometry fields of *cfg (hidden, expert_ffn, shared_ffn, n_experts,
 * top_k, n_layers, the three expert tensor types, w_scale, rms_eps) from the qwen4exp.* keys
 * (src/qwen38_layout.hpp:102-142) and the tensors' own extents, and leaves ep_rank, ep_size, max_tokens,
 * device and cache_mib to the caller. wd_engine_load_gguf hands every layer's tensors
 * (blk.N.ffn_gate_inp.weight [+ .bias], ffn_{gate,up,down}_exps.weight, ffn_gate_inp_shexp.weight,
 * ffn_{gate,up,down}_shexp.weight, optional ffn_norm.weight; src/qwen38_moe.cuh:569-573, :601-612) to an
 * engine created from that config. Expert tensors are used in place (a capped cache streams its misses
 * straight from the mapping): close the file only after the engine is destroyed.
 * wd_gguf_tensor returns a pointer into the mapping plus ggml type id and extents (GGUF order). */
typedef struct wd_gguf wd_gguf;
int wd_gguf_open(const char *path, wd_gguf **out);
void wd_gguf_close(wd_gguf *g);
int wd_gguf_config(const wd_gguf *g, wd_config *cfg);
int wd_gguf_tensor(const wd_gguf *g, const char *name, const void **data, int *type, int64_t dims[4], int *n_dims);
int wd_engine_load_gguf(wd_engine *e, const wd_gguf *g);

/* ---- expert parallelism ------------------------------------------------------------------ */
/* The reference runs on one GPU; its expert tables (src/expert_cache.cuh:2116-2146) shard by expert, and
 * these calls add that. An engine created with ep_size > 1 holds and computes only the experts of its
 * rank; the router and the shared expert are replicated, so every rank selects the same experts. Until
 * it is connected, wd_moe_forward returns this rank's PARTIAL routed sum (+ shared expert). Once
 * connected, the kernel of every rank stores the output rows of its selected experts straight into
 * every peer's row buffer (value and layer tag in one 8-byte store over NVLink), and every rank performs
 * the ordered combine over all top_k rows: results are bit-identical to one GPU for any ep_size.
 * All ranks must then issue the same sequence of forward calls; a rank that waits about a second for
 * a peer's rows gives up and raises device status bit 1.
 * wd_ep_export writes wd_ep_handle_bytes() bytes that another PROCESS passes to wd_ep_connect
 * (`handles` = the ep_size - 1 other ranks' handles back to back, any order); engines of one process
 * on different devices use wd_ep_connect_local. Disconnect (or destroy) only while no rank is running. */
int wd_ep_handle_bytes(void);
int wd_ep_export(wd_engine *e, void *handle_out);
int wd_ep_connect(wd_engine *e, int n_peers, const void *handles);
int wd_ep_connect_local(wd_engine *e, int n_peers, wd_engine *const *peers);
int wd_ep_disconnect(wd_engine *e);
/* Clears the status word, the layer-tag epoch and every exchange word of this engine. After any rank of a
 * connected group reported a non-zero device status, call this on EVERY rank (all idle) before the next
 * forward: the ranks' tag epochs must agree. (wd_device_status does it for the reporting engine only.) */
int wd_reset_exchange(wd_engine *e);

/* ---- dense Q4_0 matvec (the plain decoder path) ------------------------------------------ */
/* y = W x for a Q4_0 matrix [rows][cols] against the Q8_0-quantised activation, the operator of
 * q4_0_q8_0_gemv_kernel + q8_0_quantize_half_kernel (src/warodecode.cu:1535-1562, :1504). The matrix is
 * packed once (planarize_q4, src/warodecode.cu:1027-1098, here: 32-row tiles, 16-byte quants then f16
 * scales; 18 bytes per 32 weights) from ggml blocks on the host or on the device; the returned device
 * pointer belongs to the caller until wd_dense_free. x_dev [cols] and y_dev [rows] are F32 device buffers;
 * the call enqueues one kernel on `stream`. rows % 32 == 0, cols % 256 == 0, cols <= 32768.
 * Float order: ggml's ggml_vec_dot_q4_0_q8_0 (eight lanes, one fmaf per block, 8-lane tree). */
int wd_dense_pack_q4_0(const void *w_ggml_host, int rows, int cols, void **packed_dev);
int wd_dense_pack_q4_0_device(const void *w_ggml_dev, int rows, int cols, void **packed_dev, void *stream);
int wd_dense_matvec_q4_0(const void *packed_dev, int rows, int cols, const float *x_dev, float *y_dev, void *stream);
int wd_dense_free(void *packed_dev);
/* Output head: token = arg-max over the finite logits of W x, W a Q8_0 matrix [rows = vocab][cols = hidden]
 * packed like the Q4_0 one (wd_dense_pack_q8_0*; free with wd_dense_free). The operator of the head GEMV
 * plus q38_argmax_kernel (src/qwen38_forward.cuh:450-486): largest value, ties to the lowest index,
 * non-finite logits skipped and reported in *nonfinite_dev (nullable), token 0 when nothing is finite.
 * logits_dev (nullable) receives the F32 logits [rows]. One matvec kernel with the arg-max fused
 * (64-bit monotone key + atomicMax, as src/warodecode.cu:1603-1632) and a one-thread finish kernel on
 * `stream`; calls on the same packed matrix must not overlap (its arg-max state sits behind the matrix). */
int wd_dense_pack_q8_0(const void *w_ggml_host, int rows, int cols, void **packed_dev);
int wd_dense_pack_q8_0_device(const void *w_ggml_dev, int rows, int cols, void **packed_dev, void *stream);
/* out_dev[cols] = row *token_dev of a Q8_0 embedding table [rows][cols] in ggml layout on the device
 * (d * q per value; the token is clamped to the table). With wd_stack_step and wd_head_argmax_q8_0 a greedy
 * decode loop of the MoE stack stays on the device: embed -> layers -> head -> token. */
int wd_embed_q8_0(const void *table_ggml_dev, int rows, int cols, const int *token_dev, float *out_dev, void *stream);
int wd_head_argmax_q8_0(void *packed_dev, int rows, int cols, const float *x_dev, float *logits_dev, int *token_dev,
                        int *nonfinite_dev, void *stream);

/* Has no counterpart in the reference. y = W x for one IQ3_S matrix like wd_matvec_host, for callers
 * that must not allocate device memory (HBM already handed to the expert pool, a latency-critical
 * token loop where cudaMalloc's device-wide synchronisation is unacceptable, memory owned by another
 * allocator): w_dev (ggml layout), x_dev, y_dev are DEVICE buffers of the caller; the only scratch is
 * a fixed 8 MiB array inside the library that every GPU loading it holds until exit, so rows*cols/256*110
 * must not exceed 8 MiB - 1 KiB (larger is refused with a message). Work is enqueued on `stream`.
 * The first call on each device looks up the array's device address and uploads the 1 KiB codebook into
 * its front with a blocking copy (later calls only enqueue kernels); make that call before any stream
 * capture. All calls share the array, which keeps the last call's contents (nothing needs clearing:
 * every byte read is first rewritten); calls that overlap on the GPU race on it. */
int wd_matvec_iq3s_noalloc(const void *w_dev, int rows, int cols, const float *x_dev, float *y_dev,
                           void *stream);

/* ---- synthetic model generator (device side) ----------------------------------------------- */
/* Fills `dst` (device) with `rows` x `cols` N(0, sigma) weights drawn from (seed, stream_id)
 * and quantised to `type` (WD_TYPE_F32 or WD_TYPE_Q8_0; IQ3_S tensors come from wd_synth_model) in
 * ggml layout. Used to build full-size synthetic tensors (embedding table, output head) in HBM. */
int wd_synth_tensor_device(int type, int rows, int cols, float sigma, uint64_t seed,
                           uint64_t stream_id, void *dst_dev, void *stream);
/* Builds every layer of the engine's model from `seed` directly on the device. */
int wd_synth_model(wd_engine *e, uint64_t seed, float sigma, float bias_sigma);
/* Copies one owned expert's ggml-layout tensors (as the generator produced them) to host
 * buffers so a CPU oracle can consume the same bytes. Regenerates them from the seed. */
int wd_synth_expert_host(wd_engine *e, uint64_t seed, float sigma, int layer, int expert,
                         void *gate, void *up, void *down);
int wd_synth_dense_host(wd_engine *e, uint64_t seed, float sigma, float bias_sigma, int layer,
                        void *router, float *bias, float *gate_vec, void *sh_gate, void *sh_up,
                        void *sh_down);

#ifdef __cplusplus
}
#endif
#endif /* WARPDECODE_B200_H */
