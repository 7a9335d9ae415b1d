/* jllm_b200.h — C ABI of the B200 (sm_100a) kernel library behind genie-ai-runtime's
 * kernel API.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream passed as
 * `void*` (a cudaStream_t), and returns a status code (0 = ok).  The functions in the
 * first part mirror, one for one, the C++ functions the reference engine calls
 * (include/jllm_kernels.h in the reference; the same library also exports those C++
 * symbols with identical mangling, see jllm_b200_api.hpp, so the engine's objects link
 * against it unchanged).  The second part holds additive extension entry points.
 *
 * Differences from the reference's behaviour, by design: there is no CPU fallback.
 * Where the reference logs and falls back (or zero-fills), these functions record an
 * error retrievable with jllm_b200_last_error(), zero-fill the output where the
 * reference does, and return a non-zero status.
 *
 * All pointers are device pointers unless stated otherwise.  `half` buffers are IEEE
 * binary16.  ggml_type: 12 = Q4_K, 13 = Q5_K, 14 = Q6_K (GGUF block layouts unchanged).
 */
#ifndef JLLM_B200_H
#define JLLM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define JLLM_B200_OK          0
#define JLLM_B200_ERR_ARG     1   /* bad size / shape */
#define JLLM_B200_ERR_TYPE    2   /* unsupported ggml / dense type */
#define JLLM_B200_ERR_PTR     3   /* null, unresolvable or misaligned pointer */
#define JLLM_B200_ERR_CUDA    4   /* CUDA runtime error (text in last_error) */
#define JLLM_B200_ERR_NOMEM   5   /* library scratch could not be (re)allocated */
#define JLLM_B200_ERR_LIMIT   6   /* size beyond a documented maximum */
#define JLLM_B200_ERR_TIMEOUT 7   /* a bounded device-side wait ran out */
#define JLLM_B200_ERR_STATE   8   /* call not valid in the current state */

/* ── library state ───────────────────────────────────────────────────────── */
/* Creates the per-device context (status word, SM count) for `device` (-1 = current).
 * Implicit on first use; call it explicitly before CUDA-graph capture. */
int         jllm_b200_init(int device);
const char* jllm_b200_last_error(void);          /* thread-local text of the last error */
int         jllm_b200_last_error_code(void);
void        jllm_b200_clear_error(void);
/* Synchronises `stream` and returns the device status word (0, or ERR_TIMEOUT if a
 * bounded wait inside a kernel gave up); the word is cleared. */
int         jllm_b200_device_status(void* stream);
long long   jllm_b200_launch_count(void);        /* kernels launched by this library so far */
void        jllm_b200_set_pdl(int on);           /* programmatic dependent launch on/off (default on) */

/* Diagnostic: the NEXT GEMV-family call on this thread also records sixteen %globaltimer stamps (ns) per CTA into
 * device_buf[cta * 16 + k]: 0 kernel entry, 1 first bulk copies issued, 2 producer kernel complete, 3 activation vector
 * staged, 4 first row group landed, 5 warp 0 done, 6 last warp done, 8 + 2u / 9 + 2u task u (< 4) of warp 0 landed /
 * multiplied.  device_buf needs 16 x 2 x SM-count entries. */
void        jllm_b200_debug_gemv_trace(unsigned long long* device_buf);

/* ── mapped-weight registry — include/jllm_kernels.h:40-43, src/engine/model.cpp:39-66 ── */
const void* jllm_b200_resolve_mapped_weight_device_ptr(const void* host_ptr);
void        jllm_b200_register_mapped_weight_region(const void* host_base, const void* device_base, int64_t bytes);
void        jllm_b200_clear_mapped_weight_region(const void* host_base);

/* ── K-quant GEMV family (decode) ────────────────────────────────────────── */
/* gemv_quant — include/jllm_kernels.h:64-72, src/kernels/gemv_q4.cu:2633-2688.
 * y[M] half = W[M x K] . x[K].  Q4_K/Q6_K: x quantised to q8_1, integer dots; Q5_K: float. */
int jllm_b200_gemv_quant(void* y, const void* W, int ggml_type, const void* x, int M, int K, void* stream);
/* gemv_q4 — include/jllm_kernels.h:51-60 (forwards to gemv_quant with Q4_K, gemv_q4.cu:1238-1243). */
int jllm_b200_gemv_q4(void* y, const void* W_q4, const void* scales, const void* x, int M, int K, int group_size, void* stream);
/* gemv_quant_add — :78-87, gemv_q4.cu:2690-2718.  y = half(half(W.x) + residual); fp16-x arithmetic. */
int jllm_b200_gemv_quant_add(void* y, const void* W, int ggml_type, const void* x, const void* residual, int M, int K, void* stream);
/* gemv_quant_pair — :92-104, gemv_q4.cu:2720-2734.  Two projections sharing x. */
int jllm_b200_gemv_quant_pair(void* y0, const void* W0, int type0, int M0, void* y1, const void* W1, int type1, int M1,
                              const void* x, int K, void* stream);
/* gemv_quant_triple — :106-122, gemv_q4.cu:2736-2753.  Three projections sharing x. */
int jllm_b200_gemv_quant_triple(void* y0, const void* W0, int type0, int M0, void* y1, const void* W1, int type1, int M1,
                                void* y2, const void* W2, int type2, int M2, const void* x, int K, void* stream);
/* gemv_quant_f32 — :148-156, gemv_q4.cu:2755-2775.  fp32 output (logits). */
int jllm_b200_gemv_quant_f32(float* y, const void* W, int ggml_type, const void* x, int M, int K, void* stream);
/* gemm_quant_batched — :135-144, gemv_q4.cu:2478-2517.  y[N x M] = x[N x K] . W^T; N == 1 is gemv_quant. */
int jllm_b200_gemm_quant_batched(void* y, const void* W, int ggml_type, const void* x, int M, int N, int K, void* stream);
/* dequant_embedding_row — :160-167, gemv_q4.cu:2777-2809.  Returns 0 on success (the C++ symbol returns bool). */
int jllm_b200_dequant_embedding_row(void* dst, const void* W, int ggml_type, int token_id, int hidden_dim, void* stream);
/* gemv_dense / gemm_dense_batched — :220-227, gemv_q4.cu:2842-2885.  wtype 0 = F32, 1 = F16, 30 = BF16. */
int jllm_b200_gemv_dense(void* out, const void* W, int wtype, const void* x, int M, int K, void* stream);
int jllm_b200_gemm_dense_batched(void* out, const void* W, int wtype, const void* x, int M, int N, int K, void* stream);

/* ── element-wise family ─────────────────────────────────────────────────── */
/* fused_rmsnorm_residual — :174-184, src/kernels/fused_norm.cu:103-165. */
int jllm_b200_fused_rmsnorm_residual(void* output, const void* x, const void* residual, const void* weight,
                                     int rows, int hidden_dim, float eps, int weight_fp32, void* stream);
/* fused_swiglu / fused_geglu — :191-210, src/kernels/convert.cu:106-148. */
int jllm_b200_fused_swiglu(void* output, const void* gate, const void* up, int rows, int intermediate_dim, void* stream);
int jllm_b200_fused_geglu(void* output, const void* gate, const void* up, int rows, int intermediate_dim, void* stream);
/* vec_scale / logit_softcap — :213-216, convert.cu:152-181. */
int jllm_b200_vec_scale(void* x, int n, float s, void* stream);
int jllm_b200_logit_softcap(float* x, int n, float cap, void* stream);
/* softmax_inplace — :406-410, src/kernels/softmax.cu:76-82. */
int jllm_b200_softmax_inplace(float* x, int n, void* stream);
/* fp16_to_int8 — :413-420, convert.cu:71-75.  One absmax scale per row. */
int jllm_b200_fp16_to_int8(int8_t* dst, float* scale_out, const void* src, int rows, int cols, void* stream);

/* ── RoPE — :238-316, src/kernels/rope.cu ─────────────────────────────────── */
int jllm_b200_rope_precompute_table(int max_seq, int head_dim, float theta_base);
int jllm_b200_rope_clear_tables(void);
int jllm_b200_rope_inplace(void* q, void* k, int n_heads, int n_kv_heads, int head_dim, int position, float theta_base, int neox, void* stream);
int jllm_b200_rope_inplace_store_kv_fp16(void* q, void* k, const void* v, void* k_cache_dst, void* v_cache_dst, int n_heads,
                                         int n_kv_heads, int head_dim, int position, float theta_base, int neox, void* stream);
int jllm_b200_rope_inplace_batched(void* q, void* k, int n_heads, int n_kv_heads, int head_dim, int start_pos, int N,
                                   int q_stride, int k_stride, float theta_base, int neox, void* stream);
int jllm_b200_rope_inplace_store_kv_fp16_batched(void* q, void* k, const void* v, void* k_cache_base, void* v_cache_base, int kv_slot,
                                                 int n_heads, int n_kv_heads, int head_dim, int start_pos, int N, int q_stride,
                                                 int kv_stride, float theta_base, int neox, void* stream);
int jllm_b200_rope_inplace_store_kv_fp16_dyn(void* q, void* k, const void* v, void* k_cache_layer_base, void* v_cache_layer_base,
                                             int n_heads, int n_kv_heads, int head_dim, int cache_head_dim, const int* d_pos,
                                             float theta_base, int neox, void* stream);
int jllm_b200_rope_inplace_dyn(void* q, void* k, int n_heads, int n_kv_heads, int head_dim, const int* d_pos, float theta_base,
                               int neox, void* stream);

/* ── attention ───────────────────────────────────────────────────────────── */
/* flash_attention_decode — :323-342, src/kernels/attention.cu:1036-1137.  k_scales / v_scales are fp32,
 * indexed [pos * n_kv_heads + kv_head] (null for FP16 KV). */
int jllm_b200_flash_attention_decode(void* output, const void* q, const void* k_cache, const void* v_cache, int n_heads,
                                     int n_kv_heads, int head_dim, int cache_head_dim, int seq_len, float scale, int kv_int8,
                                     const float* k_scales, const float* v_scales, int window, void* stream);
/* flash_attention_prefill_batched — :354-373, attention.cu:617-697. */
int jllm_b200_flash_attention_prefill_batched(void* output, const void* q, const void* k_cache, const void* v_cache, int n_heads,
                                              int n_kv_heads, int head_dim, int cache_head_dim, int N, int start_pos, float scale,
                                              int kv_int8, const float* k_scales, const float* v_scales, int window, void* stream);
/* flash_attention_decode_dyn — :380-396, attention.cu:1007-1034.  seq_len = *d_pos + 1. */
int jllm_b200_flash_attention_decode_dyn(void* output, const void* q, const void* k_cache, const void* v_cache, int n_heads,
                                         int n_kv_heads, int head_dim, int cache_head_dim, const int* d_pos, float scale, int kv_int8,
                                         const float* kv_scales, int window, int n_splits, void* stream);
/* decode_attn_splits / get_splitk_partials — :402-403, attention.cu:975-1005. */
int    jllm_b200_decode_attn_splits(int seq_len);
float* jllm_b200_get_splitk_partials(int n_heads, int n_splits, int head_dim);

/* ── memory pools — include/jllm_memory.h:104-222, src/memory/kv_cache.cpp, pool.cpp ──
 * Opaque handles over the C++ classes jllm::KVCachePool / jllm::ScratchPool (same object
 * layout as the reference's, see jllm_b200_api.hpp). */
typedef struct jllm_b200_kv_pool jllm_b200_kv_pool;
typedef struct jllm_b200_scratch jllm_b200_scratch;
jllm_b200_kv_pool* jllm_b200_kv_pool_create(int n_layers, int n_kv_heads, int head_dim, int max_context, int overflow_context, int kv_type_bytes);
void     jllm_b200_kv_pool_destroy(jllm_b200_kv_pool* p);
void*    jllm_b200_kv_pool_key_ptr(jllm_b200_kv_pool* p, int layer, int pos);
void*    jllm_b200_kv_pool_val_ptr(jllm_b200_kv_pool* p, int layer, int pos);
float*   jllm_b200_kv_pool_scale_ptr(jllm_b200_kv_pool* p, int layer, int pos, int is_value);
int64_t  jllm_b200_kv_pool_scales_bytes(jllm_b200_kv_pool* p);
int64_t  jllm_b200_kv_pool_capacity_bytes(jllm_b200_kv_pool* p);
int64_t  jllm_b200_kv_pool_used_bytes(jllm_b200_kv_pool* p);
int64_t  jllm_b200_kv_pool_packed_used_bytes(jllm_b200_kv_pool* p, int used_tokens);
int      jllm_b200_kv_pool_gather_used_to_host(jllm_b200_kv_pool* p, void* host_dst, int used_tokens);
int      jllm_b200_kv_pool_scatter_from_host(jllm_b200_kv_pool* p, const void* host_src, int used_tokens, int zero_remaining);
int      jllm_b200_kv_pool_used_tokens(jllm_b200_kv_pool* p);
void     jllm_b200_kv_pool_clear(jllm_b200_kv_pool* p);
jllm_b200_scratch* jllm_b200_scratch_create(int64_t size_bytes);
void     jllm_b200_scratch_destroy(jllm_b200_scratch* s);
void*    jllm_b200_scratch_get(jllm_b200_scratch* s, int64_t size);
void     jllm_b200_scratch_reset(jllm_b200_scratch* s);
int64_t  jllm_b200_scratch_mark(jllm_b200_scratch* s);
void     jllm_b200_scratch_rewind_to(jllm_b200_scratch* s, int64_t saved);
int64_t  jllm_b200_scratch_used(jllm_b200_scratch* s);
int64_t  jllm_b200_scratch_capacity(jllm_b200_scratch* s);

/* ══ extension entry points (no counterpart in the reference API) ══════════ */
/* Integer accumulators of the dp4a GEMV path for one matrix: dots[M][K/32] (Q4_K: Σ over a
 * 32-element sub-block of q4*q8) or dots[M][K/16] (Q6_K: Σ over a 16-element scale group of
 * (q6-32)*q8), written by the same kernel that produces y (used by the bit-exactness tests). */
int jllm_b200_gemv_quant_int_dots(void* y, int32_t* dots, const void* W, int ggml_type, const void* x, int M, int K, void* stream);
/* Same for the batched GEMM: dots[N][M][K/32] or [N][M][K/16]. */
int jllm_b200_gemm_quant_batched_int_dots(void* y, int32_t* dots, const void* W, int ggml_type, const void* x, int M, int N, int K, void* stream);
/* Two batched products over the same activations (the gate and up projections of a layer): y0[N x M0] = x . W0^T and
 * y1[N x M1] = x . W1^T, equal to two jllm_b200_gemm_quant_batched calls.  With more than 64 tokens (or the large matrices
 * from 49) and both matrices Q4_K or both Q6_K the row tiles of the two share one launch; otherwise two launches, the
 * second reusing the quantised activations.  N >= 2. */
int jllm_b200_gemm_quant_batched_pair(void* y0, const void* W0, int type0, int M0, void* y1, const void* W1, int type1, int M1,
                                      const void* x, int N, int K, void* stream);
/* RMSNorm fused into the shared-activation GEMVs: x := half(x * rrms * w) is formed in shared
 * memory and quantised there, equal to fused_rmsnorm_residual -> gemv_quant_pair / _triple. */
int jllm_b200_norm_gemv_quant_pair(void* y0, const void* W0, int type0, int M0, void* y1, const void* W1, int type1, int M1,
                                   const void* x, const void* norm_weight, int weight_fp32, float eps, int K, void* stream);
int jllm_b200_norm_gemv_quant_triple(void* y0, const void* W0, int type0, int M0, void* y1, const void* W1, int type1, int M1,
                                     void* y2, const void* W2, int type2, int M2, const void* x, const void* norm_weight,
                                     int weight_fp32, float eps, int K, void* stream);
/* gate/up pair with the SwiGLU applied in the epilogue: out[M] = silu(half(Wg.x)) * half(Wu.x). */
int jllm_b200_norm_gemv_pair_swiglu(void* out, const void* Wgate, const void* Wup, int type, int M, const void* x,
                                    const void* norm_weight, int weight_fp32, float eps, int K, void* stream);
/* Per-head RMSNorm of q and k (weights fp32, may be null), RoPE, and int8 quantisation of the new
 * K and V rows into the cache at `position` (or *d_pos) — the five launches of
 * Engine::transformer_layer_attn_compute (src/engine/decode.cu:1443-1478) in one. */
int jllm_b200_qkv_prep_int8(void* q, const void* k, const void* v, const float* q_norm, const float* k_norm, float eps,
                            int8_t* k_cache_layer, int8_t* v_cache_layer, float* k_scales_layer, float* v_scales_layer,
                            int n_heads, int n_kv_heads, int head_dim, int position, const int* d_pos, float theta_base,
                            int neox, void* stream);
/* Ragged batched decode attention: sequence b has its own cache bases and length (device arrays of
 * `batch` entries); q/out are [batch][n_heads][head_dim].  Equals a loop over flash_attention_decode. */
int jllm_b200_flash_attention_decode_batched(void* output, const void* q, const void* const* k_list, const void* const* v_list,
                                             const float* const* ks_list, const float* const* vs_list, const int* seq_lens,
                                             int batch, int max_seq_len, int n_heads, int n_kv_heads, int head_dim, float scale,
                                             int kv_int8, void* stream);

/* Ragged batched decode attention over a FIXED set of INT8 caches (head_dim 128): the plan holds one pair of TMA tensor
 * maps per sequence, built once on the host, so the kernel fetches K/V tiles by 2-D tensor copies as the single-sequence
 * path does.  k_list / v_list / ks_list / vs_list are HOST arrays of `batch` DEVICE pointers (cache bases, 16-byte
 * aligned; fp32 scales [pos][n_kv_heads]); every cache holds max_seq_len positions.  seq_lens is a device array that
 * may change from call to call.  Same result as jllm_b200_flash_attention_decode_batched. */
typedef struct jllm_b200_attn_plan jllm_b200_attn_plan;
jllm_b200_attn_plan* jllm_b200_attn_plan_create(const void* const* k_list, const void* const* v_list, const float* const* ks_list,
                                                const float* const* vs_list, int batch, int max_seq_len, int n_kv_heads, int head_dim);
void jllm_b200_attn_plan_destroy(jllm_b200_attn_plan* plan);
int  jllm_b200_flash_attention_decode_planned(const jllm_b200_attn_plan* plan, void* output, const void* q, const int* seq_lens,
                                              int n_heads, float scale, void* stream);

/* ── decoder session (extension; stands where Engine::decode_step / transformer_layer sit,
 * src/engine/decode.cu:1169-1246, :1437-1530, :2101-2194) ─────────────────────────────
 * Host-side sequencing of the kernels above for a Qwen3/Llama-shaped decoder with INT8 KV:
 * per layer RMSNorm -> Q/K/V GEMV -> QK-norm + RoPE + KV int8 store -> decode attention ->
 * Wo + residual -> RMSNorm -> gate/up GEMV -> SwiGLU -> W_down + residual, then the final norm,
 * fp32 logits and a greedy argmax on the device (lowest index among equal maxima, non-finite
 * logits skipped, as sample_greedy does, src/engine/sample.cpp:160-170).  Position and token
 * live in device memory, so one captured CUDA graph replays for every step. */
typedef struct {
    const void *wq, *wk, *wv, *wo, *w_gate, *w_up, *w_down;     /* K-quant block images (device) */
    int type_wq, type_wk, type_wv, type_wo, type_w_gate, type_w_up, type_w_down;
    const float *rms_attn, *rms_ffn, *q_norm, *k_norm;          /* fp32 norm weights; q_norm/k_norm may be null */
} jllm_b200_layer_desc;
typedef struct {
    int n_layers, hidden_dim, n_heads, n_kv_heads, head_dim, intermediate_dim, vocab_size, max_context;
    float rope_theta, rms_eps;
    int rope_neox;
    const void* tok_embd; int embd_type;
    const void* output;   int output_type;
    const float* output_norm;
    const jllm_b200_layer_desc* layers;                          /* host array of n_layers entries */
} jllm_b200_model_desc;
typedef struct jllm_b200_decoder jllm_b200_decoder;
/* flags: bit 4 = jllm_b200_decoder_generate prefills the prompt in one batched pass (jllm_b200_decoder_prefill) instead of
 * one decode step per prompt token — the reference's default for prompts (its prefill arithmetic differs from the decode
 * arithmetic in the activation quantiser, so the two give slightly different logits);
 * bit 0 = fused kernels (norm+GEMV, SwiGLU epilogue, one QKV-prep launch) instead of the reference's
 * launch-for-launch sequence (both give identical bits); bit 1 = replay a captured CUDA graph per step;
 * bit 3 = with bit 0, run Wo / gate-up / W_down / next Q-K-V as ONE chained launch with grid-wide barriers instead of
 * four launches (same bits; measured slower on B200, where dependent launches overlap per SM, so it is off by default). */
jllm_b200_decoder* jllm_b200_decoder_create(const jllm_b200_model_desc* model, int flags);
void   jllm_b200_decoder_destroy(jllm_b200_decoder* d);
int    jllm_b200_decoder_reset(jllm_b200_decoder* d);
/* Runs one step for `token` at `position`; logits stay on the device (see _logits); returns the status. */
int    jllm_b200_decoder_step(jllm_b200_decoder* d, int token, int position, void* stream);
/* Feeds `n_prompt` host tokens (one decode step each), then generates `n_new` tokens greedily; the
 * generated ids are copied to host_out.  Inputs and outputs cross the host/device boundary inside the call. */
int    jllm_b200_decoder_generate(jllm_b200_decoder* d, const int* host_prompt, int n_prompt, int n_new, int* host_out, void* stream);
/* Batched prompt prefill (stands where Engine::transformer_prefill sits, src/engine/decode.cu:1760-1884): n_tokens >= 2 host
 * token ids at positions start_pos .. start_pos+n_tokens-1 go through every layer together — RMSNorm over rows, batched
 * K-quant products, QK-norm + RoPE + INT8 KV store, query-tiled causal attention, SwiGLU FFN — in chunks of at most
 * 2048 tokens (jllm_b200_decoder_set_prefill_chunk changes that); then the logits of the LAST token and its greedy token
 * are computed on the device.  Afterwards the session stands at position start_pos + n_tokens with that token, so
 * jllm_b200_decoder_step_device continues the stream and jllm_b200_decoder_last_token reads the token.  Enqueues only;
 * not available in a tensor-parallel session. */
int    jllm_b200_decoder_prefill(jllm_b200_decoder* d, const int* host_tokens, int n_tokens, int start_pos, void* stream);
int    jllm_b200_decoder_set_prefill_chunk(jllm_b200_decoder* d, int tokens);
/* One step with the host boundary inside: host_pos_token = {position, token} (pinned host memory recommended) is copied
 * to the device, the step runs, the greedy token is copied to *host_next and the call returns once it has arrived. */
int    jllm_b200_decoder_step_sync(jllm_b200_decoder* d, const int* host_pos_token, int* host_next, void* stream);
/* Enqueues the following step from the position and token the previous step left on the device; no host copy, no wait. */
int    jllm_b200_decoder_step_device(jllm_b200_decoder* d, void* stream);
const float* jllm_b200_decoder_logits(jllm_b200_decoder* d);     /* device pointer, vocab_size floats */
int    jllm_b200_decoder_last_token(jllm_b200_decoder* d, void* stream);   /* argmax of the last step (synchronises) */
int    jllm_b200_decoder_kernels_per_step(jllm_b200_decoder* d);
/* Every step appends its greedy token to a device-side record (cleared by _reset and _generate; it holds max_context + 8
 * entries).  Returns how many tokens have been recorded (-1 on error; synchronises) and copies up to n of them, starting
 * at index `first`, to host_out. */
int    jllm_b200_decoder_recorded_tokens(jllm_b200_decoder* d, int first, int n, int* host_out, void* stream);
/* Internal activation buffers of the last step, for tests: 0 x, 1 x2, 2 q, 3 k, 4 v, 5 attention out, 6 SwiGLU out,
 * 7 layer-0 K cache, 8 layer-0 K scales. */
const void* jllm_b200_decoder_buffer(jllm_b200_decoder* d, int which);

/* ── tensor-parallel decoder session (extension; the reference is single-GPU) ───────────────────────────
 * One process per GPU.  Rank r of `world` (2, 4 or 8) owns rows [r*M/world, (r+1)*M/world) of every weight matrix
 * (a contiguous byte range of the GGUF image) and the KV heads that go with its query heads.  `model` carries the
 * FULL dimensions, the weight pointers are the rank's slices (tok_embd and the norm vectors are whole).  After each
 * sharded product the slices are gathered through the exchange regions: regions[i] is rank i's region as mapped
 * into this process (jllm_b200_tp_alloc on the owner, jllm_b200_tp_export / _open across processes), all of
 * jllm_b200_tp_region_bytes() bytes.  All ranks must run the same steps in the same order; the greedy token is
 * reduced across ranks on the device, so every rank returns the same token.  jllm_b200_decoder_logits() gives the
 * rank's vocab_size/world slice.  Waits between ranks are bounded: a rank that never arrives shows up as
 * JLLM_B200_ERR_TIMEOUT in jllm_b200_device_status().  Create clears this rank's own region (packets of an earlier session
 * must not pass for fresh ones): let every rank return from create before any rank runs a step.  Weight types other than
 * Q4_K / Q6_K are refused (JLLM_B200_ERR_TYPE).  flags: bit 1 = CUDA graph as above. */
jllm_b200_decoder* jllm_b200_decoder_create_tp(const jllm_b200_model_desc* model, int flags, int rank, int world, void* const* regions);
size_t jllm_b200_tp_region_bytes(int hidden_dim, int q_dim, int intermediate_dim);
void*  jllm_b200_tp_alloc(size_t bytes);                    /* zeroed device memory for an exchange region */
int    jllm_b200_tp_free(void* region);
int    jllm_b200_tp_export(void* region, void* handle64);   /* 64-byte CUDA IPC handle */
void*  jllm_b200_tp_open(const void* handle64);             /* maps a peer's region, enabling peer access */
int    jllm_b200_tp_close(void* mapped);

/* ── lock-step batch decoder session (extension) ────────────────────────────────────────────────
 * n_streams independent requests, all at the same position, one token each per step: per layer the n_streams hidden
 * vectors go through the batched kernels above (RMSNorm over rows, jllm_b200_gemm_quant_batched with N = n_streams,
 * per-stream QK-norm + RoPE + INT8 KV store, ragged-batch decode attention, SwiGLU, residual adds), so the weights are
 * read once per step for all streams; greedy argmax per stream on the device.  host_prompts is [n_streams][n_prompt]
 * (equal prompt lengths), host_out receives [n_new][n_streams] token ids. */
typedef struct jllm_b200_batch_decoder jllm_b200_batch_decoder;
jllm_b200_batch_decoder* jllm_b200_batch_decoder_create(const jllm_b200_model_desc* model, int n_streams);
void   jllm_b200_batch_decoder_destroy(jllm_b200_batch_decoder* d);
int    jllm_b200_batch_decoder_generate(jllm_b200_batch_decoder* d, const int* host_prompts, int n_prompt, int n_new, int* host_out, void* stream);
int    jllm_b200_batch_decoder_step_device(jllm_b200_batch_decoder* d, void* stream);   /* one more step from the device-side state */
const void* jllm_b200_batch_decoder_logits(jllm_b200_batch_decoder* d);                /* device, fp16 [n_streams][vocab_size] of the last step */
int    jllm_b200_batch_decoder_kernels_per_step(jllm_b200_batch_decoder* d);

/* ── allocation-free decode attention (no counterpart in the reference) ─────────────────────────
 * For hosts that cannot let the library allocate device memory: an engine whose own pools already hold
 * all of the GPU's free memory, or a request loop that must avoid driver calls which can stall the device.
 * Same arguments and result as jllm_b200_flash_attention_decode;
 * the split-K partials live in a fixed array built into the library (JLLM_B200_NOALLOC_MAX_FLOATS floats
 * per GPU that loads the library, held until the process exits) instead of a buffer grown on demand.
 *   - n_heads * n_slices * (head_dim + 2) must not exceed JLLM_B200_NOALLOC_MAX_FLOATS (n_slices =
 *     ceil(seq_len / max(128, ceil(seq_len / 32)))); larger requests return JLLM_B200_ERR_LIMIT.
 *   - The first call on each device looks up the array's device address; make that call before starting
 *     any stream capture.
 *   - All calls share the array.  Nothing needs clearing between calls (every record read is written first),
 *     but calls that overlap in time on one GPU race on it: keep them on one stream or order them.
 *   - It never calls cudaMalloc / cudaFree or any allocating routine. */
#define JLLM_B200_NOALLOC_MAX_FLOATS (256 * 1024)
int jllm_b200_flash_attention_decode_noalloc(void* output, const void* q, const void* k_cache, const void* v_cache, int n_heads,
                                             int n_kv_heads, int head_dim, int cache_head_dim, int seq_len, float scale, int kv_int8,
                                             const float* k_scales, const float* v_scales, int window, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JLLM_B200_H */
