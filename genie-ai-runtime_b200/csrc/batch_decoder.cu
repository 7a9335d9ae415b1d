// batch_decoder.cu — B independent request streams decoded in lockstep (all at the same position), one token each
// per step: the second workload of the whole-decoder benchmark (64 concurrent streams).
//
// Per layer the B hidden vectors go through the reference's BATCHED kernels: RMSNorm over rows, K-quant GEMMs with
// N = B tokens (gemm_quant_batched, src/kernels/gemv_q4.cu:2478-2495 — the prefill arithmetic, which is what the
// reference uses whenever more than one token is in flight), per-head q/k norm + RoPE + INT8 KV store for every stream,
// ragged-batch decode attention over the B caches, SwiGLU, residual adds; then the final norm, fp16 logits for the B
// rows and a greedy argmax per row on the device.  Weights are read once per step for all streams.
#include "../../include/jllm_b200.h"
#include "../../include/jllm_b200_api.hpp"
#include "common.cuh"
#include "elementwise.cuh"
#include "attention.cuh"
#include "mmq.cuh"
#include "gemv.cuh"
#include <cmath>
#include <new>
#include <vector>

namespace jb {

// greedy argmax of every row of fp16 logits [B][V] (lowest index among equal maxima, non-finite skipped); block b = row b.
// Also records the tokens of this step and, in block 0, advances the shared position.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const __half* logits, int V, int* tokens, int* state, int* out, int out_cap, int B) {
    pdl_wait();
    __shared__ float sv[32]; __shared__ int si[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, b = blockIdx.x;
    const __half* row = logits + (size_t)b * V;
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = tid; i < V; i += blockDim.x) {
        const float v = __half2float(row[i]);
        if (isfinite(v) && (v > best || (v == best && i < bi))) { best = v; bi = i; }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o); const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        if (bi == 0x7FFFFFFF) bi = 0;
        tokens[b] = bi;
        const int k = state[2];                       // steps recorded so far (read by every block before block 0 bumps it: see below)
        if (out && k < out_cap) out[(size_t)k * B + b] = bi;
    }
}
// state[0] = position, state[2] = steps recorded; seq_lens[b] = position + 1 for the attention of the NEXT step
__global__ void batch_advance_kernel(int* state, int* seq_lens, int B) {
    pdl_wait();
    const int p = state[0] + 1;
    if (threadIdx.x == 0) { state[0] = p; state[2] = state[2] + 1; }
    for (int b = threadIdx.x; b < B; b += blockDim.x) seq_lens[b] = p + 1;
}
__global__ void batch_begin_kernel(int* state, int* seq_lens, int* tokens, const int* prompt, int n_prompt, int B) {
    pdl_wait();
    const int p = state[0];
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        seq_lens[b] = p + 1;
        if (prompt && p < n_prompt) tokens[b] = prompt[(size_t)b * n_prompt + p];
    }
}

}  // namespace jb

using namespace jb;

struct jllm_b200_batch_decoder {
    jllm_b200_model_desc m;
    std::vector<jllm_b200_layer_desc> layers;
    std::vector<jllm::KVCachePool> kv;
    int B = 0;
    __half *x = nullptr, *x2 = nullptr, *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *gate = nullptr,
           *up = nullptr, *sw = nullptr, *y = nullptr, *logits = nullptr;
    int *state = nullptr, *tokens = nullptr, *seq_lens = nullptr, *out_tokens = nullptr, *prompt_dev = nullptr;
    int out_cap = 0, prompt_cap = 0;
    void** lists = nullptr;            // device: [layer][4 (k, v, k scales, v scales)][B] pointers
    std::vector<unsigned char> maps;   // host: [layer][B][K, V] TMA tensor maps of the caches (128 bytes each), passed to the kernel as parameters
    void* slab = nullptr;
    int kernels_per_step = 0;
    cudaGraphExec_t graph_exec = nullptr;   // one decode step from the device-side state
    int host_pos = -1;                      // host mirror of the device-side position (-1 until generate has run): the bound of step_device
};

#define BCHK(call) do { const int rc__ = (call); if (rc__) return rc__; } while (0)

static int bdec_enqueue_step(jllm_b200_batch_decoder* d, const int* prompt, int n_prompt, cudaStream_t st) {
    const jllm_b200_model_desc& m = d->m;
    const int B = d->B, H = m.hidden_dim, QD = m.n_heads * m.head_dim, KVD = m.n_kv_heads * m.head_dim, I = m.intermediate_dim, V = m.vocab_size;
    const float scale = 1.0f / sqrtf((float)m.head_dim);
    const long long l0 = jllm_b200_launch_count();
    JB_CUDA(launch_k(batch_begin_kernel, dim3(1), dim3(128), 0, st, pdl_enabled(), d->state, d->seq_lens, d->tokens, prompt, n_prompt, B));
    count_launch();
    BCHK(launch_embed_rows(d->x, m.tok_embd, m.embd_type, d->tokens, B, H, st));
    for (int l = 0; l < m.n_layers; ++l) {
        const jllm_b200_layer_desc& w = d->layers[l];
        void** L = d->lists + (size_t)l * 4 * B;
        BCHK(launch_rmsnorm(d->normed, d->x, nullptr, w.rms_attn, true, B, H, m.rms_eps, st));
        BCHK(launch_mmq(d->q, resolve_weight(w.wq), w.type_wq, d->normed, QD, B, H, nullptr, st));
        BCHK(launch_mmq_ex(d->k, resolve_weight(w.wk), w.type_wk, d->normed, KVD, B, H, nullptr, true, st));      // same activations as Q
        BCHK(launch_mmq_ex(d->v, resolve_weight(w.wv), w.type_wv, d->normed, KVD, B, H, nullptr, true, st));
        BCHK(launch_qkv_prep_batched(d->q, d->k, d->v, w.q_norm, w.k_norm, m.rms_eps, (int8_t* const*)L, (int8_t* const*)(L + B),
                                     (float* const*)(L + 2 * B), (float* const*)(L + 3 * B), B, m.n_heads, m.n_kv_heads, m.head_dim,
                                     d->state, m.rope_theta, m.rope_neox != 0, st));
        AttnCall c;
        c.out = d->att; c.q = d->q; c.k_list = (const void* const*)L; c.v_list = (const void* const*)(L + B);
        c.ks_list = (const float* const*)(L + 2 * B); c.vs_list = (const float* const*)(L + 3 * B); c.seq_lens = d->seq_lens;
        c.tma_maps = d->maps.empty() ? nullptr : d->maps.data() + (size_t)l * B * 2 * 128;
        c.batch = B; c.max_seq = m.max_context; c.n_heads = m.n_heads; c.n_kv = m.n_kv_heads; c.hd = m.head_dim; c.chd = m.head_dim;
        c.scale = scale; c.kv_int8 = 1;
        c.n_splits = 1;      // the step is one captured graph for every position: no slices (the streams of a step are short or many)
        BCHK(launch_attention(c, st));
        BCHK(launch_mmq_ex(d->x2, resolve_weight(w.wo), w.type_wo, d->att, H, B, QD, d->x, false, st));           // + residual
        BCHK(launch_rmsnorm(d->normed, d->x2, nullptr, w.rms_ffn, true, B, H, m.rms_eps, st));
        BCHK(launch_mmq_pair(d->gate, d->up, resolve_weight(w.w_gate), w.type_w_gate, resolve_weight(w.w_up), w.type_w_up, d->normed, I, I, B, H, st));   // one launch where the tensor-core kernel serves both
        BCHK(launch_glu(d->sw, d->gate, d->up, B, I, false, st));
        BCHK(launch_mmq_ex(d->x, resolve_weight(w.w_down), w.type_w_down, d->sw, H, B, I, d->x2, false, st));     // + residual
    }
    BCHK(launch_rmsnorm(d->normed, d->x, nullptr, m.output_norm, true, B, H, m.rms_eps, st));
    BCHK(launch_mmq(d->logits, resolve_weight(m.output), m.output_type, d->normed, V, B, H, nullptr, st));
    JB_CUDA(launch_k(argmax_rows_kernel, dim3(B), dim3(1024), 0, st, pdl_enabled(), (const __half*)d->logits, V, d->tokens, d->state,
                     d->out_tokens, d->out_cap, B));
    count_launch();
    JB_CUDA(launch_k(batch_advance_kernel, dim3(1), dim3(128), 0, st, pdl_enabled(), d->state, d->seq_lens, B));
    count_launch();
    d->kernels_per_step = (int)(jllm_b200_launch_count() - l0);
    return JB_OK;
}

extern "C" {

jllm_b200_batch_decoder* jllm_b200_batch_decoder_create(const jllm_b200_model_desc* model, int n_streams) {
    if (!model || !model->layers || model->n_layers <= 0 || n_streams < 2 || n_streams > 1024) { set_error(JB_ERR_ARG, "batch decoder: bad model description or stream count"); return nullptr; }
    if (model->hidden_dim % QK_K || model->intermediate_dim % QK_K || (model->n_heads * model->head_dim) % QK_K) {
        set_error(JB_ERR_ARG, "batch decoder: hidden/intermediate/q dims must be multiples of 256"); return nullptr;
    }
    if (!ctx()) return nullptr;
    jllm_b200_batch_decoder* d = new (std::nothrow) jllm_b200_batch_decoder();
    if (!d) return nullptr;
    d->m = *model; d->B = n_streams;
    d->layers.assign(model->layers, model->layers + model->n_layers);
    d->m.layers = d->layers.data();
    const int B = n_streams;
    const size_t H = model->hidden_dim, QD = (size_t)model->n_heads * model->head_dim, KVD = (size_t)model->n_kv_heads * model->head_dim,
                 I = model->intermediate_dim, V = model->vocab_size;
    d->kv.resize(B);
    jllm::KVCachePool::Config c = { model->n_layers, model->n_kv_heads, model->head_dim, model->max_context, 0, 1 };
    for (int b = 0; b < B; ++b)
        if (!d->kv[b].init(c) || !d->kv[b].kv_scale_ptr(0, 0, false)) { set_error(JB_ERR_NOMEM, "batch decoder: KV pool %d", b); jllm_b200_batch_decoder_destroy(d); return nullptr; }
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    d->out_cap = model->max_context + 8; d->prompt_cap = model->max_context + 8;
    const size_t total = 4 * al(B * H * 2) + 2 * al(B * QD * 2) + 2 * al(B * KVD * 2) + 3 * al(B * I * 2) + al(B * V * 2) + al(64) + 2 * al((size_t)B * 4) +
                         al((size_t)d->out_cap * B * 4) + al((size_t)d->prompt_cap * B * 4) + al((size_t)model->n_layers * 4 * B * sizeof(void*));
    if (cudaMalloc(&d->slab, total) != cudaSuccess) { cudaGetLastError(); set_error(JB_ERR_NOMEM, "batch decoder: %zu B of activations", total); jllm_b200_batch_decoder_destroy(d); return nullptr; }
    cudaMemset(d->slab, 0, total);
    char* p = (char*)d->slab;
    auto take = [&](size_t b) { char* r = p; p += al(b); return r; };
    d->x = (__half*)take(B * H * 2); d->x2 = (__half*)take(B * H * 2); d->normed = (__half*)take(B * H * 2); d->y = (__half*)take(B * H * 2);
    d->q = (__half*)take(B * QD * 2); d->att = (__half*)take(B * QD * 2);
    d->k = (__half*)take(B * KVD * 2); d->v = (__half*)take(B * KVD * 2);
    d->gate = (__half*)take(B * I * 2); d->up = (__half*)take(B * I * 2); d->sw = (__half*)take(B * I * 2);
    d->logits = (__half*)take(B * V * 2);
    d->state = (int*)take(64); d->tokens = (int*)take((size_t)B * 4); d->seq_lens = (int*)take((size_t)B * 4);
    d->out_tokens = (int*)take((size_t)d->out_cap * B * 4); d->prompt_dev = (int*)take((size_t)d->prompt_cap * B * 4);
    d->lists = (void**)take((size_t)model->n_layers * 4 * B * sizeof(void*));
    std::vector<void*> host((size_t)model->n_layers * 4 * B);
    for (int l = 0; l < model->n_layers; ++l)
        for (int b = 0; b < B; ++b) {
            host[((size_t)l * 4 + 0) * B + b] = d->kv[b].key_ptr(l, 0);
            host[((size_t)l * 4 + 1) * B + b] = d->kv[b].val_ptr(l, 0);
            host[((size_t)l * 4 + 2) * B + b] = d->kv[b].kv_scale_ptr(l, 0, false);
            host[((size_t)l * 4 + 3) * B + b] = d->kv[b].kv_scale_ptr(l, 0, true);
        }
    cudaMemcpy(d->lists, host.data(), host.size() * sizeof(void*), cudaMemcpyHostToDevice);
    if (model->head_dim == 128) {       // tensor maps of every (layer, stream) cache for the TMA attention path
        std::vector<unsigned char> maps((size_t)model->n_layers * B * 2 * 128);
        bool ok = true;
        for (int l = 0; l < model->n_layers && ok; ++l)
            for (int b = 0; b < B && ok; ++b)
                ok = attn_tma_encode(&maps[(((size_t)l * B + b) * 2 + 0) * 128], d->kv[b].key_ptr(l, 0), model->max_context, model->n_kv_heads) &&
                     attn_tma_encode(&maps[(((size_t)l * B + b) * 2 + 1) * 128], d->kv[b].val_ptr(l, 0), model->max_context, model->n_kv_heads);
        if (ok) d->maps.swap(maps);       // else: the general attention kernel serves the pointer lists
    }
    // scratch the kernels would otherwise grow on first use
    size_t need = 0;
    const int Ms[4] = { (int)QD, (int)I, (int)H, (int)V }; const int Ks[4] = { (int)H, (int)H, (int)I, (int)H };
    for (int i = 0; i < 4; ++i) {
        const size_t a = mmq_tc_scratch_bytes(T_Q6K, Ms[i], B, Ks[i]), b2 = mmq_tc_scratch_bytes(T_Q4K, Ms[i], B, Ks[i]), c2 = mmq_scratch_bytes(B, Ks[i]);
        need = a > need ? a : need; need = b2 > need ? b2 : need; need = c2 > need ? c2 : need;
    }
    { const size_t a = mmq_tc_scratch_bytes(T_Q6K, (int)H, B, (int)QD), b2 = mmq_tc_scratch_bytes(T_Q4K, (int)H, B, (int)QD); need = a > need ? a : need; need = b2 > need ? b2 : need; }
    { const size_t a = mmq_tc_scratch_bytes_pair(T_Q6K, (int)I, (int)I, B, (int)H), b2 = mmq_tc_scratch_bytes_pair(T_Q4K, (int)I, (int)I, B, (int)H); need = a > need ? a : need; need = b2 > need ? b2 : need; }
    mmq_scratch(need, true);
    splitk_buffer((size_t)B * model->n_heads * 64 * (model->head_dim + 4), true);
    return d;
}
void jllm_b200_batch_decoder_destroy(jllm_b200_batch_decoder* d) {
    if (!d) return;
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->slab) cudaFree(d->slab);
    for (auto& p : d->kv) p.destroy();
    delete d;
}
int jllm_b200_batch_decoder_generate(jllm_b200_batch_decoder* d, const int* host_prompts, int n_prompt, int n_new, int* host_out, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    const int B = d->B;
    if (n_prompt <= 0 || n_new < 0 || !host_prompts) return set_error(JB_ERR_ARG, "batch decoder: n_prompt=%d n_new=%d", n_prompt, n_new);
    if (n_prompt + n_new > d->m.max_context || n_prompt > d->prompt_cap) return set_error(JB_ERR_LIMIT, "batch decoder: %d tokens exceed the context of %d", n_prompt + n_new, d->m.max_context);
    for (long long i = 0; i < (long long)B * n_prompt; ++i)
        if (host_prompts[i] < 0 || host_prompts[i] >= d->m.vocab_size) return set_error(JB_ERR_ARG, "batch decoder: prompt token %d outside the vocabulary", host_prompts[i]);
    JB_CUDA(cudaMemcpyAsync(d->prompt_dev, host_prompts, (size_t)B * n_prompt * sizeof(int), cudaMemcpyHostToDevice, st));
    JB_CUDA(cudaMemsetAsync(d->state, 0, 64, st));
    for (auto& p : d->kv) p.clear();
    const int total_steps = n_prompt + (n_new > 0 ? n_new - 1 : 0);
    d->host_pos = -1;
    for (int s = 0; s < total_steps; ++s) BCHK(bdec_enqueue_step(d, d->prompt_dev, n_prompt, st));
    d->host_pos = total_steps;              // every step advances the device-side position by one
    if (n_new > 0 && host_out)
        JB_CUDA(cudaMemcpyAsync(host_out, d->out_tokens + (size_t)(n_prompt - 1) * B, (size_t)n_new * B * sizeof(int), cudaMemcpyDeviceToHost, st));
    JB_CUDA(cudaStreamSynchronize(st));
    return jllm_b200_device_status(stream);
}
/* one more step from the device-side state (after generate): no host copy, no wait */
int jllm_b200_batch_decoder_step_device(jllm_b200_batch_decoder* d, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    // The position lives on the device; the host mirror keeps a step from writing K/V rows past the per-stream pools.
    if (d->host_pos < 0) return set_error(JB_ERR_STATE, "batch decoder: step_device before generate");
    if (d->host_pos >= d->m.max_context) return set_error(JB_ERR_LIMIT, "batch decoder: position %d is outside the context of %d", d->host_pos, d->m.max_context);
    ++d->host_pos;
    if (st == nullptr || st == cudaStreamLegacy) return bdec_enqueue_step(d, nullptr, 0, st);   // the default stream cannot be captured
    if (!d->graph_exec) {
        cudaGraph_t g = nullptr;
        JB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = bdec_enqueue_step(d, nullptr, 0, st);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) return cuda_error(e, "cudaStreamEndCapture");
        const cudaError_t ie = cudaGraphInstantiate(&d->graph_exec, g, 0);
        cudaGraphDestroy(g);
        if (ie != cudaSuccess) { d->graph_exec = nullptr; return cuda_error(ie, "cudaGraphInstantiate"); }
    }
    JB_CUDA(cudaGraphLaunch(d->graph_exec, st));
    count_launch(d->kernels_per_step);
    return JB_OK;
}
const void* jllm_b200_batch_decoder_logits(jllm_b200_batch_decoder* d) { return d->logits; }
int jllm_b200_batch_decoder_kernels_per_step(jllm_b200_batch_decoder* d) { return d->kernels_per_step; }

}  // extern "C"
