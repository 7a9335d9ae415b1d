// decoder.cu — host-side sequencing of one decode step (and greedy generation) over the kernel
// API, with the token and the position kept in device memory so that a single captured CUDA
// graph serves every step.  Order of operations follows the reference engine:
// Engine::decode_step (src/engine/decode.cu:2101-2194), transformer_layer (:1169-1246),
// transformer_layer_attn_compute (:1437-1497), attn/ffn exits (:1499-1522).
#include "../../include/jllm_b200.h"
#include "../../include/jllm_b200_api.hpp"
#include "common.cuh"
#include "gemv.cuh"
#include "elementwise.cuh"
#include "attention.cuh"
#include "mmq.cuh"
#include "tp.cuh"
#include <cfloat>
#include <cstdlib>
#include <new>
#include <vector>

namespace jb {

// greedy argmax over fp32 logits; also advances the device-side step state:
// state[0] = position, state[1] = current token, state[2] = number of tokens written to `out`.
// Several CTAs scan slices of the vocabulary; each leaves its best (value, index) in scratch, and the last one to
// finish (atomic ticket, no waiting) reduces them and advances the state.  scratch: [0] ticket, [32..32+G) values,
// [32+G..32+2G) indices, G = gridDim.x <= 64.
__global__ void __launch_bounds__(1024) argmax_advance_kernel(const float* logits, int n, int* state, int* out, int out_cap, unsigned int* scratch) {
    pdl_wait();
    __shared__ float sv[32]; __shared__ int si[32]; __shared__ int last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, G = gridDim.x;
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = blockIdx.x * blockDim.x + tid; i < n; i += G * blockDim.x) {
        const float v = logits[i];
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
        reinterpret_cast<float*>(scratch)[32 + blockIdx.x] = best;
        reinterpret_cast<int*>(scratch)[32 + G + blockIdx.x] = bi;
        __threadfence();
        last = atomicAdd(scratch, 1u) == (unsigned)G - 1;
    }
    __syncthreads();
    if (!last || tid != 0) return;
    __threadfence();
    scratch[0] = 0u;
    best = -INFINITY; bi = 0x7FFFFFFF;
    for (int g = 0; g < G; ++g) {
        const float v = reinterpret_cast<volatile float*>(scratch)[32 + g]; const int i = reinterpret_cast<volatile int*>(scratch)[32 + G + g];
        if (i != 0x7FFFFFFF && (v > best || (v == best && i < bi))) { best = v; bi = i; }
    }
    if (bi == 0x7FFFFFFF) bi = 0;
    const int k = state[2];
    if (out && k < out_cap) out[k] = bi;
    state[2] = k + 1;
    state[1] = bi;
    state[0] = state[0] + 1;
}

__global__ void set_state_kernel(int* state, int pos, int token) {
    pdl_wait();
    if (threadIdx.x == 0) { state[0] = pos; state[1] = token; }
}
// prompt feeding inside a graph: token for this step comes from a device list
__global__ void next_prompt_kernel(int* state, const int* prompt, int idx_base) {
    pdl_wait();
    if (threadIdx.x == 0) { const int p = state[0]; state[1] = prompt[p - idx_base]; }
}

}  // namespace jb

using namespace jb;

struct jllm_b200_decoder {
    jllm_b200_model_desc m;
    std::vector<jllm_b200_layer_desc> layers;
    jllm::KVCachePool kv;
    bool fused = true, use_graph = false, chain = false;
    __half *x = nullptr, *x2 = nullptr, *normed = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *gate = nullptr, *up = nullptr, *sw = nullptr;
    float* logits = nullptr;
    int* state = nullptr;       // [pos, token, n_out]
    int* out_tokens = nullptr; int out_cap = 0;
    int* prompt_dev = nullptr; int prompt_cap = 0;
    cudaGraphExec_t graph_exec = nullptr; int graph_splits = 0;
    int host_pos = 0;                    // host mirror of the device-side position (next step's position)
    cudaStream_t own_stream = nullptr;   // used when the caller passes the legacy default stream, which cannot be captured
    int kernels_per_step = 0;
    void* slab = nullptr;
    // tensor-parallel session: m keeps the full dimensions, the weights are this rank's row slices
    bool tp_on = false, tp_fused = true;
    TpDev tp;
    int tp_off[6] = {0, 0, 0, 0, 0, 0};
    int nh_l = 0, nkv_l = 0, I_l = 0, H_l = 0, V_l = 0;
    uint32_t* seq = nullptr;
    // batched prompt prefill (flag bit 4): activations of up to pf_cap prompt tokens, allocated on first use
    bool batched_prefill = false;
    void* pf_slab = nullptr; int pf_cap = 0, pf_chunk = 2048;
    __half *pf_x = nullptr, *pf_x2 = nullptr, *pf_normed = nullptr, *pf_y = nullptr, *pf_q = nullptr, *pf_att = nullptr, *pf_k = nullptr,
           *pf_v = nullptr, *pf_gate = nullptr, *pf_up = nullptr, *pf_sw = nullptr;
    int* pf_tokens = nullptr;
};

static int dec_alloc(jllm_b200_decoder* d) {
    const jllm_b200_model_desc& m = d->m;
    // (a tensor-parallel rank could do with slice-sized buffers; the full sizes are a few hundred KB)
    const size_t H = m.hidden_dim, QD = (size_t)m.n_heads * m.head_dim, KVD = (size_t)m.n_kv_heads * m.head_dim, I = m.intermediate_dim;
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t total = 3 * al(H * 2) + 2 * al(QD * 2) + 2 * al(KVD * 2) + 3 * al(I * 2) + al((size_t)m.vocab_size * 4) + al(1024) +
                         al((size_t)(m.max_context + 8) * 4) * 2;
    if (cudaMalloc(&d->slab, total) != cudaSuccess) { cudaGetLastError(); return set_error(JB_ERR_NOMEM, "decoder: %zu B of activations", total); }
    cudaMemset(d->slab, 0, total);
    char* p = (char*)d->slab;
    auto take = [&](size_t b) { char* r = p; p += al(b); return r; };
    d->x = (__half*)take(H * 2); d->x2 = (__half*)take(H * 2); d->normed = (__half*)take(H * 2);
    d->q = (__half*)take(QD * 2); d->att = (__half*)take(QD * 2);
    d->k = (__half*)take(KVD * 2); d->v = (__half*)take(KVD * 2);
    d->gate = (__half*)take(I * 2); d->up = (__half*)take(I * 2); d->sw = (__half*)take(I * 2);
    d->logits = (float*)take((size_t)m.vocab_size * 4);
    d->state = (int*)take(1024);        // [0..3] step state, [32..] argmax scratch
    d->out_cap = m.max_context + 8; d->out_tokens = (int*)take((size_t)d->out_cap * 4);
    d->prompt_cap = m.max_context + 8; d->prompt_dev = (int*)take((size_t)d->prompt_cap * 4);
    return JB_OK;
}

#define DCHK(call) do { const int rc__ = (call); if (rc__) return rc__; } while (0)

// Enqueues one decode step that reads position and token from d->state.  n_splits is fixed per
// enqueue (a captured graph keeps the value it was captured with).
static int dec_enqueue_step_tp(jllm_b200_decoder* d, int n_splits, cudaStream_t st);
static int dec_enqueue_step(jllm_b200_decoder* d, int n_splits, cudaStream_t st) {
    if (d->tp_on) return dec_enqueue_step_tp(d, n_splits, st);
    const jllm_b200_model_desc& m = d->m;
    const int H = m.hidden_dim, QD = m.n_heads * m.head_dim, KVD = m.n_kv_heads * m.head_dim, I = m.intermediate_dim;
    const int* d_pos = d->state; const int* d_tok = d->state + 1;
    const float scale = 1.0f / sqrtf((float)m.head_dim);
    const long long l0 = jllm_b200_launch_count();
    DCHK(launch_embed_row(d->x, m.tok_embd, m.embd_type, 0, d_tok, H, st));
    if (d->fused && d->chain) {
        // Q/K/V of layer 0 alone, then per layer: QKV prep, attention, and ONE chained launch for Wo + residual ->
        // norm + gate/up + SwiGLU -> W_down + residual -> norm + Q/K/V of the next layer
        auto triple_args = [&](int l) {
            const jllm_b200_layer_desc& w = d->layers[l];
            GemvArgs a;
            a.nseg = 3;
            a.seg[0] = GemvSeg{ resolve_weight(w.wq), d->q, QD, w.type_wq };
            a.seg[1] = GemvSeg{ resolve_weight(w.wk), d->k, KVD, w.type_wk };
            a.seg[2] = GemvSeg{ resolve_weight(w.wv), d->v, KVD, w.type_wv };
            a.x = d->x; a.K = H; a.xmode = triple_dp4a(w.type_wq, w.type_wk, w.type_wv) ? 0 : 1; a.out_mode = 0;
            a.do_norm = 1; a.norm_w = w.rms_attn; a.norm_w_fp32 = 1; a.eps = m.rms_eps;
            return a;
        };
        { const GemvArgs a0 = triple_args(0); DCHK(launch_gemv(a0, st)); }
        for (int l = 0; l < m.n_layers; ++l) {
            const jllm_b200_layer_desc& w = d->layers[l];
            int8_t* kc = (int8_t*)d->kv.key_ptr(l, 0); int8_t* vc = (int8_t*)d->kv.val_ptr(l, 0);
            float* ks = d->kv.kv_scale_ptr(l, 0, false); float* vs = d->kv.kv_scale_ptr(l, 0, true);
            DCHK(launch_qkv_prep(d->q, d->k, d->v, w.q_norm, w.k_norm, m.rms_eps, kc, vc, ks, vs, m.n_heads, m.n_kv_heads, m.head_dim,
                                 0, d_pos, m.rope_theta, m.rope_neox != 0, true, st));
            AttnCall c;
            c.out = d->att; c.q = d->q; c.k = kc; c.v = vc; c.ks = ks; c.vs = vs; c.n_heads = m.n_heads; c.n_kv = m.n_kv_heads;
            c.hd = m.head_dim; c.chd = m.head_dim; c.d_pos = d_pos; c.scale = scale; c.kv_int8 = 1; c.n_splits = n_splits; c.max_seq = m.max_context;
            DCHK(launch_attention(c, st));
            GemvArgs ph[4];
            int n = 0;
            ph[n].nseg = 1; ph[n].seg[0] = GemvSeg{ resolve_weight(w.wo), d->x2, H, w.type_wo };
            ph[n].x = d->att; ph[n].K = QD; ph[n].xmode = 1; ph[n].out_mode = 2; ph[n].residual = d->x; ++n;
            ph[n].nseg = 2; ph[n].seg[0] = GemvSeg{ resolve_weight(w.w_gate), d->sw, I, w.type_w_gate };
            ph[n].seg[1] = GemvSeg{ resolve_weight(w.w_up), d->sw, I, w.type_w_up };
            ph[n].x = d->x2; ph[n].K = H; ph[n].xmode = (w.type_w_gate == T_Q4K && w.type_w_up == T_Q4K) ? 0 : 1; ph[n].out_mode = 3;
            ph[n].do_norm = 1; ph[n].norm_w = w.rms_ffn; ph[n].norm_w_fp32 = 1; ph[n].eps = m.rms_eps; ++n;
            ph[n].nseg = 1; ph[n].seg[0] = GemvSeg{ resolve_weight(w.w_down), d->x, H, w.type_w_down };
            ph[n].x = d->sw; ph[n].K = I; ph[n].xmode = 1; ph[n].out_mode = 2; ph[n].residual = d->x2; ++n;
            if (l + 1 < m.n_layers) ph[n++] = triple_args(l + 1);
            DCHK(launch_gemv_chain(ph, n, (unsigned int*)(d->state + 200), st));
        }
    } else
    for (int l = 0; l < m.n_layers; ++l) {
        const jllm_b200_layer_desc& w = d->layers[l];
        int8_t* kc = (int8_t*)d->kv.key_ptr(l, 0); int8_t* vc = (int8_t*)d->kv.val_ptr(l, 0);
        float* ks = d->kv.kv_scale_ptr(l, 0, false); float* vs = d->kv.kv_scale_ptr(l, 0, true);
        if (d->fused) {
            DCHK(jllm_b200_norm_gemv_quant_triple(d->q, w.wq, w.type_wq, QD, d->k, w.wk, w.type_wk, KVD, d->v, w.wv, w.type_wv, KVD,
                                                  d->x, w.rms_attn, 1, m.rms_eps, H, st));
            DCHK(launch_qkv_prep(d->q, d->k, d->v, w.q_norm, w.k_norm, m.rms_eps, kc, vc, ks, vs, m.n_heads, m.n_kv_heads, m.head_dim,
                                 0, d_pos, m.rope_theta, m.rope_neox != 0, true, st));
        } else {
            DCHK(launch_rmsnorm(d->normed, d->x, nullptr, w.rms_attn, true, 1, H, m.rms_eps, st));
            DCHK(jllm_b200_gemv_quant_triple(d->q, w.wq, w.type_wq, QD, d->k, w.wk, w.type_wk, KVD, d->v, w.wv, w.type_wv, KVD, d->normed, H, st));
            if (w.q_norm && w.k_norm) {
                DCHK(launch_rmsnorm(d->q, d->q, nullptr, w.q_norm, true, m.n_heads, m.head_dim, m.rms_eps, st));
                DCHK(launch_rmsnorm(d->k, d->k, nullptr, w.k_norm, true, m.n_kv_heads, m.head_dim, m.rms_eps, st));
            }
            DCHK(launch_rope(d->q, d->k, nullptr, nullptr, nullptr, m.n_heads, m.n_kv_heads, m.head_dim, m.head_dim, 0, d_pos, m.rope_theta,
                             m.rope_neox != 0, 1, 0, 0, 0, false, st));
            // K/V rows of this step: one absmax scale per kv head, written at *d_pos (fp16_to_int8 arithmetic;
            // norms and rotation are already applied, so the prep kernel only quantises)
            DCHK(launch_qkv_prep(d->q, d->k, d->v, nullptr, nullptr, m.rms_eps, kc, vc, ks, vs, 0, m.n_kv_heads, m.head_dim, 0, d_pos,
                                 m.rope_theta, m.rope_neox != 0, false, st));
        }
        AttnCall c;
        c.out = d->att; c.q = d->q; c.k = kc; c.v = vc; c.ks = ks; c.vs = vs; c.n_heads = m.n_heads; c.n_kv = m.n_kv_heads;
        c.hd = m.head_dim; c.chd = m.head_dim; c.d_pos = d_pos; c.scale = scale; c.kv_int8 = 1; c.n_splits = n_splits; c.max_seq = m.max_context;
        DCHK(launch_attention(c, st));
        DCHK(jllm_b200_gemv_quant_add(d->x2, w.wo, w.type_wo, d->att, d->x, H, QD, st));
        if (d->fused) {
            DCHK(jllm_b200_norm_gemv_pair_swiglu(d->sw, w.w_gate, w.w_up, w.type_w_gate, I, d->x2, w.rms_ffn, 1, m.rms_eps, H, st));
        } else {
            DCHK(launch_rmsnorm(d->normed, d->x2, nullptr, w.rms_ffn, true, 1, H, m.rms_eps, st));
            DCHK(jllm_b200_gemv_quant_pair(d->gate, w.w_gate, w.type_w_gate, I, d->up, w.w_up, w.type_w_up, I, d->normed, H, st));
            DCHK(launch_glu(d->sw, d->gate, d->up, 1, I, false, st));
        }
        DCHK(jllm_b200_gemv_quant_add(d->x, w.w_down, w.type_w_down, d->sw, d->x2, H, I, st));
    }
    DCHK(launch_rmsnorm(d->normed, d->x, nullptr, m.output_norm, true, 1, H, m.rms_eps, st));
    DCHK(jllm_b200_gemv_quant_f32(d->logits, m.output, m.output_type, d->normed, m.vocab_size, H, st));
    const int ag = m.vocab_size >= 64 * 1024 ? 64 : (m.vocab_size + 1023) / 1024;
    JB_CUDA(launch_k(argmax_advance_kernel, dim3(ag), dim3(1024), 0, st, pdl_enabled(), (const float*)d->logits, m.vocab_size, d->state,
                     d->out_tokens, d->out_cap, (unsigned int*)(d->state + 32)));
    count_launch();
    d->kernels_per_step = (int)(jllm_b200_launch_count() - l0);
    return JB_OK;
}


// One decode step of a tensor-parallel rank: the single-GPU sequence on this rank's rows and heads.  The Wo, gate/up
// and W_down kernels send every finished row as a packet to all ranks from their epilogue, the attention output goes
// out through one small push kernel, and each consuming GEMV polls the packets of its own region while it stages
// its activation vector (after its weight prefetch is under way), so an exchange costs one one-way NVLink trip and,
// but for the attention output, no launch.  Plain fp16 copies of this rank's own slices stay local for the residuals.
static int dec_enqueue_step_tp(jllm_b200_decoder* d, int n_splits, cudaStream_t st) {
    const jllm_b200_model_desc& m = d->m;
    const int H = m.hidden_dim, QD = m.n_heads * m.head_dim, I = m.intermediate_dim, hd = m.head_dim;
    const int QD_l = d->nh_l * hd, KVD_l = d->nkv_l * hd, rank = d->tp.rank, world = d->tp.world;
    unsigned char* mine = d->tp.peer[rank];
    const __half* att_pk = (const __half*)(mine + d->tp_off[0]); const __half* x2_pk = (const __half*)(mine + d->tp_off[1]);
    const __half* sw_pk = (const __half*)(mine + d->tp_off[2]);  const __half* x_pk = (const __half*)(mine + d->tp_off[3]);
    const int* d_pos = d->state; const int* d_tok = d->state + 1;
    const float scale = 1.0f / sqrtf((float)hd);
    const long long l0 = jllm_b200_launch_count();
    auto wait_hook = [&](int layer) { GemvTpWait w; w.seq = d->seq; w.epochs_per_step = m.n_layers; w.layer = layer; return w; };
    auto push_hook = [&](int point, int layer, int rows_local) {
        GemvTpPush q;
        for (int r = 0; r < 8; ++r) q.peer[r] = r < world ? d->tp.peer[r] : nullptr;
        q.world = world; q.buf_off = d->tp_off[point]; q.row_off = rank * rows_local;
        q.seq = d->seq; q.epochs_per_step = m.n_layers; q.layer = layer;
        return q;
    };
    // d->normed holds the plain full x of layer 0 (the embedding row, computed by every rank); d->x / d->x2 hold this
    // rank's own slices of x / x2
    DCHK(launch_embed_row(d->normed, m.tok_embd, m.embd_type, 0, d_tok, H, st));
    for (int l = 0; l < m.n_layers; ++l) {
        const jllm_b200_layer_desc& w = d->layers[l];
        int8_t* kc = (int8_t*)d->kv.key_ptr(l, 0); int8_t* vc = (int8_t*)d->kv.val_ptr(l, 0);
        float* ks = d->kv.kv_scale_ptr(l, 0, false); float* vs = d->kv.kv_scale_ptr(l, 0, true);
        auto triple_args = [&](int ll, const GemvTpWait* wh) {
            const jllm_b200_layer_desc& ww = d->layers[ll];
            GemvArgs a;
            a.nseg = 3;
            a.seg[0] = GemvSeg{ resolve_weight(ww.wq), d->q, QD_l, ww.type_wq };
            a.seg[1] = GemvSeg{ resolve_weight(ww.wk), d->k, KVD_l, ww.type_wk };
            a.seg[2] = GemvSeg{ resolve_weight(ww.wv), d->v, KVD_l, ww.type_wv };
            a.x = ll > 0 ? x_pk : d->normed; a.K = H; a.xmode = triple_dp4a(ww.type_wq, ww.type_wk, ww.type_wv) ? 0 : 1; a.out_mode = 0;
            a.do_norm = 1; a.norm_w = ww.rms_attn; a.norm_w_fp32 = 1; a.eps = m.rms_eps;
            a.tp_wait = ll > 0 ? wh : nullptr;
            return a;
        };
        int rc = 0;
        if (l == 0 || !d->chain) {
            const GemvTpWait wh = wait_hook(l - 1);
            const GemvArgs a0 = triple_args(l, &wh);
            DCHK(launch_gemv(a0, st));
        }
        DCHK(launch_qkv_prep(d->q, d->k, d->v, w.q_norm, w.k_norm, m.rms_eps, kc, vc, ks, vs, d->nh_l, d->nkv_l, hd,
                             0, d_pos, m.rope_theta, m.rope_neox != 0, true, st));
        AttnCall c;
        c.out = d->att; c.q = d->q; c.k = kc; c.v = vc; c.ks = ks; c.vs = vs; c.n_heads = d->nh_l; c.n_kv = d->nkv_l;
        c.hd = hd; c.chd = hd; c.d_pos = d_pos; c.scale = scale; c.kv_int8 = 1; c.n_splits = n_splits; c.max_seq = m.max_context;
        DCHK(launch_attention(c, st));
        DCHK(launch_tp_push(d->tp, d->att, QD_l, d->tp_off[0], rank * QD_l, l, st));
        if (d->chain) {
            // Wo -> gate/up -> W_down -> next layer's Q/K/V in one launch; no grid barrier: every input of a later phase
            // (activation vector and residual rows) is read as packets, which carry their own arrival mark
            const GemvTpWait wh = wait_hook(l);
            const GemvTpPush p_x2 = push_hook(TP_POINT_X2, l, d->H_l), p_sw = push_hook(TP_POINT_SW, l, d->I_l), p_x = push_hook(TP_POINT_X, l, d->H_l);
            GemvArgs ph[4];
            int n = 0;
            ph[n].nseg = 1; ph[n].seg[0] = GemvSeg{ resolve_weight(w.wo), d->x2, d->H_l, w.type_wo };
            ph[n].x = att_pk; ph[n].K = QD; ph[n].xmode = 1; ph[n].out_mode = 2;
            ph[n].residual = l > 0 ? d->x : d->normed + (size_t)rank * d->H_l; ph[n].tp_wait = &wh; ph[n].tp_push = &p_x2; ++n;
            ph[n].nseg = 2; ph[n].seg[0] = GemvSeg{ resolve_weight(w.w_gate), d->sw, d->I_l, w.type_w_gate };
            ph[n].seg[1] = GemvSeg{ resolve_weight(w.w_up), d->sw, d->I_l, w.type_w_up };
            ph[n].x = x2_pk; ph[n].K = H; ph[n].xmode = (w.type_w_gate == T_Q4K && w.type_w_up == T_Q4K) ? 0 : 1; ph[n].out_mode = 3;
            ph[n].do_norm = 1; ph[n].norm_w = w.rms_ffn; ph[n].norm_w_fp32 = 1; ph[n].eps = m.rms_eps; ph[n].tp_wait = &wh; ph[n].tp_push = &p_sw; ++n;
            ph[n].nseg = 1; ph[n].seg[0] = GemvSeg{ resolve_weight(w.w_down), d->x, d->H_l, w.type_w_down };
            ph[n].x = sw_pk; ph[n].K = I; ph[n].xmode = 1; ph[n].out_mode = 2;
            ph[n].residual_pk = reinterpret_cast<const uint2*>(x2_pk) + (size_t)rank * d->H_l; ph[n].tp_wait = &wh; ph[n].tp_push = &p_x; ++n;
            if (l + 1 < m.n_layers) ph[n++] = triple_args(l + 1, &wh);
            DCHK(launch_gemv_chain(ph, n, nullptr, st));
            continue;
        }
        {
            const GemvTpWait wh = wait_hook(l); const GemvTpPush ph = push_hook(TP_POINT_X2, l, d->H_l);
            gemv_set_tp_hooks(&wh, &ph);
            const __half* resid = l > 0 ? d->x : d->normed + (size_t)rank * d->H_l;
            rc = jllm_b200_gemv_quant_add(d->x2, w.wo, w.type_wo, att_pk, resid, d->H_l, QD, st);
            gemv_set_tp_hooks(nullptr, nullptr);
            DCHK(rc);
        }
        {
            const GemvTpWait wh = wait_hook(l); const GemvTpPush ph = push_hook(TP_POINT_SW, l, d->I_l);
            gemv_set_tp_hooks(&wh, &ph);
            rc = jllm_b200_norm_gemv_pair_swiglu(d->sw, w.w_gate, w.w_up, w.type_w_gate, d->I_l, x2_pk, w.rms_ffn, 1, m.rms_eps, H, st);
            gemv_set_tp_hooks(nullptr, nullptr);
            DCHK(rc);
        }
        {
            const GemvTpWait wh = wait_hook(l); const GemvTpPush ph = push_hook(TP_POINT_X, l, d->H_l);
            gemv_set_tp_hooks(&wh, &ph);
            rc = jllm_b200_gemv_quant_add(d->x, w.w_down, w.type_w_down, sw_pk, d->x2, d->H_l, I, st);
            gemv_set_tp_hooks(nullptr, nullptr);
            DCHK(rc);
        }
    }
    DCHK(launch_tp_unpack(d->tp, d->gate, H, d->tp_off[3], m.n_layers - 1, st));          // d->gate: free scratch of at least H halves
    DCHK(launch_rmsnorm(d->normed, d->gate, nullptr, m.output_norm, true, 1, H, m.rms_eps, st));
    DCHK(jllm_b200_gemv_quant_f32(d->logits, m.output, m.output_type, d->normed, d->V_l, H, st));
    DCHK(launch_tp_argmax(d->tp, d->logits, d->V_l, d->state, d->out_tokens, d->out_cap, st));
    d->kernels_per_step = (int)(jllm_b200_launch_count() - l0);
    return JB_OK;
}

static int splits_for_ctx(const jllm_b200_decoder* d, int upto_pos) { return attn_splits_for(upto_pos + 1); }

// graph of one step; re-captured when the split count of the attention changes
static int dec_graph_for(jllm_b200_decoder* d, int n_splits, cudaStream_t st) {
    if (d->graph_exec && d->graph_splits == n_splits) return JB_OK;
    if (d->graph_exec) { cudaGraphExecDestroy(d->graph_exec); d->graph_exec = nullptr; }
    cudaGraph_t g = nullptr;
    JB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    const int rc = dec_enqueue_step(d, n_splits, st);
    const cudaError_t e = cudaStreamEndCapture(st, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return cuda_error(e, "cudaStreamEndCapture");
    const cudaError_t ie = cudaGraphInstantiate(&d->graph_exec, g, 0);
    cudaGraphDestroy(g);
    if (ie != cudaSuccess) { d->graph_exec = nullptr; return cuda_error(ie, "cudaGraphInstantiate"); }
    d->graph_splits = n_splits;
    return JB_OK;
}

// ── batched prompt prefill: the reference's Engine::transformer_prefill (src/engine/decode.cu:1760-1884) for a chunk of
// N >= 2 prompt tokens at positions start .. start+N-1: RMSNorm over rows, batched K-quant products (prefill arithmetic),
// QK-norm + RoPE + INT8 KV store for all tokens in one launch, query-tiled causal attention, Wo, residual, RMSNorm,
// gate/up, SwiGLU, W_down, residual.  After the last chunk: final norm and logits of the last token only, greedy token.
static int dec_prefill_alloc(jllm_b200_decoder* d, int cap) {
    if (cap <= d->pf_cap) return JB_OK;
    if (d->pf_slab) { cudaFree(d->pf_slab); d->pf_slab = nullptr; d->pf_cap = 0; }
    const jllm_b200_model_desc& m = d->m;
    const size_t N = (size_t)cap, H = m.hidden_dim, QD = (size_t)m.n_heads * m.head_dim, KVD = (size_t)m.n_kv_heads * m.head_dim, I = m.intermediate_dim;
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const size_t total = 4 * al(N * H * 2) + 2 * al(N * QD * 2) + 2 * al(N * KVD * 2) + 3 * al(N * I * 2) + al(N * 4);
    if (cudaMalloc(&d->pf_slab, total) != cudaSuccess) { cudaGetLastError(); return set_error(JB_ERR_NOMEM, "decoder: %zu B of prefill activations", total); }
    char* p = (char*)d->pf_slab;
    auto take = [&](size_t b) { char* r = p; p += al(b); return r; };
    d->pf_x = (__half*)take(N * H * 2); d->pf_x2 = (__half*)take(N * H * 2); d->pf_normed = (__half*)take(N * H * 2); d->pf_y = (__half*)take(N * H * 2);
    d->pf_q = (__half*)take(N * QD * 2); d->pf_att = (__half*)take(N * QD * 2);
    d->pf_k = (__half*)take(N * KVD * 2); d->pf_v = (__half*)take(N * KVD * 2);
    d->pf_gate = (__half*)take(N * I * 2); d->pf_up = (__half*)take(N * I * 2); d->pf_sw = (__half*)take(N * I * 2);
    d->pf_tokens = (int*)take(N * 4);
    d->pf_cap = cap;
    return JB_OK;
}

static int dec_prefill_chunk(jllm_b200_decoder* d, const int* dev_tokens, int N, int start, cudaStream_t st) {
    const jllm_b200_model_desc& m = d->m;
    const int H = m.hidden_dim, QD = m.n_heads * m.head_dim, KVD = m.n_kv_heads * m.head_dim, I = m.intermediate_dim;
    const float scale = 1.0f / sqrtf((float)m.head_dim);
    DCHK(launch_embed_rows(d->pf_x, m.tok_embd, m.embd_type, dev_tokens, N, H, st));
    for (int l = 0; l < m.n_layers; ++l) {
        const jllm_b200_layer_desc& w = d->layers[l];
        int8_t* kc = (int8_t*)d->kv.key_ptr(l, 0); int8_t* vc = (int8_t*)d->kv.val_ptr(l, 0);
        float* ks = d->kv.kv_scale_ptr(l, 0, false); float* vs = d->kv.kv_scale_ptr(l, 0, true);
        DCHK(launch_rmsnorm(d->pf_normed, d->pf_x, nullptr, w.rms_attn, true, N, H, m.rms_eps, st));
        DCHK(launch_mmq(d->pf_q, resolve_weight(w.wq), w.type_wq, d->pf_normed, QD, N, H, nullptr, st));
        DCHK(launch_mmq_ex(d->pf_k, resolve_weight(w.wk), w.type_wk, d->pf_normed, KVD, N, H, nullptr, true, st));      // the operand of the product before
        DCHK(launch_mmq_ex(d->pf_v, resolve_weight(w.wv), w.type_wv, d->pf_normed, KVD, N, H, nullptr, true, st));      // the operand of the product before
        DCHK(launch_qkv_prep_tokens(d->pf_q, d->pf_k, d->pf_v, w.q_norm, w.k_norm, m.rms_eps, kc, vc, ks, vs, N, m.n_heads, m.n_kv_heads,
                                    m.head_dim, start, m.rope_theta, m.rope_neox != 0, st));
        AttnCall c;
        c.out = d->pf_att; c.q = d->pf_q; c.k = kc; c.v = vc; c.ks = ks; c.vs = vs; c.n_heads = m.n_heads; c.n_kv = m.n_kv_heads;
        c.hd = m.head_dim; c.chd = m.head_dim; c.scale = scale; c.kv_int8 = 1; c.causal_start = start; c.batch = N; c.n_splits = 1;
        DCHK(attention_prefill_fast_applies(c) ? launch_attention_prefill_fast(c, st) : launch_attention_general(c, st));
        DCHK(launch_mmq(d->pf_y, resolve_weight(w.wo), w.type_wo, d->pf_att, H, N, QD, nullptr, st));
        DCHK(launch_add_half(d->pf_x2, d->pf_x, d->pf_y, (long long)N * H, st));
        DCHK(launch_rmsnorm(d->pf_normed, d->pf_x2, nullptr, w.rms_ffn, true, N, H, m.rms_eps, st));
        DCHK(launch_mmq_pair(d->pf_gate, d->pf_up, resolve_weight(w.w_gate), w.type_w_gate, resolve_weight(w.w_up), w.type_w_up, d->pf_normed, I, I, N, H, st));
        DCHK(launch_glu(d->pf_sw, d->pf_gate, d->pf_up, N, I, false, st));
        DCHK(launch_mmq(d->pf_y, resolve_weight(w.w_down), w.type_w_down, d->pf_sw, H, N, I, nullptr, st));
        DCHK(launch_add_half(d->pf_x, d->pf_x2, d->pf_y, (long long)N * H, st));
    }
    return JB_OK;
}

extern "C" {

jllm_b200_decoder* jllm_b200_decoder_create(const jllm_b200_model_desc* model, int flags) {
    if (!model || !model->layers || model->n_layers <= 0) { set_error(JB_ERR_ARG, "decoder: empty model description"); return nullptr; }
    if (model->hidden_dim % QK_K || model->intermediate_dim % QK_K || (model->n_heads * model->head_dim) % QK_K) {
        set_error(JB_ERR_ARG, "decoder: hidden/intermediate/q dims must be multiples of 256"); return nullptr;
    }
    if (!ctx()) return nullptr;
    jllm_b200_decoder* d = new (std::nothrow) jllm_b200_decoder();
    if (!d) return nullptr;
    d->m = *model;
    d->layers.assign(model->layers, model->layers + model->n_layers);
    d->m.layers = d->layers.data();
    d->fused = (flags & 1) != 0; d->use_graph = (flags & 2) != 0; d->chain = (flags & 8) != 0; d->batched_prefill = (flags & 16) != 0;
    jllm::KVCachePool::Config c = { model->n_layers, model->n_kv_heads, model->head_dim, model->max_context, 0, 1 };
    if (!d->kv.init(c) || !d->kv.kv_scale_ptr(0, 0, false)) { set_error(JB_ERR_NOMEM, "decoder: KV pool allocation failed"); d->kv.destroy(); delete d; return nullptr; }
    if (dec_alloc(d)) { d->kv.destroy(); delete d; return nullptr; }
    // scratch that must exist before any graph capture
    splitk_buffer((size_t)model->n_heads * 64 * (model->head_dim + 4), true);
    return d;
}

jllm_b200_decoder* jllm_b200_decoder_create_tp(const jllm_b200_model_desc* model, int flags, int rank, int world, void* const* regions) {
    if (!model || !model->layers || model->n_layers <= 0 || !regions) { set_error(JB_ERR_ARG, "decoder: empty model description"); return nullptr; }
    if (world < 2 || world > TP_MAX_WORLD || rank < 0 || rank >= world) { set_error(JB_ERR_ARG, "decoder: rank %d of %d", rank, world); return nullptr; }
    const int hd = model->head_dim;
    if (model->n_heads % world || model->n_kv_heads % world || model->intermediate_dim % world || model->hidden_dim % world || model->vocab_size % world ||
        ((model->n_heads / world) * hd * 2) % 16 || ((model->hidden_dim / world) * 2) % 16 || ((model->intermediate_dim / world) * 2) % 16) {
        set_error(JB_ERR_ARG, "decoder: heads, hidden, intermediate and vocabulary sizes must split evenly over %d ranks in 16-byte slices", world); return nullptr;
    }
    if (model->hidden_dim % QK_K || model->intermediate_dim % QK_K || (model->n_heads * hd) % QK_K || model->intermediate_dim < model->hidden_dim) {
        set_error(JB_ERR_ARG, "decoder: hidden/intermediate/q dims must be multiples of 256, intermediate >= hidden"); return nullptr;
    }
    // every sharded product pushes its rows from the epilogue of the streaming GEMV, which exists for Q4_K and Q6_K only
    for (int l = 0; l < model->n_layers; ++l) {
        const jllm_b200_layer_desc& w = model->layers[l];
        const int ts[7] = { w.type_wq, w.type_wk, w.type_wv, w.type_wo, w.type_w_gate, w.type_w_up, w.type_w_down };
        for (int t : ts)
            if (t != T_Q4K && t != T_Q6K) { set_error(JB_ERR_TYPE, "decoder: ggml type %d in layer %d has no tensor-parallel path (Q4_K and Q6_K only)", t, l); return nullptr; }
    }
    if (model->output_type != T_Q4K && model->output_type != T_Q6K) { set_error(JB_ERR_TYPE, "decoder: output type %d has no tensor-parallel path", model->output_type); return nullptr; }
    if (!ctx()) return nullptr;
    // This rank's own region may hold the packets of an earlier session, whose epochs would pass for fresh ones: clear it.
    // (The caller must let every rank finish its create before any rank runs a step: a barrier, as TPDecoder does.)
    if (cudaMemset(regions[rank], 0, jllm_b200_tp_region_bytes(model->hidden_dim, model->n_heads * hd, model->intermediate_dim)) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaMemset(exchange region)"); return nullptr; }
    jllm_b200_decoder* d = new (std::nothrow) jllm_b200_decoder();
    if (!d) return nullptr;
    d->m = *model;
    d->layers.assign(model->layers, model->layers + model->n_layers);
    d->m.layers = d->layers.data();
    d->fused = true; d->use_graph = (flags & 2) != 0; d->chain = (flags & 8) != 0;
    d->tp_on = true;
    d->nh_l = model->n_heads / world; d->nkv_l = model->n_kv_heads / world; d->I_l = model->intermediate_dim / world;
    d->H_l = model->hidden_dim / world; d->V_l = model->vocab_size / world;
    tp_region_layout(model->hidden_dim, model->n_heads * hd, model->intermediate_dim, d->tp_off);
    for (int r = 0; r < TP_MAX_WORLD; ++r) d->tp.peer[r] = r < world ? (unsigned char*)regions[r] : nullptr;
    d->tp.rank = rank; d->tp.world = world; d->tp.flags_off = d->tp_off[4]; d->tp.argmax_off = d->tp_off[5];
    d->tp.epochs_per_step = model->n_layers; d->tp.status = ctx()->d_status;
    if (cudaMalloc(&d->seq, 256) != cudaSuccess) { cudaGetLastError(); set_error(JB_ERR_NOMEM, "decoder: step counter"); delete d; return nullptr; }
    cudaMemset(d->seq, 0, 256);
    d->tp.seq = d->seq;
    jllm::KVCachePool::Config c = { model->n_layers, d->nkv_l, hd, model->max_context, 0, 1 };
    if (!d->kv.init(c) || !d->kv.kv_scale_ptr(0, 0, false)) { set_error(JB_ERR_NOMEM, "decoder: KV pool allocation failed"); d->kv.destroy(); cudaFree(d->seq); delete d; return nullptr; }
    if (dec_alloc(d)) { d->kv.destroy(); cudaFree(d->seq); delete d; return nullptr; }
    splitk_buffer((size_t)d->nh_l * 64 * (hd + 4), true);
    return d;
}
void jllm_b200_decoder_destroy(jllm_b200_decoder* d) {
    if (!d) return;
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->own_stream) cudaStreamDestroy(d->own_stream);
    if (d->slab) cudaFree(d->slab);
    if (d->pf_slab) cudaFree(d->pf_slab);
    if (d->seq) cudaFree(d->seq);
    d->kv.destroy();
    delete d;
}
int jllm_b200_decoder_reset(jllm_b200_decoder* d) {
    JB_CUDA(cudaMemset(d->state, 0, 64));
    d->kv.clear();
    return JB_OK;
}
int jllm_b200_decoder_step(jllm_b200_decoder* d, int token, int position, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (position < 0 || position >= d->m.max_context) return set_error(JB_ERR_ARG, "decoder: position %d outside the context of %d", position, d->m.max_context);
    if (token < 0 || token >= d->m.vocab_size) return set_error(JB_ERR_ARG, "decoder: token %d outside the vocabulary", token);
    JB_CUDA(launch_k(set_state_kernel, dim3(1), dim3(32), 0, st, false, d->state, position, token));
    count_launch();
    return dec_enqueue_step(d, splits_for_ctx(d, position), st);
}

int jllm_b200_decoder_prefill(jllm_b200_decoder* d, const int* host_tokens, int n_tokens, int start_pos, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (d->tp_on) return set_error(JB_ERR_STATE, "decoder: batched prefill is not available in a tensor-parallel session");
    if (!host_tokens || n_tokens < 2) return set_error(JB_ERR_ARG, "decoder: batched prefill needs at least two tokens (got %d)", n_tokens);
    if (start_pos < 0 || start_pos + n_tokens > d->m.max_context) return set_error(JB_ERR_LIMIT, "decoder: positions %d..%d exceed the context of %d", start_pos, start_pos + n_tokens - 1, d->m.max_context);
    for (int i = 0; i < n_tokens; ++i)
        if (host_tokens[i] < 0 || host_tokens[i] >= d->m.vocab_size) return set_error(JB_ERR_ARG, "decoder: prompt token %d outside the vocabulary", host_tokens[i]);
    const int chunk = d->pf_chunk < 2 ? 2 : d->pf_chunk;
    DCHK(dec_prefill_alloc(d, n_tokens < chunk ? n_tokens : chunk));
    const jllm_b200_model_desc& m = d->m;
    const int H = m.hidden_dim;
    int done = 0, last_n = 0;
    while (done < n_tokens) {
        int n = n_tokens - done < chunk ? n_tokens - done : chunk;
        if (n_tokens - done - n == 1) --n;                  // never leave a chunk of one token: a batched product needs two
        JB_CUDA(cudaMemcpyAsync(d->pf_tokens, host_tokens + done, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, st));
        DCHK(dec_prefill_chunk(d, d->pf_tokens, n, start_pos + done, st));
        done += n; last_n = n;
    }
    // logits of the last prompt token only (src/engine/decode.cu:2019-2050), greedy token on the device; the step state
    // moves to the position after the prompt, so jllm_b200_decoder_step_device continues from there
    JB_CUDA(launch_k(set_state_kernel, dim3(1), dim3(32), 0, st, false, d->state, start_pos + n_tokens - 1, host_tokens[n_tokens - 1]));
    count_launch();
    DCHK(launch_rmsnorm(d->normed, d->pf_x + (size_t)(last_n - 1) * H, nullptr, m.output_norm, true, 1, H, m.rms_eps, st));
    DCHK(jllm_b200_gemv_quant_f32(d->logits, m.output, m.output_type, d->normed, m.vocab_size, H, st));
    const int ag = m.vocab_size >= 64 * 1024 ? 64 : (m.vocab_size + 1023) / 1024;
    JB_CUDA(launch_k(argmax_advance_kernel, dim3(ag), dim3(1024), 0, st, pdl_enabled(), (const float*)d->logits, m.vocab_size, d->state,
                     d->out_tokens, d->out_cap, (unsigned int*)(d->state + 32)));
    count_launch();
    d->host_pos = start_pos + n_tokens;
    return JB_OK;
}
int jllm_b200_decoder_set_prefill_chunk(jllm_b200_decoder* d, int tokens) {
    if (tokens < 2) return set_error(JB_ERR_ARG, "decoder: prefill chunk of %d tokens", tokens);
    d->pf_chunk = tokens;
    return JB_OK;
}

int jllm_b200_decoder_generate(jllm_b200_decoder* d, const int* host_prompt, int n_prompt, int n_new, int* host_out, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (d->use_graph && (st == nullptr || st == cudaStreamLegacy)) {
        if (!d->own_stream) JB_CUDA(cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking));
        JB_CUDA(cudaStreamSynchronize(st));          // order after whatever the caller queued on the default stream
        st = d->own_stream; stream = (void*)st;
    }
    if (n_prompt <= 0 || n_new < 0 || !host_prompt) return set_error(JB_ERR_ARG, "decoder: n_prompt=%d n_new=%d", n_prompt, n_new);
    if (n_prompt + n_new > d->m.max_context) return set_error(JB_ERR_LIMIT, "decoder: %d tokens exceed the context of %d", n_prompt + n_new, d->m.max_context);
    for (int i = 0; i < n_prompt; ++i)
        if (host_prompt[i] < 0 || host_prompt[i] >= d->m.vocab_size) return set_error(JB_ERR_ARG, "decoder: prompt token %d outside the vocabulary", host_prompt[i]);
    if (d->batched_prefill && !d->tp_on && n_prompt >= 2) {
        // the prompt in one batched pass (the first generated token comes out of it), then n_new - 1 self-feeding decode steps
        JB_CUDA(cudaMemsetAsync(d->state, 0, 64, st));
        d->kv.clear();
        DCHK(jllm_b200_decoder_prefill(d, host_prompt, n_prompt, 0, stream));
        for (int s = 1; s < n_new; ++s) DCHK(jllm_b200_decoder_step_device(d, stream));
        if (n_new > 0 && host_out) JB_CUDA(cudaMemcpyAsync(host_out, d->out_tokens, (size_t)n_new * sizeof(int), cudaMemcpyDeviceToHost, st));
        JB_CUDA(cudaStreamSynchronize(st));
        return jllm_b200_device_status(stream);
    }
    JB_CUDA(cudaMemcpyAsync(d->prompt_dev, host_prompt, (size_t)n_prompt * sizeof(int), cudaMemcpyHostToDevice, st));
    JB_CUDA(cudaMemsetAsync(d->state, 0, 64, st));
    d->kv.clear();
    // steps 0 .. n_prompt-1 consume prompt tokens; every step's argmax is recorded, the first n_prompt-1 are discarded below
    const int total_steps = n_prompt + (n_new > 0 ? n_new - 1 : 0);
    for (int s = 0; s < total_steps; ++s) {
        if (s < n_prompt) {
            JB_CUDA(launch_k(next_prompt_kernel, dim3(1), dim3(32), 0, st, false, d->state, (const int*)d->prompt_dev, 0));
            count_launch();
        }
        const int ns = splits_for_ctx(d, s);
        if (d->use_graph) {
            DCHK(dec_graph_for(d, ns, st));
            JB_CUDA(cudaGraphLaunch(d->graph_exec, st));
            count_launch(d->kernels_per_step);
        } else {
            DCHK(dec_enqueue_step(d, ns, st));
        }
    }
    if (n_new > 0 && host_out)
        JB_CUDA(cudaMemcpyAsync(host_out, d->out_tokens + (n_prompt - 1), (size_t)n_new * sizeof(int), cudaMemcpyDeviceToHost, st));
    JB_CUDA(cudaStreamSynchronize(st));
    return jllm_b200_device_status(stream);
}
// One user-facing step: token and position come from (pinned) host memory, the sampled token goes back to
// host memory, and the call returns when it is there — the per-token host/device boundary of the reference
// engine (src/engine/decode.cu:2170-2175), minus the 600 KB logits copy (sampling runs on the device).
int jllm_b200_decoder_step_sync(jllm_b200_decoder* d, const int* host_pos_token, int* host_next, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!host_pos_token || !host_next) return set_error(JB_ERR_PTR, "decoder: null host pointer");
    if (d->use_graph && (st == nullptr || st == cudaStreamLegacy)) {
        if (!d->own_stream) JB_CUDA(cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking));
        st = d->own_stream;
    }
    const int pos = host_pos_token[0], tok = host_pos_token[1];
    if (pos < 0 || pos >= d->m.max_context) return set_error(JB_ERR_ARG, "decoder: position %d outside the context of %d", pos, d->m.max_context);
    if (tok < 0 || tok >= d->m.vocab_size) return set_error(JB_ERR_ARG, "decoder: token %d outside the vocabulary", tok);
    JB_CUDA(cudaMemcpyAsync(d->state, host_pos_token, 2 * sizeof(int), cudaMemcpyHostToDevice, st));
    const int ns = splits_for_ctx(d, pos);
    if (d->use_graph) {
        DCHK(dec_graph_for(d, ns, st));
        JB_CUDA(cudaGraphLaunch(d->graph_exec, st));
        count_launch(d->kernels_per_step);
    } else {
        DCHK(dec_enqueue_step(d, ns, st));
    }
    JB_CUDA(cudaMemcpyAsync(host_next, d->state + 1, sizeof(int), cudaMemcpyDeviceToHost, st));
    JB_CUDA(cudaStreamSynchronize(st));
    d->host_pos = pos + 1;
    return JB_OK;
}
// Enqueues the next step entirely from device-side state (position and token left by the previous step's argmax);
// nothing crosses the host boundary and the call does not wait.
int jllm_b200_decoder_step_device(jllm_b200_decoder* d, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (d->use_graph && (st == nullptr || st == cudaStreamLegacy)) return set_error(JB_ERR_ARG, "decoder: graph replay needs a non-default stream");
    if (d->host_pos >= d->m.max_context) return set_error(JB_ERR_LIMIT, "decoder: context of %d exhausted", d->m.max_context);
    const int ns = splits_for_ctx(d, d->host_pos);
    if (d->use_graph) {
        DCHK(dec_graph_for(d, ns, st));
        JB_CUDA(cudaGraphLaunch(d->graph_exec, st));
        count_launch(d->kernels_per_step);
    } else {
        DCHK(dec_enqueue_step(d, ns, st));
    }
    d->host_pos += 1;
    return JB_OK;
}
const float* jllm_b200_decoder_logits(jllm_b200_decoder* d) { return d->logits; }
int jllm_b200_decoder_last_token(jllm_b200_decoder* d, void* stream) {
    int h[3] = { 0, 0, 0 };
    if (cudaMemcpyAsync(h, d->state, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess) return -1;
    cudaStreamSynchronize((cudaStream_t)stream);
    return h[1];
}
int jllm_b200_decoder_kernels_per_step(jllm_b200_decoder* d) { return d->kernels_per_step; }
int jllm_b200_decoder_recorded_tokens(jllm_b200_decoder* d, int first, int n, int* host_out, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    int h[3] = { 0, 0, 0 };
    if (cudaMemcpyAsync(h, d->state, sizeof h, cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
    const int have = h[2] < d->out_cap ? h[2] : d->out_cap;
    if (host_out && n > 0 && first >= 0 && first < have) {
        const int m = first + n <= have ? n : have - first;
        if (cudaMemcpyAsync(host_out, d->out_tokens + first, (size_t)m * sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
        cudaStreamSynchronize(st);
    }
    return h[2];
}
const void* jllm_b200_decoder_buffer(jllm_b200_decoder* d, int which) {
    switch (which) {
        case 0: return d->x;   case 1: return d->x2; case 2: return d->q;  case 3: return d->k; case 4: return d->v;
        case 5: return d->att; case 6: return d->sw; case 7: return d->kv.key_ptr(0, 0); case 8: return d->kv.kv_scale_ptr(0, 0, false);
        default: return nullptr;
    }
}

}  // extern "C"
