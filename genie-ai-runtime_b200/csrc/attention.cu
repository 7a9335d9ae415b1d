// attention.cu — decode / prefill attention over an FP16 or INT8 KV cache, sm_100a.
//
// Reference: src/kernels/attention.cu — single-query decode (:244-375), split-K partial +
// reduce (:837-969), batched causal prefill (:382-514).  INT8 K/V carry one fp32 scale per
// (position, kv head): k = k8*ks inside the QK dot, v = v8*vs inside PV.
//
// This file holds the general kernel: any head_dim <= 512, FP16 or INT8 cache, sliding
// window, cache slot stride != head_dim, device-side position, ragged batches.  The
// INT8 / head_dim 128 fast path lives in attention_fast.cu.
#include "attention.cuh"
#include <cfloat>

namespace jb {

constexpr int AT_THREADS = 128;
constexpr int AT_TILE    = 64;

// Split policy: slices of at least 128 keys, at most 32 slices per head
// (the reference caps at 8 slices for its 8-SM part, attention.cu:1000-1005).
int attn_splits_for(int seq_len) {
    if (seq_len < 256) return 1;
    int per = (seq_len + 31) / 32;
    if (per < 128) per = 128;
    return (seq_len + per - 1) / per;
}

struct AttnArgs {
    __half* out; const __half* q;
    const void* k; const void* v; const float* ks; const float* vs;
    // ragged batch (extension): per-sequence cache bases and lengths; null for one sequence
    const void* const* k_list; const void* const* v_list; const float* const* ks_list; const float* const* vs_list;
    const int* seq_lens;
    int n_heads, n_kv, hd, chd, seq_len; const int* d_pos;
    float scale; int kv_int8, window, n_splits;
    int causal_start;       // prefill: query t sees start+t+1 keys (blockIdx.z = t); -1 = decode
    float* part;            // [z][head][split] m | l | acc[hd]
};

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    #pragma unroll
    for (int w = 1; w < AT_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

__global__ void __launch_bounds__(AT_THREADS) attn_general_kernel(const AttnArgs a) {
    pdl_wait();
    const int head = blockIdx.x, split = blockIdx.y, z = blockIdx.z;
    const int kvh = head / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.hd, kv_dim = a.n_kv * a.chd, kv_off = kvh * a.chd;
    const void* kc = a.k; const void* vc = a.v; const float* ks = a.ks; const float* vs = a.vs;
    int seq = a.d_pos ? (*a.d_pos + 1) : a.seq_len;
    if (a.k_list) { kc = a.k_list[z]; vc = a.v_list[z]; ks = a.ks_list ? a.ks_list[z] : nullptr; vs = a.vs_list ? a.vs_list[z] : nullptr; seq = a.seq_lens[z]; }
    if (a.causal_start >= 0) seq = a.causal_start + z + 1;
    const int per = (seq + a.n_splits - 1) / a.n_splits;
    const int kv0 = split * per, kv1 = min(kv0 + per, seq);
    const size_t qoff = ((size_t)z * a.n_heads + head) * hd;

    extern __shared__ float sm[];
    float* s_sc = sm; float* s_out = sm + AT_TILE; float* s_q = s_out + hd;
    __shared__ float red[AT_THREADS / 32];
    for (int d = tid; d < hd; d += AT_THREADS) { s_out[d] = 0.f; s_q[d] = __half2float(a.q[qoff + d]); }
    float run_max = -FLT_MAX, run_sum = 0.f;
    __syncthreads();

    for (int t0 = kv0; t0 < kv1; t0 += AT_TILE) {
        const int tl = min(AT_TILE, kv1 - t0);
        for (int t = warp; t < tl; t += AT_THREADS / 32) {
            const int p = t0 + t;
            float dot = 0.f;
            if (a.window > 0 && p < seq - a.window) { if (lane == 0) s_sc[t] = -INFINITY; continue; }
            if (a.kv_int8) {
                const int8_t* kr = reinterpret_cast<const int8_t*>(kc) + (size_t)p * kv_dim + kv_off;
                const float sc = ks ? ks[(size_t)p * a.n_kv + kvh] : 1.0f;
                for (int d = lane; d < hd; d += 32) dot += s_q[d] * ((float)kr[d] * sc);
            } else {
                const __half* kr = reinterpret_cast<const __half*>(kc) + (size_t)p * kv_dim + kv_off;
                for (int d = lane; d < hd; d += 32) dot += s_q[d] * __half2float(kr[d]);
            }
            dot = warp_sum(dot);
            if (lane == 0) s_sc[t] = dot * a.scale;
        }
        __syncthreads();
        float lm = -FLT_MAX;
        for (int t = tid; t < tl; t += AT_THREADS) lm = fmaxf(lm, s_sc[t]);
        const float tmax = block_reduce(lm, red, true);
        const float new_max = fmaxf(run_max, tmax);
        const float corr = expf(run_max - new_max);
        run_max = new_max;
        float ls = 0.f;
        for (int t = tid; t < tl; t += AT_THREADS) { const float pv = expf(s_sc[t] - run_max); s_sc[t] = pv; ls += pv; }
        const float tsum = block_reduce(ls, red, false);
        run_sum = run_sum * corr + tsum;
        for (int d = tid; d < hd; d += AT_THREADS) {
            float acc = 0.f;
            for (int t = 0; t < tl; ++t) {
                const int p = t0 + t;
                float vv;
                if (a.kv_int8) vv = (float)reinterpret_cast<const int8_t*>(vc)[(size_t)p * kv_dim + kv_off + d] * (vs ? vs[(size_t)p * a.n_kv + kvh] : 1.0f);
                else vv = __half2float(reinterpret_cast<const __half*>(vc)[(size_t)p * kv_dim + kv_off + d]);
                acc += s_sc[t] * vv;
            }
            s_out[d] = s_out[d] * corr + acc;
        }
        __syncthreads();
    }
    if (a.n_splits == 1) {
        const float inv = run_sum > 0.f ? 1.0f / run_sum : 0.f;
        for (int d = tid; d < hd; d += AT_THREADS) a.out[qoff + d] = __float2half_rn(s_out[d] * inv);
    } else {
        float* pb = a.part + (((size_t)z * a.n_heads + head) * a.n_splits + split) * (hd + 2);
        if (tid == 0) { pb[0] = kv0 < kv1 ? run_max : -FLT_MAX; pb[1] = run_sum; }
        for (int d = tid; d < hd; d += AT_THREADS) pb[2 + d] = s_out[d];
    }
}

// out = Σ_s acc_s e^{m_s-M} / Σ_s l_s e^{m_s-M}   (reference :944-969)
__global__ void attn_reduce_kernel(__half* out, const float* part, int n_heads, int hd, int n_splits) {
    pdl_wait();
    const int head = blockIdx.x, z = blockIdx.y;
    const float* pb = part + ((size_t)z * n_heads + head) * n_splits * (hd + 2);
    float M = -FLT_MAX;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, pb[(size_t)s * (hd + 2)]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) L += pb[(size_t)s * (hd + 2) + 1] * expf(pb[(size_t)s * (hd + 2)] - M);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) acc += pb[(size_t)s * (hd + 2) + 2 + d] * expf(pb[(size_t)s * (hd + 2)] - M);
        out[((size_t)z * n_heads + head) * hd + d] = __float2half_rn(acc * inv);
    }
}

float* splitk_buffer(size_t floats, bool may_alloc) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    if (floats > c->splitk_floats) {
        if (!may_alloc) return nullptr;
        if (c->splitk) cudaFree(c->splitk);
        c->splitk = nullptr; c->splitk_floats = 0;
        if (cudaMalloc(&c->splitk, floats * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        c->splitk_floats = floats;
    }
    return c->splitk;
}

static bool stream_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

int launch_attention_general(const AttnCall& c, cudaStream_t st) {
    if (c.n_heads <= 0 || c.n_kv <= 0 || c.n_heads % c.n_kv) return set_error(JB_ERR_ARG, "attention: n_heads=%d n_kv_heads=%d", c.n_heads, c.n_kv);
    if (c.hd <= 0 || c.hd > 512 || c.chd < c.hd) return set_error(JB_ERR_ARG, "attention: head_dim=%d cache_head_dim=%d", c.hd, c.chd);
    if (!c.out || !c.q) return set_error(JB_ERR_PTR, "attention: null q/out");
    if (!c.k_list && (!c.k || !c.v)) return set_error(JB_ERR_PTR, "attention: null cache pointer");
    const int batch = c.batch > 0 ? c.batch : 1;
    int n_splits = c.n_splits > 0 ? c.n_splits : (c.d_pos || c.causal_start >= 0 ? 1 : attn_splits_for(c.k_list ? c.max_seq : c.seq_len));
    if (!c.d_pos && !c.k_list && c.causal_start < 0 && c.seq_len <= 0) {     // nothing to attend to: zeros, like an empty softmax
        JB_CUDA(cudaMemsetAsync(c.out, 0, (size_t)c.n_heads * c.hd * sizeof(__half), st));
        return JB_OK;
    }
    AttnArgs a = {};
    a.out = c.out; a.q = c.q; a.k = c.k; a.v = c.v; a.ks = c.ks; a.vs = c.vs;
    a.k_list = c.k_list; a.v_list = c.v_list; a.ks_list = c.ks_list; a.vs_list = c.vs_list; a.seq_lens = c.seq_lens;
    a.n_heads = c.n_heads; a.n_kv = c.n_kv; a.hd = c.hd; a.chd = c.chd; a.seq_len = c.seq_len; a.d_pos = c.d_pos;
    a.scale = c.scale; a.kv_int8 = c.kv_int8; a.window = c.window; a.causal_start = c.causal_start;
    if (n_splits > 1) {
        const size_t need = (size_t)batch * c.n_heads * n_splits * (c.hd + 2);
        a.part = splitk_buffer(need, !stream_capturing(st));
        if (!a.part) n_splits = 1;       // no scratch (or capture in progress): one slice per head, still on the GPU
    }
    a.n_splits = n_splits;
    const size_t smem = (size_t)(AT_TILE + 2 * c.hd) * sizeof(float);
    JB_CUDA(launch_k(attn_general_kernel, dim3(c.n_heads, n_splits, batch), dim3(AT_THREADS), smem, st, pdl_enabled(), a));
    count_launch();
    if (n_splits > 1) {
        JB_CUDA(launch_k(attn_reduce_kernel, dim3(c.n_heads, batch), dim3(128), 0, st, pdl_enabled(), c.out, (const float*)a.part, c.n_heads, c.hd, n_splits));
        count_launch();
    }
    return JB_OK;
}

int launch_attn_reduce(__half* out, const float* part, int n_heads, int hd, int n_splits, int batch, cudaStream_t st) {
    JB_CUDA(launch_k(attn_reduce_kernel, dim3(n_heads, batch), dim3(128), 0, st, pdl_enabled(), out, part, n_heads, hd, n_splits));
    count_launch();
    return JB_OK;
}

int launch_attention(const AttnCall& c, cudaStream_t st) {
    if (c.n_heads <= 0 || c.n_kv <= 0 || c.n_heads % c.n_kv) return set_error(JB_ERR_ARG, "attention: n_heads=%d n_kv_heads=%d", c.n_heads, c.n_kv);
    if (!c.out || !c.q) return set_error(JB_ERR_PTR, "attention: null q/out");
    if (!c.k_list && (!c.k || !c.v)) return set_error(JB_ERR_PTR, "attention: null cache pointer");
    return attention_fast_applies(c) ? launch_attention_fast(c, st) : launch_attention_general(c, st);
}

}  // namespace jb
