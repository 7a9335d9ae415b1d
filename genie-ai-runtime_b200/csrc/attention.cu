// attention.cu — decode / prefill attention over an FP16 or INT8 KV cache, sm_100a.
//
// Reference: src/kernels/attention.cu — single-query decode (:244-375), split-K partial +
// reduce (:837-969), batched causal prefill (:382-514).  INT8 K/V carry one fp32 scale per
// (position, kv head): k = k8*ks inside the QK dot, v = v8*vs inside PV.
//
// This file holds the general kernel: any head_dim <= 512, FP16 or INT8 cache, sliding
// window, cache slot stride != head_dim, device-side position, ragged batches, causal prefill
// (the slice itself is attention_general.cuh).  The INT8 / head_dim 128 paths live in
// attention_tma.cu (decode, 2-D TMA tiles) and attention_prefill.cu (causal prefill with query tiling).
#include "attention.cuh"
#include <cstdlib>
#include "attention_general.cuh"
#include <cfloat>

namespace jb {

// Split policy (also what the decoder session keys its captured graphs on): one slice below 640 keys (a sliced call pays the
// partials, a ticket and the merge), then slices of at least 128 keys (512 from 2048 keys on), at most 32 (the reference caps at
// 8 slices for its 8-SM part, attention.cu:1000-1005).
int attn_splits_for(int seq_len) {
    if (seq_len < 640) return 1;
    const int n = seq_len < 2048 ? seq_len / 128 : seq_len / 512;
    return n > 32 ? 32 : n;
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

__global__ void __launch_bounds__(AG_THREADS) attn_general_kernel(const AttnArgs a) {
    pdl_wait();
    extern __shared__ float sm[];
    const int head = blockIdx.x, split = blockIdx.y, z = blockIdx.z;
    const int kvh = head / (a.n_heads / a.n_kv);
    AgCache c = { a.k, a.v, a.ks, a.vs, a.n_kv, a.chd, a.kv_int8, a.window };
    int seq = a.d_pos ? (*a.d_pos + 1) : a.seq_len;
    if (a.k_list) { c.k = a.k_list[z]; c.v = a.v_list[z]; c.ks = a.ks_list ? a.ks_list[z] : nullptr; c.vs = a.vs_list ? a.vs_list[z] : nullptr; seq = a.seq_lens[z]; }
    if (a.causal_start >= 0) seq = a.causal_start + z + 1;
    const int per = (seq + a.n_splits - 1) / a.n_splits;
    const int kv0 = split * per, kv1 = min(kv0 + per, seq);
    const size_t qoff = ((size_t)z * a.n_heads + head) * a.hd;
    float M, L;
    if (a.n_splits == 1) {
        // emit() runs after M and L are final, so the normalisation can be applied on the way out
        ag_slice(a.q + qoff, c, kvh, a.hd, seq, kv0, kv1, a.scale, sm, M, L,
                 [&](int d, float o) { a.out[qoff + d] = __float2half_rn(L > 0.f ? o * (1.0f / L) : 0.f); });
    } else {
        float* pb = a.part + (((size_t)z * a.n_heads + head) * a.n_splits + split) * (a.hd + 2);
        ag_slice(a.q + qoff, c, kvh, a.hd, seq, kv0, kv1, a.scale, sm, M, L, [&](int d, float o) { pb[2 + d] = o; });
        if (threadIdx.x == 0) { pb[0] = L > 0.f ? M : -FLT_MAX; pb[1] = L; }
    }
}

__global__ void attn_reduce_kernel(__half* out, const float* part, int n_heads, int hd, int n_splits) {
    pdl_wait();
    const int head = blockIdx.x, z = blockIdx.y;
    ag_merge_slices(out + ((size_t)z * n_heads + head) * hd, part + ((size_t)z * n_heads + head) * n_splits * (hd + 2), hd, n_splits);
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
    JB_CUDA(launch_k(attn_general_kernel, dim3(c.n_heads, n_splits, batch), dim3(AG_THREADS), ag_smem_bytes(c.hd), st, pdl_enabled(), a));
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
    // INT8 / head_dim 128 with a known cache extent (a length, a device-side position with its bound, or a plan of tensor
    // maps for a ragged batch): 2-D TMA tiles on the tensor cores; everything else — FP16 caches, other head sizes, sliding
    // windows, pointer lists that live in device memory — goes to the general kernel
    return attention_tma_applies(c) ? launch_attention_tma(c, st) : launch_attention_general(c, st);
}

}  // namespace jb
