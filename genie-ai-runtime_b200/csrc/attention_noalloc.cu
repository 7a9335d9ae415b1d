// attention_noalloc.cu — decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot let it call cudaMalloc: an engine that has already handed every free
// byte of the GPU to its own KV and scratch pools, a serving loop that forbids driver calls which may
// synchronise the whole device in the middle of a request, or code that is recording a CUDA graph (where an
// allocation is an error).  The regular split-K attention grows a per-device partials buffer on demand; this
// file offers the same computation with that buffer replaced by a fixed array compiled into the library.
//
// The array lives in every GPU context that loads the library (JLLM_B200_NOALLOC_MAX_FLOATS floats, 1 MiB)
// until the process exits.  All calls share it and it keeps the previous call's values: the kernels below
// overwrite every (head, slice) record they later read, so nothing has to be cleared, but two calls that run
// at the same time on one GPU (different streams) would overwrite each other's partials — callers must
// order them.
#include "../../include/jllm_b200.h"
#include "common.cuh"
#include <cfloat>

namespace jb {

constexpr int NA_THREADS = 128;
constexpr int NA_TILE    = 64;

static __device__ __align__(256) float g_na_scratch[JLLM_B200_NOALLOC_MAX_FLOATS];

// per-device address of the array, resolved once with that device current
static float* g_na_ptr[16] = {};
static int    g_na_sms[16] = {};

struct NaArgs {
    __half* out; const __half* q; const void* k; const void* v; const float* ks; const float* vs;
    int n_heads, n_kv, hd, chd, seq, kv_int8, window, n_splits; float scale; float* part;
};

__device__ __forceinline__ float na_block_reduce(float v, float* red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    #pragma unroll
    for (int w = 1; w < NA_THREADS / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

// One CTA per (query head, KV slice): online softmax over the slice, unnormalised partial (m, l, acc[hd])
// written to the fixed array.  Arithmetic as in the reference's split-K kernel, src/kernels/attention.cu:837-941.
__global__ void __launch_bounds__(NA_THREADS) attn_noalloc_partial_kernel(const NaArgs a) {
    pdl_wait();
    const int head = blockIdx.x, split = blockIdx.y;
    const int kvh = head / (a.n_heads / a.n_kv);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.hd, kv_dim = a.n_kv * a.chd, kv_off = kvh * a.chd;
    const int per = (a.seq + a.n_splits - 1) / a.n_splits;
    const int kv0 = split * per, kv1 = min(kv0 + per, a.seq);
    extern __shared__ float sm[];
    float* s_sc = sm; float* s_out = sm + NA_TILE; float* s_q = s_out + hd;
    __shared__ float red[NA_THREADS / 32];
    for (int d = tid; d < hd; d += NA_THREADS) { s_out[d] = 0.f; s_q[d] = __half2float(a.q[(size_t)head * hd + d]); }
    float run_max = -FLT_MAX, run_sum = 0.f;
    __syncthreads();
    for (int t0 = kv0; t0 < kv1; t0 += NA_TILE) {
        const int tl = min(NA_TILE, kv1 - t0);
        for (int t = warp; t < tl; t += NA_THREADS / 32) {
            const int p = t0 + t;
            float dot = 0.f;
            if (a.window > 0 && p < a.seq - a.window) { if (lane == 0) s_sc[t] = -INFINITY; continue; }
            if (a.kv_int8) {
                const int8_t* kr = reinterpret_cast<const int8_t*>(a.k) + (size_t)p * kv_dim + kv_off;
                const float sc = a.ks ? a.ks[(size_t)p * a.n_kv + kvh] : 1.0f;
                for (int d = lane; d < hd; d += 32) dot += s_q[d] * ((float)kr[d] * sc);
            } else {
                const __half* kr = reinterpret_cast<const __half*>(a.k) + (size_t)p * kv_dim + kv_off;
                for (int d = lane; d < hd; d += 32) dot += s_q[d] * __half2float(kr[d]);
            }
            dot = warp_sum(dot);
            if (lane == 0) s_sc[t] = dot * a.scale;
        }
        __syncthreads();
        float lm = -FLT_MAX;
        for (int t = tid; t < tl; t += NA_THREADS) lm = fmaxf(lm, s_sc[t]);
        const float new_max = fmaxf(run_max, na_block_reduce(lm, red, true));
        const float corr = expf(run_max - new_max);
        run_max = new_max;
        float ls = 0.f;
        for (int t = tid; t < tl; t += NA_THREADS) { const float pv = expf(s_sc[t] - run_max); s_sc[t] = pv; ls += pv; }
        run_sum = run_sum * corr + na_block_reduce(ls, red, false);
        for (int d = tid; d < hd; d += NA_THREADS) {
            float acc = 0.f;
            for (int t = 0; t < tl; ++t) {
                const size_t idx = (size_t)(t0 + t) * kv_dim + kv_off + d;
                const float vv = a.kv_int8 ? (float)reinterpret_cast<const int8_t*>(a.v)[idx] * (a.vs ? a.vs[(size_t)(t0 + t) * a.n_kv + kvh] : 1.0f)
                                           : __half2float(reinterpret_cast<const __half*>(a.v)[idx]);
                acc += s_sc[t] * vv;
            }
            s_out[d] = s_out[d] * corr + acc;
        }
        __syncthreads();
    }
    // every record of this call is written here, empty slices included, so stale contents are never read
    float* pb = a.part + ((size_t)head * a.n_splits + split) * (hd + 2);
    if (tid == 0) { pb[0] = kv0 < kv1 ? run_max : -FLT_MAX; pb[1] = run_sum; }
    for (int d = tid; d < hd; d += NA_THREADS) pb[2 + d] = s_out[d];
}

// out = Σ_s acc_s e^{m_s-M} / Σ_s l_s e^{m_s-M}  (reference :944-969)
__global__ void attn_noalloc_reduce_kernel(__half* out, const float* part, int hd, int n_splits) {
    pdl_wait();
    const int head = blockIdx.x;
    const float* pb = part + (size_t)head * n_splits * (hd + 2);
    float M = -FLT_MAX;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, pb[(size_t)s * (hd + 2)]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) L += pb[(size_t)s * (hd + 2) + 1] * expf(pb[(size_t)s * (hd + 2)] - M);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) acc += pb[(size_t)s * (hd + 2) + 2 + d] * expf(pb[(size_t)s * (hd + 2)] - M);
        out[(size_t)head * hd + d] = __float2half_rn(acc * inv);
    }
}

}  // namespace jb

using namespace jb;

extern "C" int jllm_b200_flash_attention_decode_noalloc(void* output, const void* q, const void* k_cache, const void* v_cache,
                                                        int n_heads, int n_kv_heads, int head_dim, int cache_head_dim, int seq_len,
                                                        float scale, int kv_int8, const float* k_scales, const float* v_scales,
                                                        int window, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return set_error(JB_ERR_ARG, "attention (no-alloc): n_heads=%d n_kv_heads=%d", n_heads, n_kv_heads);
    if (head_dim <= 0 || head_dim > 512 || cache_head_dim < head_dim) return set_error(JB_ERR_ARG, "attention (no-alloc): head_dim=%d cache_head_dim=%d", head_dim, cache_head_dim);
    if (!output || !q || !k_cache || !v_cache) return set_error(JB_ERR_PTR, "attention (no-alloc): null pointer");
    if (seq_len <= 0) { JB_CUDA(cudaMemsetAsync(output, 0, (size_t)n_heads * head_dim * sizeof(__half), st)); return JB_OK; }
    // slices of at least 128 keys, at most 32 per head
    int per = (seq_len + 31) / 32; if (per < 128) per = 128;
    const int n_splits = (seq_len + per - 1) / per;
    const long long need = (long long)n_heads * n_splits * (head_dim + 2);
    if (need > JLLM_B200_NOALLOC_MAX_FLOATS)
        return set_error(JB_ERR_LIMIT, "attention (no-alloc): %d heads x %d slices x (%d+2) floats = %lld exceed the built-in scratch of %d floats",
                         n_heads, n_splits, head_dim, need, JLLM_B200_NOALLOC_MAX_FLOATS);
    int dev = 0;
    JB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return set_error(JB_ERR_LIMIT, "attention (no-alloc): device ordinal %d out of range", dev);
    if (!g_na_ptr[dev]) {
        // First call on this device: resolve the device address of the array.  The array's name is only a host-side
        // handle; kernels need the address the runtime reports for the current device.
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_na_scratch);
        if (e != cudaSuccess || !ptr) return cuda_error(e, "cudaGetSymbolAddress(no-alloc scratch)");
        int sms = 0;
        JB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_na_sms[dev] = sms;
        g_na_ptr[dev] = ptr;
    }
    NaArgs a = { (__half*)output, (const __half*)q, k_cache, v_cache, k_scales, v_scales, n_heads, n_kv_heads, head_dim, cache_head_dim,
                 seq_len, kv_int8, window, n_splits, scale, g_na_ptr[dev] };
    const size_t smem = (size_t)(NA_TILE + 2 * head_dim) * sizeof(float);
    JB_CUDA(launch_k(attn_noalloc_partial_kernel, dim3(n_heads, n_splits), dim3(NA_THREADS), smem, st, pdl_enabled(), a));
    JB_CUDA(launch_k(attn_noalloc_reduce_kernel, dim3(n_heads), dim3(128), 0, st, pdl_enabled(), (__half*)output, (const float*)g_na_ptr[dev], head_dim, n_splits));
    count_launch(2);
    return JB_OK;
}
