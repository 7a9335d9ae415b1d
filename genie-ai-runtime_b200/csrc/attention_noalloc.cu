// attention_noalloc.cu — decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot let it call cudaMalloc: an engine that has already handed every free
// byte of the GPU to its own KV and scratch pools, a serving loop that forbids driver calls which may
// synchronise the whole device in the middle of a request.  The regular split-K attention grows a per-device partials buffer on demand; this
// file offers the same computation with that buffer replaced by a fixed array compiled into the library.
//
// The array lives in every GPU context that loads the library (JLLM_B200_NOALLOC_MAX_FLOATS floats, 1 MiB)
// until the process exits.  All calls share it and it keeps the previous call's values: the kernels below
// overwrite every (head, slice) record they later read, so nothing has to be cleared, but two calls that run
// at the same time on one GPU (different streams) would overwrite each other's partials — callers must
// order them.
#include "../../include/jllm_b200.h"
#include "common.cuh"
#include "attention_general.cuh"
#include <cfloat>

namespace jb {

static __device__ __align__(256) float g_na_scratch[JLLM_B200_NOALLOC_MAX_FLOATS];

// per-device address of the array, resolved once with that device current
static float* g_na_ptr[16] = {};

struct NaArgs {
    __half* out; const __half* q; const void* k; const void* v; const float* ks; const float* vs;
    int n_heads, n_kv, hd, chd, seq, kv_int8, window, n_splits; float scale; float* part;
};

// One CTA per (query head, KV slice): the general attention slice (attention_general.cuh), its unnormalised partial
// (m, l, acc[hd]) written to the fixed array.
__global__ void __launch_bounds__(AG_THREADS) attn_noalloc_partial_kernel(const NaArgs a) {
    pdl_wait();
    extern __shared__ float sm[];
    const int head = blockIdx.x, split = blockIdx.y;
    const int kvh = head / (a.n_heads / a.n_kv);
    const AgCache c = { a.k, a.v, a.ks, a.vs, a.n_kv, a.chd, a.kv_int8, a.window };
    const int per = (a.seq + a.n_splits - 1) / a.n_splits;
    const int kv0 = split * per, kv1 = min(kv0 + per, a.seq);
    // every record of this call is written here, empty slices included, so stale contents are never read
    float* pb = a.part + ((size_t)head * a.n_splits + split) * (a.hd + 2);
    float M, L;
    ag_slice(a.q + (size_t)head * a.hd, c, kvh, a.hd, a.seq, kv0, kv1, a.scale, sm, M, L, [&](int d, float o) { pb[2 + d] = o; });
    if (threadIdx.x == 0) { pb[0] = L > 0.f ? M : -FLT_MAX; pb[1] = L; }
}

__global__ void attn_noalloc_reduce_kernel(__half* out, const float* part, int hd, int n_splits) {
    pdl_wait();
    ag_merge_slices(out + (size_t)blockIdx.x * hd, part + (size_t)blockIdx.x * n_splits * (hd + 2), hd, n_splits);
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
        g_na_ptr[dev] = ptr;
    }
    NaArgs a = { (__half*)output, (const __half*)q, k_cache, v_cache, k_scales, v_scales, n_heads, n_kv_heads, head_dim, cache_head_dim,
                 seq_len, kv_int8, window, n_splits, scale, g_na_ptr[dev] };
    JB_CUDA(launch_k(attn_noalloc_partial_kernel, dim3(n_heads, n_splits), dim3(AG_THREADS), ag_smem_bytes(head_dim), st, pdl_enabled(), a));
    JB_CUDA(launch_k(attn_noalloc_reduce_kernel, dim3(n_heads), dim3(128), 0, st, pdl_enabled(), (__half*)output, (const float*)g_na_ptr[dev], head_dim, n_splits));
    count_launch(2);
    return JB_OK;
}
