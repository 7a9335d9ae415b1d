// mmq.cu — batched K-quant GEMM (prefill), first CUDA-core version.
//
// Arithmetic mirrors the reference's default prefill path: activations are quantised
// per 32 without clamping; Q4_K keeps (half d, half sum-of-x) per group and folds the
// weight sub-scales as half products, Q6_K keeps fp32 d (mmq_q4k_llama.cu:383-404,
// :159-163, :321-322; mmq_q6k_llama.cu:424-438, :208, :361).
#include "mmq.cuh"
#include <cstdlib>
#include <cstring>

namespace jb {

struct ActQ { int8_t* q; float* d; float* s; };   // [N][K] codes, [N][K/32] scale, [N][K/32] sum

size_t mmq_scratch_bytes(int N, int K) { return (size_t)N * K + 2 * (size_t)N * (K / 32) * sizeof(float) + 256; }

void* mmq_scratch(size_t bytes, bool may_alloc) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    if (bytes > c->mmq_act_bytes) {
        if (!may_alloc) return nullptr;
        if (c->mmq_act) cudaFree(c->mmq_act);
        c->mmq_act = nullptr; c->mmq_act_bytes = 0;
        if (cudaMalloc(&c->mmq_act, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        c->mmq_act_bytes = bytes;
    }
    return c->mmq_act;
}

// one warp per 32-element group of one token
__global__ void mmq_quantize_kernel(const __half* x, ActQ a, int N, int K, int ds4) {
    pdl_wait();
    const long long g = (long long)blockIdx.x * blockDim.y + threadIdx.y;
    const int lane = threadIdx.x, G = K / 32;
    if (g >= (long long)N * G) return;
    const float v = __half2float(x[g * 32 + lane]);
    const float amax = warp_max(fabsf(v));
    float sum = v;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    const float d = __fdiv_rn(amax, 127.0f), dinv = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    a.q[g * 32 + lane] = (int8_t)__float2int_rn(__fmul_rn(v, dinv));
    if (lane == 0) {
        a.d[g] = ds4 ? __half2float(__float2half_rn(d)) : d;
        a.s[g] = ds4 ? __half2float(__float2half_rn(sum)) : 0.f;
    }
}

// one warp per (row, token); lanes stride over 32-groups (Q4_K) / 16-groups (Q6_K)
__global__ void mmq_simple_kernel(__half* y, const uint8_t* W, int type, ActQ a, int M, int N, int K, int32_t* dbg) {
    pdl_wait();
    const int row = blockIdx.x * blockDim.y + threadIdx.y, tok = blockIdx.y, lane = threadIdx.x;
    if (row >= M) return;
    const int nb = K / QK_K;
    const int8_t* q8 = a.q + (size_t)tok * K;
    const float* d8 = a.d + (size_t)tok * (K / 32);
    const float* s8 = a.s + (size_t)tok * (K / 32);
    float acc = 0.f;
    if (type == T_Q4K) {
        for (int g = lane; g < nb * 8; g += 32) {
            const uint8_t* blk = W + ((size_t)row * nb + (g >> 3)) * Q4K_BYTES;
            const int j = g & 7;
            const uint32_t* s = reinterpret_cast<const uint32_t*>(blk + 4);
            int sc, mn; scale_min_k4(j, s[0], s[1], s[2], sc, mn);
            const uint32_t* qs = reinterpret_cast<const uint32_t*>(blk + 16 + 32 * (j >> 1));
            const int* xq = reinterpret_cast<const int*>(q8 + g * 32);
            int dot = 0;
            #pragma unroll
            for (int w = 0; w < 8; ++w) dot = dp4a_us((j & 1) ? (qs[w] >> 4) & 0x0F0F0F0Fu : qs[w] & 0x0F0F0F0Fu, xq[w], dot);
            if (dbg) dbg[((size_t)tok * M + row) * (nb * 8) + g] = dot;
            const __half dh = __ushort_as_half(*reinterpret_cast<const unsigned short*>(blk));
            const __half mh = __hneg(__ushort_as_half(*reinterpret_cast<const unsigned short*>(blk + 2)));
            const float ax = __half2float(__hmul(dh, __float2half_rn((float)sc)));
            const float ay = __half2float(__hmul(mh, __float2half_rn((float)mn)));
            acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(ax, d8[g]), (float)dot));
            acc = __fadd_rn(acc, __fmul_rn(ay, s8[g]));
        }
    } else {
        for (int g = lane; g < nb * 16; g += 32) {
            const uint8_t* blk = W + ((size_t)row * nb + (g >> 4)) * Q6K_BYTES;
            const int e0 = (g & 15) * 16;
            int dot = 0;
            for (int i = 0; i < 16; ++i) {
                const int e = e0 + i, n = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;
                int lo = (quarter & 1) ? blk[64 * n + 32 + l] : blk[64 * n + l];
                lo = (quarter & 2) ? (lo >> 4) : (lo & 0xF);
                const int qv = (lo | (((blk[128 + 32 * n + l] >> (2 * quarter)) & 3) << 4)) - 32;
                dot += qv * (int)q8[(g >> 4) * 256 + e];
            }
            if (dbg) dbg[((size_t)tok * M + row) * (nb * 16) + g] = dot;
            const float d = h2f_bits(blk[208] | (blk[209] << 8));
            acc += __fmul_rn(__fmul_rn(__fmul_rn((float)dot, (float)(int8_t)blk[192 + (g & 15)]), d8[g >> 1]), d);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)tok * M + row] = __float2half_rn(acc);
}

static bool capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

int launch_add_half(__half* out, const __half* a, const __half* b, long long n, cudaStream_t st);      // elementwise.cu

static int launch_mmq_impl(__half* y, const void* W, int type, const __half* x, int M, int N, int K, int32_t* dbg, const __half* residual,
                           bool same_x, cudaStream_t st);

int launch_mmq(__half* y, const void* W, int type, const __half* x, int M, int N, int K, int32_t* dbg, cudaStream_t st) {
    return launch_mmq_impl(y, W, type, x, M, N, K, dbg, nullptr, false, st);
}
int launch_mmq_ex(__half* y, const void* W, int type, const __half* x, int M, int N, int K, const __half* residual, bool same_x, cudaStream_t st) {
    return launch_mmq_impl(y, W, type, x, M, N, K, nullptr, residual, same_x, st);
}

// Two products over the same activations (gate and up): one launch of the tensor-core kernel when both matrices are of one
// type and that kernel is the one each would get on its own; else one product after the other, the second reusing the
// quantised operand of the first.
int launch_mmq_pair(__half* y1, __half* y2, const void* W1, int type1, const void* W2, int type2, const __half* x, int M1, int M2, int N, int K,
                    cudaStream_t st) {
    static const bool tc_off = [] { const char* e = getenv("JLLM_B200_MMQ"); return e && !strcmp(e, "cuda"); }();
    static const bool pair_off = [] { const char* e = getenv("JLLM_B200_MMQ_PAIR"); return e && e[0] == '0'; }();
    const bool ok = !tc_off && !pair_off && type1 == type2 && M1 > 0 && M2 > 0 && N > 0 && K > 0 && K % QK_K == 0 && y1 && y2 && W1 && W2 && x &&
                    (type1 == T_Q4K || type1 == T_Q6K) && !mmq_stream_applies(W1, type1, M1, N, K) && !mmq_stream_applies(W2, type2, M2, N, K) &&
                    mmq_tc_applies(W1, type1, M1, N, K) && mmq_tc_applies(W2, type2, M2, N, K);
    if (!ok) {
        const int rc = launch_mmq_impl(y1, W1, type1, x, M1, N, K, nullptr, nullptr, false, st);
        return rc ? rc : launch_mmq_impl(y2, W2, type2, x, M2, N, K, nullptr, nullptr, true, st);
    }
    const size_t need = mmq_tc_scratch_bytes_pair(type1, M1, M2, N, K);
    __half* xq = (__half*)mmq_scratch(need, !capturing(st));
    if (!xq) return set_error(JB_ERR_NOMEM, "batched gemm: %zu B of activation scratch unavailable", need);
    if (DeviceCtx* c = ctx()) c->mms_op_x = nullptr;
    return launch_mmq_tc_pair(y1, y2, W1, W2, type1, x, xq, M1, M2, N, K, false, st);
}

static int launch_mmq_impl(__half* y, const void* W, int type, const __half* x, int M, int N, int K, int32_t* dbg, const __half* residual,
                           bool same_x, cudaStream_t st) {
    if (M <= 0 || N <= 0) return JB_OK;
    if (K <= 0 || K % QK_K) return set_error(JB_ERR_ARG, "batched gemm: K=%d is not a positive multiple of 256", K);
    if (type != T_Q4K && type != T_Q6K) return set_error(JB_ERR_TYPE, "batched gemm: ggml type %d", type);
    if (!y || !W || !x) return set_error(JB_ERR_PTR, "batched gemm: null pointer");
    if (type == T_Q4K && ((uintptr_t)W & 3)) return set_error(JB_ERR_PTR, "batched gemm: Q4_K weights must be 4-byte aligned");
    // JLLM_B200_MMQ=cuda keeps the CUDA-core kernel (the one that can also export the integer accumulators)
    static const bool tc_off = [] { const char* e = getenv("JLLM_B200_MMQ"); return e && !strcmp(e, "cuda"); }();
    if (!dbg && !tc_off && mmq_stream_applies(W, type, M, N, K)) {
        const size_t need_s = mmq_stream_scratch_bytes(type, M, N, K);
        void* sc = mmq_scratch(need_s, !capturing(st));
        if (!sc) return set_error(JB_ERR_NOMEM, "batched gemm: %zu B of activation scratch unavailable", need_s);
        if (DeviceCtx* c = ctx()) c->tc_op_x = nullptr;          // the scratch is shared: the other path's operand is gone
        return launch_mmq_stream(y, W, type, x, sc, M, N, K, residual, same_x, st);
    }
    if (residual) {          // the other kernels have no fused exit: product, then the add (in place)
        const int rc = launch_mmq_impl(y, W, type, x, M, N, K, dbg, nullptr, false, st);
        return rc ? rc : launch_add_half(y, residual, y, (long long)N * M, st);
    }
    if (!dbg && !tc_off && mmq_tc_applies(W, type, M, N, K)) {
        const size_t need_tc = mmq_tc_scratch_bytes(type, M, N, K);
        __half* xq = (__half*)mmq_scratch(need_tc, !capturing(st));
        if (!xq) return set_error(JB_ERR_NOMEM, "batched gemm: %zu B of activation scratch unavailable", need_tc);
        if (DeviceCtx* c = ctx()) c->mms_op_x = nullptr;
        return launch_mmq_tc(y, W, type, x, xq, M, N, K, same_x, st);
    }
    if (DeviceCtx* c = ctx()) { c->tc_op_x = nullptr; c->mms_op_x = nullptr; }
    const size_t need = mmq_scratch_bytes(N, K);
    uint8_t* base = (uint8_t*)mmq_scratch(need, !capturing(st));
    if (!base) return set_error(JB_ERR_NOMEM, "batched gemm: %zu B of activation scratch unavailable", need);
    ActQ a;
    a.q = (int8_t*)base;
    a.d = (float*)(base + (((size_t)N * K + 255) & ~(size_t)255));
    a.s = a.d + (size_t)N * (K / 32);
    const long long groups = (long long)N * (K / 32);
    JB_CUDA(launch_k(mmq_quantize_kernel, dim3((unsigned)((groups + 3) / 4)), dim3(32, 4), 0, st, pdl_enabled(), x, a, N, K, (int)(type == T_Q4K)));
    count_launch();
    JB_CUDA(launch_k(mmq_simple_kernel, dim3((M + 3) / 4, N), dim3(32, 4), 0, st, pdl_enabled(), y, (const uint8_t*)W, type, a, M, N, K, dbg));
    count_launch();
    return JB_OK;
}

}  // namespace jb
