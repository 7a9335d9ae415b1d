// ref_shim_gpu.cu — C wrappers over the reference's own GPU entry points (include/jllm_kernels.h of the
// reference, linked from its unmodified sources into oracle/_ref/libjllm_ref.so).  TEST INFRASTRUCTURE ONLY:
// tests/golden/make_golden_gpu.py calls these on a machine with a GPU to record what the reference's kernels
// return on seeded inputs, and to time them as the same-box comparator.  The product library never links this.
//
// Every wrapper takes HOST pointers, copies them to the device, runs the reference entry point on the default
// stream, synchronises and copies the result back.  Return value: 0, or the CUDA error code.
// Timed variants run the call `iters` times over `copies` device copies of the large operand taken in turn (so
// that a matrix smaller than the L2 cache still streams from HBM) and report the mean microseconds per call.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <vector>
#include "jllm_kernels.h"

namespace jllm { void quantize_q8_1(const half* x, void* y, int K, cudaStream_t stream); }   // src/kernels/gemv_q4.cu:468

namespace {
struct Buf {
    void* p = nullptr;
    Buf(size_t bytes, const void* host = nullptr) {
        if (cudaMalloc(&p, bytes ? bytes : 1) != cudaSuccess) { p = nullptr; return; }
        if (host) cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice); else cudaMemset(p, 0, bytes);
    }
    ~Buf() { if (p) cudaFree(p); }
    template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};
struct Copies {     // `n` device copies of one host image
    std::vector<void*> v;
    Copies(const void* host, size_t bytes, int n) {
        for (int i = 0; i < (n < 1 ? 1 : n); ++i) {
            void* p = nullptr;
            if (cudaMalloc(&p, bytes) != cudaSuccess) break;
            cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice);
            v.push_back(p);
        }
    }
    ~Copies() { for (void* p : v) cudaFree(p); }
    const void* at(int i) const { return v[(size_t)i % v.size()]; }
};
int finish() { cudaError_t e = cudaDeviceSynchronize(); if (e == cudaSuccess) e = cudaGetLastError(); return (int)e; }

template <class F> float time_us(int iters, F&& call) {
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    for (int i = 0; i < 3; ++i) call(i);
    cudaDeviceSynchronize();
    cudaEventRecord(a);
    for (int i = 0; i < iters; ++i) call(i + 3);
    cudaEventRecord(b); cudaEventSynchronize(b);
    float ms = 0.f; cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    return ms * 1000.f / (float)iters;
}
}  // namespace

extern "C" {

// quantize_q8_1 (src/kernels/gemv_q4.cu:445-470): out = K/32 blocks of 36 bytes {fp16 d, fp16 s, int8 qs[32]}
int refgpu_quantize_q8_1(uint8_t* out, const uint16_t* x, int K) {
    Buf dx((size_t)K * 2, x), dy((size_t)K / 32 * 36);
    jllm::quantize_q8_1(dx.as<half>(), dy.p, K, 0);
    int rc = finish();
    cudaMemcpy(out, dy.p, (size_t)K / 32 * 36, cudaMemcpyDeviceToHost);
    return rc;
}

// gemv_quant / gemv_quant_add / gemv_quant_f32 (src/kernels/gemv_q4.cu:2633-2775).  mode 0: y half; 1: y half with
// residual; 2: y float.  `us` (may be null) receives the mean time of `iters` calls over `copies` copies of W.
int refgpu_gemv(void* y, const void* W, long long wbytes, int type, const uint16_t* x, const uint16_t* residual,
                int M, int K, int mode, int iters, int copies, float* us) {
    Copies w(W, (size_t)wbytes, us ? copies : 1);
    if (w.v.empty()) return (int)cudaErrorMemoryAllocation;
    Buf dx((size_t)K * 2, x), dr((size_t)M * 2, residual), dy((size_t)M * 4);
    auto call = [&](int i) {
        if (mode == 0) jllm::gemv_quant(dy.as<half>(), w.at(i), type, dx.as<half>(), M, K, 0);
        else if (mode == 1) jllm::gemv_quant_add(dy.as<half>(), w.at(i), type, dx.as<half>(), dr.as<half>(), M, K, 0);
        else jllm::gemv_quant_f32(dy.as<float>(), w.at(i), type, dx.as<half>(), M, K, 0);
    };
    call(0);
    int rc = finish();
    cudaMemcpy(y, dy.p, (size_t)M * (mode == 2 ? 4 : 2), cudaMemcpyDeviceToHost);
    if (rc == 0 && us) { *us = time_us(iters, call); rc = finish(); }
    return rc;
}

// gemv_quant_pair / gemv_quant_triple (src/kernels/gemv_q4.cu:2720-2753): n = 2 or 3 matrices sharing x
int refgpu_gemv_multi(int n, uint16_t* const* ys, const void* const* Ws, const long long* wbytes, const int* types, const int* Ms,
                      const uint16_t* x, int K, int iters, int copies, float* us) {
    if (n < 2 || n > 3) return -1;
    Copies w0(Ws[0], (size_t)wbytes[0], us ? copies : 1), w1(Ws[1], (size_t)wbytes[1], us ? copies : 1);
    Copies w2(Ws[n - 1], (size_t)wbytes[n - 1], us ? copies : 1);
    if (w0.v.empty() || w1.v.empty() || w2.v.empty()) return (int)cudaErrorMemoryAllocation;
    Buf dx((size_t)K * 2, x), y0((size_t)Ms[0] * 2), y1((size_t)Ms[1] * 2), y2((size_t)Ms[n - 1] * 2);
    auto call = [&](int i) {
        if (n == 2) jllm::gemv_quant_pair(y0.as<half>(), w0.at(i), types[0], Ms[0], y1.as<half>(), w1.at(i), types[1], Ms[1], dx.as<half>(), K, 0);
        else jllm::gemv_quant_triple(y0.as<half>(), w0.at(i), types[0], Ms[0], y1.as<half>(), w1.at(i), types[1], Ms[1],
                                     y2.as<half>(), w2.at(i), types[2], Ms[2], dx.as<half>(), K, 0);
    };
    call(0);
    int rc = finish();
    cudaMemcpy(ys[0], y0.p, (size_t)Ms[0] * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(ys[1], y1.p, (size_t)Ms[1] * 2, cudaMemcpyDeviceToHost);
    if (n == 3) cudaMemcpy(ys[2], y2.p, (size_t)Ms[2] * 2, cudaMemcpyDeviceToHost);
    if (rc == 0 && us) { *us = time_us(iters, call); rc = finish(); }
    return rc;
}

// gemm_quant_batched (src/kernels/gemv_q4.cu:2478-2517): y[N x M] = x[N x K] . W^T
int refgpu_gemm_batched(uint16_t* y, const void* W, long long wbytes, int type, const uint16_t* x, int M, int N, int K,
                        int iters, float* us) {
    Buf dw((size_t)wbytes, W), dx((size_t)N * K * 2, x), dy((size_t)N * M * 2);
    if (!dw.p || !dx.p || !dy.p) return (int)cudaErrorMemoryAllocation;
    auto call = [&](int) { jllm::gemm_quant_batched(dy.as<half>(), dw.p, type, dx.as<half>(), M, N, K, 0); };
    call(0);
    int rc = finish();
    cudaMemcpy(y, dy.p, (size_t)N * M * 2, cudaMemcpyDeviceToHost);
    if (rc == 0 && us) { *us = time_us(iters, call); rc = finish(); }
    return rc;
}

// flash_attention_decode with an INT8 cache (src/kernels/attention.cu:1036-1137).  k, v: int8 [L][n_kv][hd];
// ks, vs: fp32 [L][n_kv].
int refgpu_attention_decode(uint16_t* out, const uint16_t* q, const int8_t* k, const int8_t* v, const float* ks, const float* vs,
                            int n_heads, int n_kv, int hd, int L, float scale, int iters, int copies, float* us) {
    const size_t kvb = (size_t)L * n_kv * hd;
    Copies dk(k, kvb, us ? copies : 1), dv(v, kvb, us ? copies : 1);
    if (dk.v.empty() || dv.v.empty()) return (int)cudaErrorMemoryAllocation;
    Buf dq((size_t)n_heads * hd * 2, q), dks((size_t)L * n_kv * 4, ks), dvs((size_t)L * n_kv * 4, vs), dout((size_t)n_heads * hd * 2);
    auto call = [&](int i) {
        jllm::flash_attention_decode(dout.as<half>(), dq.as<half>(), dk.at(i), dv.at(i), n_heads, n_kv, hd, hd, L, scale, true,
                                     dks.as<float>(), dvs.as<float>(), 0, 0);
    };
    call(0);
    int rc = finish();
    cudaMemcpy(out, dout.p, (size_t)n_heads * hd * 2, cudaMemcpyDeviceToHost);
    if (rc == 0 && us) { *us = time_us(iters, call); rc = finish(); }
    return rc;
}

// flash_attention_prefill_batched with an INT8 cache (src/kernels/attention.cu:617-697): N queries, causal from start_pos
int refgpu_attention_prefill(uint16_t* out, const uint16_t* q, const int8_t* k, const int8_t* v, const float* ks, const float* vs,
                             int n_heads, int n_kv, int hd, int N, int start_pos, float scale, int iters, float* us) {
    const int L = start_pos + N;
    const size_t kvb = (size_t)L * n_kv * hd;
    Buf dk(kvb, k), dv(kvb, v), dq((size_t)N * n_heads * hd * 2, q), dks((size_t)L * n_kv * 4, ks), dvs((size_t)L * n_kv * 4, vs);
    Buf dout((size_t)N * n_heads * hd * 2);
    auto call = [&](int) {
        jllm::flash_attention_prefill_batched(dout.as<half>(), dq.as<half>(), dk.p, dv.p, n_heads, n_kv, hd, hd, N, start_pos, scale,
                                              true, dks.as<float>(), dvs.as<float>(), 0, 0);
    };
    call(0);
    int rc = finish();
    cudaMemcpy(out, dout.p, (size_t)N * n_heads * hd * 2, cudaMemcpyDeviceToHost);
    if (rc == 0 && us) { *us = time_us(iters, call); rc = finish(); }
    return rc;
}

// fused_rmsnorm_residual (src/kernels/fused_norm.cu:103-165); residual may be null; weight fp32
int refgpu_rmsnorm(uint16_t* out, const uint16_t* x, const uint16_t* residual, const float* w, int rows, int dim, float eps) {
    Buf dx((size_t)rows * dim * 2, x), dr((size_t)rows * dim * 2, residual), dw((size_t)dim * 4, w), dout((size_t)rows * dim * 2);
    jllm::fused_rmsnorm_residual(dout.as<half>(), dx.as<half>(), residual ? dr.as<half>() : nullptr, dw.p, rows, dim, eps, true, 0);
    int rc = finish();
    cudaMemcpy(out, dout.p, (size_t)rows * dim * 2, cudaMemcpyDeviceToHost);
    return rc;
}

// rope_inplace (src/kernels/rope.cu:427-444): q [n_heads x hd] and k [n_kv x hd] rotated in place
int refgpu_rope(uint16_t* q, uint16_t* k, int n_heads, int n_kv, int hd, int pos, float theta, int neox) {
    Buf dq((size_t)n_heads * hd * 2, q), dk((size_t)n_kv * hd * 2, k);
    jllm::rope_inplace(dq.as<half>(), dk.as<half>(), n_heads, n_kv, hd, pos, theta, neox != 0, 0);
    int rc = finish();
    cudaMemcpy(q, dq.p, (size_t)n_heads * hd * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(k, dk.p, (size_t)n_kv * hd * 2, cudaMemcpyDeviceToHost);
    return rc;
}

// fp16_to_int8 (src/kernels/convert.cu:71-75)
int refgpu_fp16_to_int8(int8_t* dst, float* scales, const uint16_t* src, int rows, int cols) {
    Buf ds((size_t)rows * cols * 2, src), dd((size_t)rows * cols), dsc((size_t)rows * 4);
    jllm::fp16_to_int8(dd.as<int8_t>(), dsc.as<float>(), ds.as<half>(), rows, cols, 0);
    int rc = finish();
    cudaMemcpy(dst, dd.p, (size_t)rows * cols, cudaMemcpyDeviceToHost);
    cudaMemcpy(scales, dsc.p, (size_t)rows * 4, cudaMemcpyDeviceToHost);
    return rc;
}

// fused_swiglu (src/kernels/convert.cu:106-112)
int refgpu_swiglu(uint16_t* out, const uint16_t* g, const uint16_t* u, int rows, int dim) {
    Buf dg((size_t)rows * dim * 2, g), du((size_t)rows * dim * 2, u), dout((size_t)rows * dim * 2);
    jllm::fused_swiglu(dout.as<half>(), dg.as<half>(), du.as<half>(), rows, dim, 0);
    int rc = finish();
    cudaMemcpy(out, dout.p, (size_t)rows * dim * 2, cudaMemcpyDeviceToHost);
    return rc;
}

// dequant_embedding_row (src/kernels/gemv_q4.cu:2777-2809)
int refgpu_embedding_row(uint16_t* dst, const void* W, long long wbytes, int type, int token, int hidden) {
    Buf dw((size_t)wbytes, W), dd((size_t)hidden * 2);
    const bool ok = jllm::dequant_embedding_row(dd.as<half>(), dw.p, type, token, hidden, 0);
    int rc = finish();
    cudaMemcpy(dst, dd.p, (size_t)hidden * 2, cudaMemcpyDeviceToHost);
    return ok ? rc : -2;
}

}  // extern "C"
