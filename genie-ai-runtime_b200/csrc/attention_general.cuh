// attention_general.cuh — the general attention slice: one query head against keys [kv0, kv1) of an FP16 or INT8
// cache of any head size up to 512, optional sliding window, cache slot stride >= head size.
//
// Same mathematics as the reference's decode / split-K / prefill kernels (src/kernels/attention.cu:244-375, :382-514,
// :837-941: s_j = scale * q . k_j with k = k8 * ks for INT8, online softmax, o = Σ p_j v_j with v = v8 * vs), arranged
// differently: the 32 lanes of a warp split the head dimension (dims lane, lane + 32, ...), every warp walks its own
// strided run of keys and keeps its running maximum, sum and output accumulators in REGISTERS — no shared score tile,
// no CTA-wide barrier per tile — and the warps' states are merged once through shared memory at the end.
// Used by the general kernels of attention.cu and by the allocation-free entry point.
#pragma once
#include "common.cuh"
#include <cfloat>

namespace jb {

constexpr int AG_WARPS = 4;
constexpr int AG_THREADS = AG_WARPS * 32;
constexpr int AG_MAXD = 16;                 // dims per lane: head sizes up to 512

struct AgCache { const void* k; const void* v; const float* ks; const float* vs; int n_kv, chd, kv_int8, window; };

inline size_t ag_smem_bytes(int hd) { return (size_t)AG_WARPS * (hd + 2) * sizeof(float); }

// Runs on all AG_THREADS threads of the CTA.  On return M and L hold the slice's running maximum and sum (the same
// on every thread; M = -FLT_MAX for an empty slice) and emit(d, acc_d) has been called once per dimension d with the
// unnormalised output, each d by exactly one thread.  `sm` = ag_smem_bytes(hd) of shared memory.
template <class Emit>
__device__ __forceinline__ void ag_slice(const __half* q, const AgCache& c, int kvh, int hd, int seq, int kv0, int kv1, float scale,
                                         float* sm, float& M, float& L, Emit emit) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t row = (size_t)c.n_kv * c.chd, off = (size_t)kvh * c.chd;
    float qr[AG_MAXD], acc[AG_MAXD];
    #pragma unroll
    for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; qr[i] = d < hd ? __half2float(q[d]) : 0.f; acc[i] = 0.f; }
    float m = -FLT_MAX, l = 0.f;
    const int first = c.window > 0 ? max(kv0, seq - c.window) : kv0;      // keys before the window contribute nothing
    for (int p = first + warp; p < kv1; p += AG_WARPS) {
        float kd[AG_MAXD], dot = 0.f;
        if (c.kv_int8) {
            const int8_t* kr = reinterpret_cast<const int8_t*>(c.k) + (size_t)p * row + off;
            const float sc = c.ks ? c.ks[(size_t)p * c.n_kv + kvh] : 1.0f;
            #pragma unroll
            for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; kd[i] = d < hd ? (float)kr[d] * sc : 0.f; }
        } else {
            const __half* kr = reinterpret_cast<const __half*>(c.k) + (size_t)p * row + off;
            #pragma unroll
            for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; kd[i] = d < hd ? __half2float(kr[d]) : 0.f; }
        }
        #pragma unroll
        for (int i = 0; i < AG_MAXD; ++i) dot += qr[i] * kd[i];
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, s), corr = expf(m - m_new), pw = expf(s - m_new);
        m = m_new;
        l = l * corr + pw;
        if (c.kv_int8) {
            const int8_t* vr = reinterpret_cast<const int8_t*>(c.v) + (size_t)p * row + off;
            const float sc = c.vs ? c.vs[(size_t)p * c.n_kv + kvh] : 1.0f;
            #pragma unroll
            for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; if (d < hd) acc[i] = acc[i] * corr + pw * ((float)vr[d] * sc); }
        } else {
            const __half* vr = reinterpret_cast<const __half*>(c.v) + (size_t)p * row + off;
            #pragma unroll
            for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; if (d < hd) acc[i] = acc[i] * corr + pw * __half2float(vr[d]); }
        }
    }
    // merge the warps' states
    float* sm_m = sm; float* sm_l = sm + AG_WARPS; float* sm_o = sm + 2 * AG_WARPS;     // [warp][hd]
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
    #pragma unroll
    for (int i = 0; i < AG_MAXD; ++i) { const int d = lane + 32 * i; if (d < hd) sm_o[warp * hd + d] = acc[i]; }
    __syncthreads();
    M = -FLT_MAX;
    #pragma unroll
    for (int w = 0; w < AG_WARPS; ++w) M = fmaxf(M, sm_m[w]);
    float e[AG_WARPS];
    L = 0.f;
    #pragma unroll
    for (int w = 0; w < AG_WARPS; ++w) { e[w] = sm_l[w] > 0.f ? expf(sm_m[w] - M) : 0.f; L += sm_l[w] * e[w]; }
    for (int d = tid; d < hd; d += AG_THREADS) {
        float o = 0.f;
        #pragma unroll
        for (int w = 0; w < AG_WARPS; ++w) o += sm_o[w * hd + d] * e[w];
        emit(d, o);
    }
}

// out = Σ_s acc_s e^{m_s-M} / Σ_s l_s e^{m_s-M} over the partial records (m, l, acc[hd]) of one head (reference :944-969)
__device__ __forceinline__ void ag_merge_slices(__half* out, const float* pb, int hd, int n_splits) {
    float M = -FLT_MAX;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, pb[(size_t)s * (hd + 2)]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) L += pb[(size_t)s * (hd + 2) + 1] * expf(pb[(size_t)s * (hd + 2)] - M);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) acc += pb[(size_t)s * (hd + 2) + 2 + d] * expf(pb[(size_t)s * (hd + 2)] - M);
        out[d] = __float2half_rn(acc * inv);
    }
}

}  // namespace jb
