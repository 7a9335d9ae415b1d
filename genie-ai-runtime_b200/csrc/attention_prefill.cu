// attention_prefill.cu — causal prefill attention over an INT8 KV cache, head_dim 128, with query tiling, sm_100a.
//
// Replaces the reference's flash_attention_prefill_batched INT8 path (src/kernels/attention.cu:617-697 -> kernel
// :382-514: one CTA per (head, token), every token re-reading all of its keys).  Same mathematics — query token t at
// absolute position start+t attends keys [0, start+t]:  s_j = scale * Σ_d q_d (k8_jd ks_j), softmax, o_d = Σ_j p_j (v8_jd vs_j).
//   * one CTA per (kv head, tile of PQ query tokens): every K/V byte fetched is used by PQ tokens x the 2..4 query heads
//     of the GQA group, so the O(N^2) key traffic of the reference drops by PQ x G;
//   * K/V tiles of 32 keys arrive by 2-D TMA tensor copies (128-byte swizzle) into per-warp rings, as in the decode
//     kernel (attention_tma.cu); the four warps of a CTA take the tiles in turn and keep private online-softmax states
//     for all PQ tokens, merged through shared memory at the end;
//   * QK^T and PV on the int8 tensor-core path (mma.sync m16n8k32), q and the softmax weights as 16-bit fixed point in two
//     int8 planes; each K fragment and each transposed V fragment is loaded once and multiplied against all PQ tokens;
//   * the causal mask is per token; a token skips the tiles that lie wholly after it.
#include "attention.cuh"
#include <cfloat>
#include <cuda.h>

namespace jb {

constexpr int AP_WARPS  = 4;
constexpr int AP_TILE   = 32;
constexpr int AP_STAGES = 2;
constexpr int AP_HD     = 128;
constexpr int AP_PQ     = 2;                          // query tokens per CTA: with 4 the accumulators took 232 registers (two CTAs per SM) and the
                                                      // kernel, bound by instruction latency, ran 10 % slower (2048 tokens: 474 against 427 us); the 69 KB of shared
                                                      // memory allow three CTAs per SM, so the register bound is the one for three (412 us)
constexpr int AP_TILE_BYTES  = AP_TILE * AP_HD;
constexpr int AP_STAGE_BYTES = 2 * AP_TILE_BYTES;
constexpr int AP_RING_BYTES  = AP_WARPS * AP_STAGES * AP_STAGE_BYTES;          // 64 KB
constexpr int AP_WSM_BYTES   = AP_WARPS * AP_PQ * 256;                         // PV weight bytes per (warp, token)
constexpr int AP_QPL_BYTES   = AP_PQ * 4 * 2 * AP_HD;                          // query planes [token][head][plane][128]
constexpr int AP_SMEM = AP_RING_BYTES + AP_WSM_BYTES + AP_QPL_BYTES + 256 + 1024;

struct ApArgs {
    __half* out; const __half* q; const float* ks; const float* vs;
    int n_heads, n_kv, N, start; float scale; int* status;
};

__device__ __forceinline__ void ap_mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ap_transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&t)[4]) {
    const uint32_t u0 = __byte_perm(r0, r1, 0x5140), u1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t u2 = __byte_perm(r0, r1, 0x7362), u3 = __byte_perm(r2, r3, 0x7362);
    t[0] = __byte_perm(u0, u1, 0x5410); t[1] = __byte_perm(u0, u1, 0x7632);
    t[2] = __byte_perm(u2, u3, 0x5410); t[3] = __byte_perm(u2, u3, 0x7632);
}
__device__ __forceinline__ void ap_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ap_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t ap_lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t ap_swz(uint32_t tile, int row, int b) {
    return tile + (uint32_t)row * 128u + (uint32_t)((((b >> 4) ^ (row & 7)) << 4) | (b & 15));
}

template <int G>
__global__ void __launch_bounds__(AP_WARPS * 32, 3) attn_prefill_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                                                                        const ApArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full[AP_WARPS][AP_STAGES];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x, tq0 = blockIdx.y * AP_PQ;                        // first query token of this CTA
    const int nq = min(AP_PQ, a.N - tq0);

    const uint32_t ring0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (ring0 - smem_u32(smem_raw));
    const uint32_t wring = ring0 + (uint32_t)warp * AP_STAGES * AP_STAGE_BYTES;
    uint8_t* wsm = smem + AP_RING_BYTES + warp * (AP_PQ * 256);                  // [token][8 columns][32 keys] int8
    int8_t*  qpl = reinterpret_cast<int8_t*>(smem + AP_RING_BYTES + AP_WSM_BYTES);
    float*   qsc = reinterpret_cast<float*>(smem + AP_RING_BYTES + AP_WSM_BYTES + AP_QPL_BYTES);     // [token][head]

    if (lane == 0) { for (int s = 0; s < AP_STAGES; ++s) mbar_init(&full[warp][s], 1); }
    if (tid == 0) {
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
    }
    __syncthreads();
    pdl_launch();
    pdl_wait();

    const int kv_end = a.start + tq0 + nq;                                       // keys [0, kv_end) are visible to the last token
    const int ntiles_cta = (kv_end + AP_TILE - 1) / AP_TILE;
    const int my_tiles = ntiles_cta > warp ? (ntiles_cta - warp + AP_WARPS - 1) / AP_WARPS : 0;
    auto issue = [&](int it) {
        const int t0 = (warp + it * AP_WARPS) * AP_TILE;
        const uint32_t st = wring + (uint32_t)(it % AP_STAGES) * AP_STAGE_BYTES;
        uint64_t* bar = &full[warp][it % AP_STAGES];
        mbar_expect_tx(bar, (uint32_t)AP_STAGE_BYTES);
        ap_tma_2d(st, &kmap, kvh * AP_HD, t0, bar);
        ap_tma_2d(st + AP_TILE_BYTES, &vmap, kvh * AP_HD, t0, bar);
    };
    if (lane == 0)
        for (int it = 0; it < AP_STAGES && it < my_tiles; ++it) issue(it);
    // lane l fetches the scales of key t0 + l (one load per array per tile); the lanes pick their four keys' with shuffles
    auto load_scales = [&](int it, float& kl, float& vl) {
        const int key = (warp + it * AP_WARPS) * AP_TILE + lane;
        const bool ok = it < my_tiles && key < kv_end;
        kl = ok ? __ldcg(a.ks + (size_t)key * a.n_kv + kvh) : 0.f;
        vl = ok ? __ldcg(a.vs + (size_t)key * a.n_kv + kvh) : 0.f;
    };
    float nks, nvs;
    load_scales(0, nks, nvs);

    // ── query planes of the PQ tokens x G heads: warp w quantises the (token, head) pairs w, w+4, ... ──
    for (int pr = warp; pr < AP_PQ * G; pr += AP_WARPS) {
        const int t = pr / G, h = pr % G;
        uint32_t hi = 0, lo = 0; float dq = 0.f;
        if (t < nq) {
            const __half* qh = a.q + ((size_t)(tq0 + t) * a.n_heads + kvh * G + h) * AP_HD + 4 * lane;
            float v[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __half2float(qh[i]);
            const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
            dq = amax / 32512.0f;
            const float id = dq > 0.f ? 1.0f / dq : 0.f;
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int Q = max(-32512, min(32512, __float2int_rn(v[i] * id)));
                const int l8 = (int)(int8_t)(Q & 0xFF), h8 = (Q - l8) >> 8;
                hi |= (uint32_t)(h8 & 0xFF) << (8 * i); lo |= (uint32_t)(l8 & 0xFF) << (8 * i);
            }
        }
        reinterpret_cast<uint32_t*>(qpl + ((t * 4 + h) * 2 + 0) * AP_HD)[lane] = hi;
        reinterpret_cast<uint32_t*>(qpl + ((t * 4 + h) * 2 + 1) * AP_HD)[lane] = lo;
        if (lane == 0) qsc[t * 4 + h] = dq * a.scale * 1.4426950408889634f;     // scores in units of log2
    }
    __syncthreads();
    // B fragments of QK^T for every token: column n = g is (head g>>1, plane g&1)
    uint32_t bq[AP_PQ][4][2];
    float sfac[AP_PQ];
    const bool head_live = c < G;
    #pragma unroll
    for (int t = 0; t < AP_PQ; ++t) {
        const bool live = (g >> 1) < G;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(qpl + ((t * 4 + (g >> 1)) * 2 + (g & 1)) * AP_HD);
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) { bq[t][ks][0] = live ? src[8 * ks + c] : 0u; bq[t][ks][1] = live ? src[8 * ks + 4 + c] : 0u; }
        sfac[t] = head_live ? qsc[t * 4 + c] : 0.f;
    }

    float m_run[AP_PQ], l_run[AP_PQ], O[AP_PQ][16];
    #pragma unroll
    for (int t = 0; t < AP_PQ; ++t) {
        m_run[t] = -FLT_MAX; l_run[t] = 0.f;
        #pragma unroll
        for (int i = 0; i < 16; ++i) O[t][i] = 0.f;
    }
    bool timed_out = false;

    for (int it = 0; it < my_tiles; ++it) {
        const int t0 = (warp + it * AP_WARPS) * AP_TILE;
        const uint32_t Kt = wring + (uint32_t)(it % AP_STAGES) * AP_STAGE_BYTES, Vt = Kt + AP_TILE_BYTES;
        float ksv[4], vsv[4];
        #pragma unroll
        for (int r = 0; r < 4; ++r) {
            ksv[r] = __shfl_sync(0xFFFFFFFFu, nks, g + 8 * r);
            vsv[r] = __shfl_sync(0xFFFFFFFFu, nvs, g + 8 * r);
        }
        load_scales(it + 1, nks, nvs);
        if (!timed_out && !mbar_wait_bounded(&full[warp][it % AP_STAGES], (it / AP_STAGES) & 1)) timed_out = true;

        // ── S = K Q^T for all tokens: each K fragment is loaded once ──
        int sacc[AP_PQ][2][4];
        #pragma unroll
        for (int t = 0; t < AP_PQ; ++t)
            #pragma unroll
            for (int mt = 0; mt < 2; ++mt) { sacc[t][mt][0] = sacc[t][mt][1] = sacc[t][mt][2] = sacc[t][mt][3] = 0; }
        #pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const uint32_t r0 = Kt + (uint32_t)(16 * mt + g) * 128u + 4u * c;
            #pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t o0 = (uint32_t)(((2 * ks) ^ g) << 4), o1 = (uint32_t)(((2 * ks + 1) ^ g) << 4);
                uint32_t af[4];
                af[0] = ap_lds32(r0 + o0); af[1] = ap_lds32(r0 + 8 * 128 + o0);
                af[2] = ap_lds32(r0 + o1); af[3] = ap_lds32(r0 + 8 * 128 + o1);
                #pragma unroll
                for (int t = 0; t < AP_PQ; ++t) ap_mma_s8(sacc[t][mt], af, bq[t][ks][0], bq[t][ks][1]);
            }
        }
        // ── per token: causal mask, online softmax relative to the tile maximum, weights as two int8 planes ──
        float corr[AP_PQ], dwt[AP_PQ];
        #pragma unroll
        for (int t = 0; t < AP_PQ; ++t) {
            const int last_key = a.start + tq0 + t;                              // token t sees keys <= last_key
            const bool on = t < nq && t0 <= last_key;                            // warp-uniform
            corr[t] = 1.f; dwt[t] = 0.f;
            uint8_t* wt = wsm + t * 256;
            if (!on) continue;
            float sc[4];
            sc[0] = (float)(sacc[t][0][0] * 256 + sacc[t][0][1]) * (sfac[t] * ksv[0]);
            sc[1] = (float)(sacc[t][0][2] * 256 + sacc[t][0][3]) * (sfac[t] * ksv[1]);
            sc[2] = (float)(sacc[t][1][0] * 256 + sacc[t][1][1]) * (sfac[t] * ksv[2]);
            sc[3] = (float)(sacc[t][1][2] * 256 + sacc[t][1][3]) * (sfac[t] * ksv[3]);
            #pragma unroll
            for (int r = 0; r < 4; ++r) if (t0 + g + 8 * r > last_key) sc[r] = -INFINITY;
            float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
            #pragma unroll
            for (int o = 4; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, o));
            const float m_new = fmaxf(m_run[t], tmax);
            corr[t] = ap_exp2(m_run[t] - m_new);
            const float tfac = ap_exp2(tmax - m_new);
            m_run[t] = m_new;
            // weights p_j * vs_j as 16-bit fixed point relative to the LARGEST weight this token gives a key of the tile (keys
            // the token cannot see, or whose V scale is far larger, must not cost it precision: early tokens see few keys)
            float psum = 0.f, pw[4], wmax = 0.f;
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float pv = ap_exp2(sc[r] - tmax);
                psum += pv;
                pw[r] = pv * vsv[r];
                wmax = fmaxf(wmax, pw[r]);
            }
            #pragma unroll
            for (int o = 4; o < 32; o <<= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xFFFFFFFFu, wmax, o));
            const float dw = wmax / 32512.0f, idw = dw > 0.f ? 1.0f / dw : 0.f;
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int W = head_live ? min(32512, __float2int_rn(pw[r] * idw)) : 0;
                const int l8 = (int)(int8_t)(W & 0xFF), h8 = (W - l8) >> 8;
                const int key = g + 8 * r;
                wt[(2 * c) * AP_TILE + key] = (uint8_t)h8;
                wt[(2 * c + 1) * AP_TILE + key] = (uint8_t)l8;
            }
            l_run[t] = l_run[t] * corr[t] + psum * tfac;
            dwt[t] = dw * tfac;
        }
        __syncwarp();
        uint32_t bw[AP_PQ][2];
        #pragma unroll
        for (int t = 0; t < AP_PQ; ++t)
            #pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                const uint8_t* wr = wsm + t * 256 + g * AP_TILE + 16 * kb + 2 * c;
                bw[t][kb] = (uint32_t)*reinterpret_cast<const unsigned short*>(wr) | ((uint32_t)*reinterpret_cast<const unsigned short*>(wr + 8) << 16);
            }
        // ── O += V^T W for all tokens: each transposed V fragment is built once ──
        #pragma unroll
        for (int s = 0; s < 2; ++s) {
            uint32_t T[2][2][4];
            #pragma unroll
            for (int kb = 0; kb < 2; ++kb)
                #pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int row = 16 * kb + 2 * c, b = 4 * (g + 8 * hf + 16 * s);
                    ap_transpose4x4(ap_lds32(ap_swz(Vt, row, b)), ap_lds32(ap_swz(Vt, row + 1, b)),
                                    ap_lds32(ap_swz(Vt, row + 8, b)), ap_lds32(ap_swz(Vt, row + 9, b)), T[kb][hf]);
                }
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t af[4] = { T[0][0][j], T[0][1][j], T[1][0][j], T[1][1][j] };
                #pragma unroll
                for (int t = 0; t < AP_PQ; ++t) {
                    if (dwt[t] == 0.f && corr[t] == 1.f) continue;              // token not touched by this tile (warp-uniform)
                    int acc[4] = { 0, 0, 0, 0 };
                    ap_mma_s8(acc, af, bw[t][0], bw[t][1]);
                    O[t][(s * 4 + j) * 2 + 0] = O[t][(s * 4 + j) * 2 + 0] * corr[t] + dwt[t] * (float)(acc[0] * 256 + acc[1]);
                    O[t][(s * 4 + j) * 2 + 1] = O[t][(s * 4 + j) * 2 + 1] * corr[t] + dwt[t] * (float)(acc[2] * 256 + acc[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && it + AP_STAGES < my_tiles) { fence_proxy_async(); issue(it + AP_STAGES); }
    }
    if (timed_out && lane == 0) atomicExch(a.status, JB_ERR_TIMEOUT);

    // ── merge the four warps token by token and write the outputs ──
    float* sm_m = reinterpret_cast<float*>(smem);           // [warp][4]
    float* sm_l = sm_m + AP_WARPS * 4;
    float* sm_o = sm_l + AP_WARPS * 4;                      // [warp][4][128]
    #pragma unroll
    for (int t = 0; t < AP_PQ; ++t) {
        float l = l_run[t];
        #pragma unroll
        for (int o = 4; o < 32; o <<= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o);
        __syncthreads();                                    // rings (first token) or the previous token's merge are done with
        if (head_live) {
            if (g == 0) { sm_m[warp * 4 + c] = m_run[t]; sm_l[warp * 4 + c] = l; }
            #pragma unroll
            for (int s = 0; s < 2; ++s)
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    sm_o[(warp * 4 + c) * AP_HD + 4 * (g + 16 * s) + j]     = O[t][(s * 4 + j) * 2 + 0];
                    sm_o[(warp * 4 + c) * AP_HD + 4 * (g + 8 + 16 * s) + j] = O[t][(s * 4 + j) * 2 + 1];
                }
        }
        __syncthreads();
        if (t < nq) {
            const int d = tid;
            for (int h = 0; h < G; ++h) {
                float M = -FLT_MAX;
                #pragma unroll
                for (int w = 0; w < AP_WARPS; ++w) M = fmaxf(M, sm_m[w * 4 + h]);
                float L = 0.f, acc = 0.f;
                #pragma unroll
                for (int w = 0; w < AP_WARPS; ++w) {
                    const float e = ap_exp2(sm_m[w * 4 + h] - M);
                    L += sm_l[w * 4 + h] * e;
                    acc += sm_o[(w * 4 + h) * AP_HD + d] * e;
                }
                a.out[((size_t)(tq0 + t) * a.n_heads + kvh * G + h) * AP_HD + d] = __float2half_rn(L > 0.f ? acc / L : 0.f);
            }
        }
    }
}

bool attention_prefill_fast_applies(const AttnCall& c) {
    const int G = c.n_kv > 0 ? c.n_heads / c.n_kv : 0;
    return c.kv_int8 && c.hd == AP_HD && c.chd == AP_HD && c.window == 0 && c.causal_start >= 0 && (G == 1 || G == 2 || G == 4) &&
           c.n_heads == G * c.n_kv && c.k && c.v && c.ks && c.vs && !((uintptr_t)c.k & 15) && !((uintptr_t)c.v & 15) && c.batch > 0;
}

// c.batch = number of query tokens, c.causal_start = absolute position of the first
int launch_attention_prefill_fast(const AttnCall& c, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    const int N = c.batch, rows = c.causal_start + N;
    alignas(64) CUtensorMap kmap, vmap;
    if (!attn_tma_encode(&kmap, c.k, rows, c.n_kv) || !attn_tma_encode(&vmap, c.v, rows, c.n_kv))
        return set_error(JB_ERR_CUDA, "prefill attention: tensor map for the KV cache refused");
    ApArgs a = { c.out, c.q, c.ks, c.vs, c.n_heads, c.n_kv, N, c.causal_start, c.scale, cx->d_status };
    const int G = c.n_heads / c.n_kv;
    auto kern = G == 4 ? attn_prefill_kernel<4> : (G == 2 ? attn_prefill_kernel<2> : attn_prefill_kernel<1>);
    const int gi = G == 4 ? 2 : (G == 2 ? 1 : 0);
    if (!cx->attn_prefill_attr[gi]) { JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM)); cx->attn_prefill_attr[gi] = true; }
    JB_CUDA(launch_k(kern, dim3(c.n_kv, (N + AP_PQ - 1) / AP_PQ), dim3(AP_WARPS * 32), (size_t)AP_SMEM, st, pdl_enabled(), kmap, vmap, a));
    count_launch();
    return JB_OK;
}

}  // namespace jb
