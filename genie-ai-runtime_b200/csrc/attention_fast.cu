// attention_fast.cu — split-K decode attention over an INT8 KV cache, head_dim 128, for sm_100a.
//
// Replaces the reference's flash_decode_splitk_partial_kernel / flash_decode_reduce_kernel
// (src/kernels/attention.cu:837-969) for the INT8 cache layout [pos][kv_head][128] with one fp32 scale per
// (pos, kv_head).  Same mathematics — s_j = scale * Σ_d q_d (k8_jd ks_j), online softmax, o_d = Σ_j p_j (v8_jd vs_j) —
// arranged for B200:
//   * one CTA per (kv head, KV slice): the 2..4 query heads of a GQA group share every K/V byte that is read;
//   * K/V rows travel HBM -> shared memory as 128-byte TMA bulk copies (cp.async.bulk + mbarrier), each warp
//     owning a private ring of 32-key tiles, so no CTA-wide barrier sits in the loop;
//   * QK^T and PV run on the int8 tensor-core path (mma.sync m16n8k32): q and the softmax weights are held as
//     16-bit fixed point split into two int8 planes (hi, lo), which keeps the integer dots exact and the result
//     within ~2^-15 of the fp32 arithmetic of the reference, far inside its fp16 output;
//   * V reaches the MMA transposed through 4x4 byte transposes in registers; the key order inside an MMA step
//     and the 144-byte row pitch are chosen so that every shared-memory read is bank-conflict free.
// A slice writes an unnormalised partial (m, l, acc[128]) per query head; attn_reduce_kernel merges slices.
#include "attention.cuh"
#include <cfloat>

namespace jb {

constexpr int AF_WARPS  = 4;
constexpr int AF_TILE   = 32;                       // keys per warp tile
constexpr int AF_PITCH  = 144;                      // bytes between key rows in shared memory (128 + 16)
constexpr int AF_STAGES = 3;
constexpr int AF_HD     = 128;
constexpr int AF_STAGE_BYTES = 2 * AF_TILE * AF_PITCH;                 // K tile + V tile
constexpr int AF_WARP_BYTES  = AF_STAGES * AF_STAGE_BYTES + 256;       // + the 8 x 32 weight bytes of the PV step
constexpr int AF_SMEM = AF_WARPS * AF_WARP_BYTES + 2048;               // + query planes and scales

struct AfArgs {
    __half* out; const __half* q;
    const int8_t* k; const int8_t* v; const float* ks; const float* vs;
    const void* const* k_list; const void* const* v_list; const float* const* ks_list; const float* const* vs_list; const int* seq_lens;
    int n_heads, n_kv, seq_len; const int* d_pos;
    float scale; int n_splits;
    float* part; int* status;
};

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// rows r0..r3 hold bytes (dim0..dim3) of four keys; t[j] = (key0..key3) bytes of dim j
__device__ __forceinline__ void transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&t)[4]) {
    const uint32_t u0 = __byte_perm(r0, r1, 0x5140), u1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t u2 = __byte_perm(r0, r1, 0x7362), u3 = __byte_perm(r2, r3, 0x7362);
    t[0] = __byte_perm(u0, u1, 0x5410); t[1] = __byte_perm(u0, u1, 0x7632);
    t[2] = __byte_perm(u2, u3, 0x5410); t[3] = __byte_perm(u2, u3, 0x7632);
}

template <int G>   // query heads per kv head: 1, 2 or 4
__global__ void __launch_bounds__(AF_WARPS * 32, 2) attn_fast_kernel(const AfArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[AF_WARPS][AF_STAGES];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x, split = blockIdx.y, z = blockIdx.z;

    uint8_t* wbase = smem + warp * AF_WARP_BYTES;
    uint8_t* wsm = wbase + AF_STAGES * AF_STAGE_BYTES;                     // [8 columns][32 keys] int8
    int8_t*  qpl = reinterpret_cast<int8_t*>(smem + AF_WARPS * AF_WARP_BYTES);   // [G][2 planes][128]
    float*   qsc = reinterpret_cast<float*>(smem + AF_WARPS * AF_WARP_BYTES + 1024);   // dq per head

    if (lane == 0) { for (int s = 0; s < AF_STAGES; ++s) mbar_init(&full[warp][s], 1); }
    if (tid == 0) fence_mbar_init();
    __syncthreads();
    pdl_wait();

    const int8_t* kc = a.k; const int8_t* vc = a.v; const float* ksp = a.ks; const float* vsp = a.vs;
    int seq = a.d_pos ? (*a.d_pos + 1) : a.seq_len;
    if (a.k_list) {
        kc = reinterpret_cast<const int8_t*>(a.k_list[z]); vc = reinterpret_cast<const int8_t*>(a.v_list[z]);
        ksp = a.ks_list[z]; vsp = a.vs_list[z]; seq = a.seq_lens[z];
    }
    int per = (seq + a.n_splits - 1) / a.n_splits;
    per = (per + AF_TILE - 1) / AF_TILE * AF_TILE;                           // slices start on tile boundaries
    const int kv0 = split * per, kv1 = min(kv0 + per, seq);
    const int ntiles_cta = kv1 > kv0 ? (kv1 - kv0 + AF_TILE - 1) / AF_TILE : 0;
    const int my_tiles = ntiles_cta > warp ? (ntiles_cta - warp + AF_WARPS - 1) / AF_WARPS : 0;
    const size_t row_stride = (size_t)a.n_kv * AF_HD;

    auto issue = [&](int it) {      // tile `it` of this warp -> stage it % AF_STAGES
        const int t0 = kv0 + (warp + it * AF_WARPS) * AF_TILE;
        const int nvalid = min(AF_TILE, kv1 - t0);
        uint8_t* st = wbase + (it % AF_STAGES) * AF_STAGE_BYTES;
        uint64_t* bar = &full[warp][it % AF_STAGES];
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)nvalid * 2u * AF_HD);
        __syncwarp();
        if (lane < nvalid) {
            const size_t off = (size_t)(t0 + lane) * row_stride + (size_t)kvh * AF_HD;
            bulk_g2s(st + lane * AF_PITCH, kc + off, AF_HD, bar);
            bulk_g2s(st + AF_TILE * AF_PITCH + lane * AF_PITCH, vc + off, AF_HD, bar);
        }
    };
    for (int it = 0; it < AF_STAGES && it < my_tiles; ++it) issue(it);

    // ── query planes: per head 16-bit fixed point, split into a high and a (signed) low byte ──
    if (warp < G) {
        const int head = kvh * G + warp;
        const __half* qh = a.q + ((size_t)z * a.n_heads + head) * AF_HD + 4 * lane;
        float v[4];
        #pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __half2float(qh[i]);
        const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
        const float dq = amax / 32512.0f, id = dq > 0.f ? 1.0f / dq : 0.f;
        uint32_t hi = 0, lo = 0;
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int Q = max(-32512, min(32512, __float2int_rn(v[i] * id)));
            const int l8 = (int)(int8_t)(Q & 0xFF), h8 = (Q - l8) >> 8;
            hi |= (uint32_t)(h8 & 0xFF) << (8 * i); lo |= (uint32_t)(l8 & 0xFF) << (8 * i);
        }
        reinterpret_cast<uint32_t*>(qpl + (warp * 2 + 0) * AF_HD)[lane] = hi;
        reinterpret_cast<uint32_t*>(qpl + (warp * 2 + 1) * AF_HD)[lane] = lo;
        if (lane == 0) qsc[warp] = dq * a.scale;
    }
    __syncthreads();
    // B fragments of QK^T: column n = g is (head g>>1, plane g&1); k-bytes = dims 32*ks + 4c.. and +16
    uint32_t bq[4][2];
    {
        const bool live = (g >> 1) < G;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(qpl + ((g >> 1) * 2 + (g & 1)) * AF_HD);
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) { bq[ks][0] = live ? src[8 * ks + c] : 0u; bq[ks][1] = live ? src[8 * ks + 4 + c] : 0u; }
    }
    const bool head_live = c < G;
    const float sfac = head_live ? qsc[c] : 0.f;

    float m_run = -FLT_MAX, l_run = 0.f;
    float O[16];
    #pragma unroll
    for (int i = 0; i < 16; ++i) O[i] = 0.f;
    bool timed_out = false;

    for (int it = 0; it < my_tiles; ++it) {
        const int t0 = kv0 + (warp + it * AF_WARPS) * AF_TILE;
        const uint8_t* Kt = wbase + (it % AF_STAGES) * AF_STAGE_BYTES;
        const uint8_t* Vt = Kt + AF_TILE * AF_PITCH;
        // scales of this lane's four keys (g, g+8, g+16, g+24)
        float ksv[4], vsv[4];
        #pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int key = t0 + g + 8 * r;
            const bool ok = key < kv1;
            ksv[r] = ok ? ksp[(size_t)key * a.n_kv + kvh] : 0.f;
            vsv[r] = ok ? vsp[(size_t)key * a.n_kv + kvh] : 0.f;
        }
        if (!timed_out && !mbar_wait_bounded(&full[warp][it % AF_STAGES], (it / AF_STAGES) & 1)) timed_out = true;

        // ── S = K Q^T: rows = keys, columns = (head, plane) ──
        float sc[4];
        #pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            int acc[4] = { 0, 0, 0, 0 };
            #pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t af[4];
                const uint8_t* r0 = Kt + (16 * mt + g) * AF_PITCH + 32 * ks + 4 * c;
                af[0] = *reinterpret_cast<const uint32_t*>(r0);
                af[1] = *reinterpret_cast<const uint32_t*>(r0 + 8 * AF_PITCH);
                af[2] = *reinterpret_cast<const uint32_t*>(r0 + 16);
                af[3] = *reinterpret_cast<const uint32_t*>(r0 + 8 * AF_PITCH + 16);
                mma_s8(acc, af, bq[ks][0], bq[ks][1]);
            }
            // thread (g, c): columns 2c, 2c+1 = (head c, hi), (head c, lo)
            sc[2 * mt]     = (float)(acc[0] * 256 + acc[1]) * (sfac * ksv[2 * mt]);
            sc[2 * mt + 1] = (float)(acc[2] * 256 + acc[3]) * (sfac * ksv[2 * mt + 1]);
        }
        #pragma unroll
        for (int r = 0; r < 4; ++r) if (t0 + g + 8 * r >= kv1) sc[r] = -INFINITY;

        // ── online softmax for head c over the tile's 32 keys ──
        float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        float vmax = fmaxf(fmaxf(vsv[0], vsv[1]), fmaxf(vsv[2], vsv[3]));
        #pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, o));
            vmax = fmaxf(vmax, __shfl_xor_sync(0xFFFFFFFFu, vmax, o));
        }
        const float m_new = fmaxf(m_run, tmax);
        const float corr = expf(m_run - m_new);
        m_run = m_new;
        const float dw = vmax / 32512.0f, idw = dw > 0.f ? 1.0f / dw : 0.f;
        float psum = 0.f;
        #pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float pv = expf(sc[r] - m_new);            // masked keys: exp(-inf) = 0
            psum += pv;
            const int W = head_live ? min(32512, __float2int_rn(pv * vsv[r] * idw)) : 0;
            const int l8 = (int)(int8_t)(W & 0xFF), h8 = (W - l8) >> 8;
            const int key = g + 8 * r;
            wsm[(2 * c) * AF_TILE + key] = (uint8_t)h8;
            wsm[(2 * c + 1) * AF_TILE + key] = (uint8_t)l8;
        }
        l_run = l_run * corr + psum;
        __syncwarp();
        // B fragments of O = V^T W: column n = g; register kb holds keys 16*kb + {2c, 2c+1, 2c+8, 2c+9}
        uint32_t bw[2];
        #pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint8_t* wr = wsm + g * AF_TILE + 16 * kb + 2 * c;
            bw[kb] = (uint32_t)*reinterpret_cast<const unsigned short*>(wr) | ((uint32_t)*reinterpret_cast<const unsigned short*>(wr + 8) << 16);
        }
        // ── O += V^T W: rows = dims, k = keys ──
        #pragma unroll
        for (int s = 0; s < 2; ++s) {
            uint32_t T[2][2][4];            // [kb][row half][dim j]
            #pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                #pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint8_t* vb = Vt + (16 * kb + 2 * c) * AF_PITCH + 4 * (g + 8 * hf + 16 * s);
                    transpose4x4(*reinterpret_cast<const uint32_t*>(vb), *reinterpret_cast<const uint32_t*>(vb + AF_PITCH),
                                 *reinterpret_cast<const uint32_t*>(vb + 8 * AF_PITCH), *reinterpret_cast<const uint32_t*>(vb + 9 * AF_PITCH),
                                 T[kb][hf]);
                }
            }
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t af[4] = { T[0][0][j], T[0][1][j], T[1][0][j], T[1][1][j] };
                int acc[4] = { 0, 0, 0, 0 };
                mma_s8(acc, af, bw[0], bw[1]);
                // rows g and g+8 of this MMA are dims 4*(g+16s)+j and 4*(g+8+16s)+j; columns 2c, 2c+1 = (head c, hi/lo)
                O[(s * 4 + j) * 2 + 0] = O[(s * 4 + j) * 2 + 0] * corr + dw * (float)(acc[0] * 256 + acc[1]);
                O[(s * 4 + j) * 2 + 1] = O[(s * 4 + j) * 2 + 1] * corr + dw * (float)(acc[2] * 256 + acc[3]);
            }
        }
        __syncwarp();
        if (it + AF_STAGES < my_tiles) { fence_proxy_async(); issue(it + AF_STAGES); }
    }
    if (timed_out && lane == 0) atomicExch(a.status, JB_ERR_TIMEOUT);

    // ── merge the four warps, write the slice's partial (or the final output when there is one slice) ──
    #pragma unroll
    for (int o = 4; o < 32; o <<= 1) l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, o);
    __syncthreads();                                        // the staging rings are free now
    float* sm_m = reinterpret_cast<float*>(smem);           // [warp][G]
    float* sm_l = sm_m + AF_WARPS * 4;
    float* sm_o = sm_l + AF_WARPS * 4;                      // [warp][G][128]
    if (head_live) {
        if (g == 0) { sm_m[warp * 4 + c] = m_run; sm_l[warp * 4 + c] = l_run; }
        #pragma unroll
        for (int s = 0; s < 2; ++s)
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                sm_o[(warp * 4 + c) * AF_HD + 4 * (g + 16 * s) + j]     = O[(s * 4 + j) * 2 + 0];
                sm_o[(warp * 4 + c) * AF_HD + 4 * (g + 8 + 16 * s) + j] = O[(s * 4 + j) * 2 + 1];
            }
    }
    __syncthreads();
    for (int h = 0; h < G; ++h) {
        const int d = tid;                                  // 128 threads = 128 dims
        float M = -FLT_MAX;
        #pragma unroll
        for (int w = 0; w < AF_WARPS; ++w) M = fmaxf(M, sm_m[w * 4 + h]);
        float L = 0.f, acc = 0.f;
        #pragma unroll
        for (int w = 0; w < AF_WARPS; ++w) {
            const float e = expf(sm_m[w * 4 + h] - M);
            L += sm_l[w * 4 + h] * e;
            acc += sm_o[(w * 4 + h) * AF_HD + d] * e;
        }
        const int head = kvh * G + h;
        if (a.n_splits == 1) {
            a.out[((size_t)z * a.n_heads + head) * AF_HD + d] = __float2half_rn(L > 0.f ? acc / L : 0.f);
        } else {
            float* pb = a.part + (((size_t)z * a.n_heads + head) * a.n_splits + split) * (AF_HD + 2);
            if (d == 0) { pb[0] = ntiles_cta > 0 ? M : -FLT_MAX; pb[1] = L; }
            pb[2 + d] = acc;
        }
    }
}


static bool af_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

// Slices: enough CTAs for two per SM, never shorter than 128 keys.
static int fast_splits(int seq, int n_kv, int batch, int sm_count) {
    const int want = (2 * sm_count + n_kv * batch - 1) / (n_kv * batch);
    int by_len = seq / 128;
    if (by_len < 1) by_len = 1;
    int ns = want < by_len ? want : by_len;
    if (ns > 64) ns = 64;
    return ns < 1 ? 1 : ns;
}

bool attention_fast_applies(const AttnCall& c) {
    const int G = c.n_kv > 0 ? c.n_heads / c.n_kv : 0;
    const bool ptrs = c.k_list ? (c.ks_list && c.vs_list && c.seq_lens) : (c.ks && c.vs && !((uintptr_t)c.k & 15) && !((uintptr_t)c.v & 15));
    return c.kv_int8 && c.hd == AF_HD && c.chd == AF_HD && c.window == 0 && c.causal_start < 0 && (G == 1 || G == 2 || G == 4) &&
           c.n_heads == G * c.n_kv && ptrs;
}

int launch_attention_fast(const AttnCall& c, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    const int batch = c.batch > 0 ? c.batch : 1;
    const int seq_for_policy = c.k_list ? c.max_seq : (c.d_pos ? c.max_seq : c.seq_len);
    if (!c.d_pos && !c.k_list && c.seq_len <= 0) {
        JB_CUDA(cudaMemsetAsync(c.out, 0, (size_t)c.n_heads * c.hd * sizeof(__half), st));
        return JB_OK;
    }
    int n_splits = c.n_splits > 0 ? c.n_splits : fast_splits(seq_for_policy > 0 ? seq_for_policy : 1, c.n_kv, batch, cx->sm_count);
    AfArgs a = {};
    a.out = c.out; a.q = c.q; a.k = (const int8_t*)c.k; a.v = (const int8_t*)c.v; a.ks = c.ks; a.vs = c.vs;
    a.k_list = c.k_list; a.v_list = c.v_list; a.ks_list = c.ks_list; a.vs_list = c.vs_list; a.seq_lens = c.seq_lens;
    a.n_heads = c.n_heads; a.n_kv = c.n_kv; a.seq_len = c.seq_len; a.d_pos = c.d_pos; a.scale = c.scale; a.status = cx->d_status;
    if (n_splits > 1) {
        a.part = splitk_buffer((size_t)batch * c.n_heads * n_splits * (c.hd + 2), !af_capturing(st));
        if (!a.part) n_splits = 1;
    }
    a.n_splits = n_splits;
    const int G = c.n_heads / c.n_kv;
    auto kern = G == 4 ? attn_fast_kernel<4> : (G == 2 ? attn_fast_kernel<2> : attn_fast_kernel<1>);
    static bool attr_done[3] = { false, false, false };
    const int gi = G == 4 ? 2 : (G == 2 ? 1 : 0);
    if (!attr_done[gi]) { JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AF_SMEM)); attr_done[gi] = true; }
    JB_CUDA(launch_k(kern, dim3(c.n_kv, n_splits, batch), dim3(AF_WARPS * 32), (size_t)AF_SMEM, st, pdl_enabled(), a));
    count_launch();
    if (n_splits > 1) {
        const int rc = launch_attn_reduce(c.out, a.part, c.n_heads, c.hd, n_splits, batch, st);
        if (rc) return rc;
    }
    return JB_OK;
}

}  // namespace jb
