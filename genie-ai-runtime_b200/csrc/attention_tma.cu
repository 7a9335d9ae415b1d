// attention_tma.cu — split-K decode attention over an INT8 KV cache, head_dim 128, for sm_100a; K/V tiles fetched by
// 2-D TMA tensor copies.
//
// Replaces the reference's flash_decode_splitk_partial_kernel + flash_decode_reduce_kernel
// (src/kernels/attention.cu:837-969) for the INT8 cache layout [pos][kv_head][128] with one fp32 scale per
// (pos, kv_head).  Same mathematics — s_j = scale * Σ_d q_d (k8_jd ks_j), online softmax, o_d = Σ_j p_j (v8_jd vs_j):
//   * one CTA per (kv head, KV slice, sequence): the 2..4 query heads of a GQA group share every K/V byte read;
//   * a tile of 32 keys is TWO TMA copies (cp.async.bulk.tensor.2d: box 128 bytes x 32 rows out of the
//     [pos][n_kv*128] byte matrix of this GPU's own cache, 128-byte swizzle, completion by byte count on an
//     mbarrier) instead of 64 row copies; every warp owns a private ring of tiles, no CTA-wide barrier in the loop;
//   * the per-key scales of the NEXT tile are fetched while the current one is being multiplied;
//   * QK^T and PV run on the int8 tensor-core path (mma.sync m16n8k32) with q and the softmax weights as 16-bit fixed
//     point in two int8 planes: integer dots exact, result within ~2^-15 of the reference's fp32 arithmetic; the
//     swizzled tile layout makes every fragment read bank-conflict free;
//   * slices are merged by the LAST CTA of each (sequence, kv head) to finish — a ticket counter next to the
//     partials — so a call is one launch; the counter returns to zero for the next call.
// Tensor maps describe this GPU's own memory only and no copy uses cluster multicast.
#include "attention.cuh"
#include <cfloat>
#include <cstdlib>
#include <cstring>
#include <cuda.h>

namespace jb {

constexpr int AM_WARPS  = 4;
constexpr int AM_TILE   = 32;                        // keys per warp tile
constexpr int AM_STAGES = 2;                        // tiles in flight per warp; three CTAs (twelve warps) share an SM
constexpr int AM_HD     = 128;
constexpr int AM_TILE_BYTES  = AM_TILE * AM_HD;       // one K (or V) tile: 4 KB, rows of 128 bytes, 128-byte swizzle
constexpr int AM_STAGE_BYTES = 2 * AM_TILE_BYTES;
constexpr int AM_RING_BYTES  = AM_WARPS * AM_STAGES * AM_STAGE_BYTES;
constexpr int AM_SCALE_BYTES = AM_WARPS * AM_STAGES * 2 * AM_TILE * 4;           // per warp and stage: K and V scales of the tile's 32 keys
constexpr int AM_SMEM = AM_RING_BYTES + AM_WARPS * 256 + 1024 + 64 + AM_SCALE_BYTES + 1024;   // + PV weight bytes, query planes, scales, alignment slack

constexpr int AM_PREC = AM_HD + 4;                    // floats of a slice's partial record: m, l, two pad words, acc[128] (16-byte aligned)
constexpr int AM_BATCH_SEQS = 14;                     // sequences per launch of a ragged batch: 28 tensor maps fit the 4 KB of kernel parameters

// Tensor maps travel as kernel parameters (constant bank).  Maps read from global memory work but were measured at several
// microseconds per tensor copy, so a ragged batch is launched in groups of AM_BATCH_SEQS sequences instead.
template <int NSEQ> struct AmMaps { CUtensorMap m[2 * NSEQ]; };

struct AmArgs {
    __half* out; const __half* q;
    const float* ks; const float* vs;
    int ragged, z0;                          // ragged batch: sequence blockIdx.z of this launch is sequence z0 + blockIdx.z of the batch
    const float* const* ks_list; const float* const* vs_list; const int* seq_lens;
    int n_heads, n_kv, seq_len; const int* d_pos;
    float scale; int n_splits;
    float* part; unsigned int* tickets; int* status;
    int nocompute;                           // diagnostic: fetch the tiles, skip the arithmetic
};

__device__ __forceinline__ void am_mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// rows r0..r3 hold bytes (dim0..dim3) of four keys; t[j] = (key0..key3) bytes of dim j
__device__ __forceinline__ void am_transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&t)[4]) {
    const uint32_t u0 = __byte_perm(r0, r1, 0x5140), u1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t u2 = __byte_perm(r0, r1, 0x7362), u3 = __byte_perm(r2, r3, 0x7362);
    t[0] = __byte_perm(u0, u1, 0x5410); t[1] = __byte_perm(u0, u1, 0x7632);
    t[2] = __byte_perm(u2, u3, 0x5410); t[3] = __byte_perm(u2, u3, 0x7632);
}
__device__ __forceinline__ void am_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// 2^x by the hardware approximation (relative error ~2^-22, far inside the fp16 output); 2^-inf = 0
__device__ __forceinline__ float am_exp2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t am_lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }

// byte (row, b) of a tile with the 128-byte swizzle: the 16-byte chunk index is xored with the row's low three bits
__device__ __forceinline__ uint32_t am_swz(uint32_t tile, int row, int b) {
    return tile + (uint32_t)row * 128u + (uint32_t)((((b >> 4) ^ (row & 7)) << 4) | (b & 15));
}

template <int G, int NSEQ>   // G: query heads per kv head (1, 2 or 4); NSEQ: sequences whose tensor maps this launch carries
__global__ void __launch_bounds__(AM_WARPS * 32, 3) attn_tma_kernel(const __grid_constant__ AmMaps<NSEQ> mp, const AmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full[AM_WARPS][AM_STAGES];
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, c = lane & 3;
    const int kvh = blockIdx.x, split = blockIdx.y, zl = blockIdx.z, z = a.z0 + zl;

    const uint32_t ring0 = (smem_u32(smem_raw) + 1023u) & ~1023u;               // swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (ring0 - smem_u32(smem_raw));
    const uint32_t wring = ring0 + (uint32_t)warp * AM_STAGES * AM_STAGE_BYTES;
    uint8_t* wsm = smem + AM_RING_BYTES + warp * 256;                            // [8 columns][32 keys] int8
    int8_t*  qpl = reinterpret_cast<int8_t*>(smem + AM_RING_BYTES + AM_WARPS * 256);        // [G][2 planes][128]
    float*   qsc = reinterpret_cast<float*>(smem + AM_RING_BYTES + AM_WARPS * 256 + 1024);  // dq per head
    float*   ssm = reinterpret_cast<float*>(smem + AM_RING_BYTES + AM_WARPS * 256 + 1024 + 64) + warp * AM_STAGES * 2 * AM_TILE;   // [stage][K | V][32]

    const CUtensorMap* km = &mp.m[2 * zl];
    const CUtensorMap* vm = &mp.m[2 * zl + 1];
    if (lane == 0) { for (int s = 0; s < AM_STAGES; ++s) mbar_init(&full[warp][s], 1 + 32); }      // lane 0's byte count + every lane's scale copies
    if (tid == 0) {
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(km) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(vm) : "memory");
    }
    __syncthreads();
    pdl_launch();
    pdl_wait();

    const float* ksp = a.ks; const float* vsp = a.vs;
    int seq = a.d_pos ? (*a.d_pos + 1) : a.seq_len;
    if (a.ragged) { ksp = a.ks_list[z]; vsp = a.vs_list[z]; seq = a.seq_lens[z]; }
    int per = (seq + a.n_splits - 1) / a.n_splits;
    per = (per + AM_TILE - 1) / AM_TILE * AM_TILE;                               // slices start on tile boundaries
    const int kv0 = split * per, kv1 = min(kv0 + per, seq);
    const int ntiles_cta = kv1 > kv0 ? (kv1 - kv0 + AM_TILE - 1) / AM_TILE : 0;
    const int my_tiles = ntiles_cta > warp ? (ntiles_cta - warp + AM_WARPS - 1) / AM_WARPS : 0;

    // Tile `it` of this warp -> stage it % AM_STAGES; called by the whole warp.  Lane 0 issues the two tensor copies; lane l
    // copies the K and V scale of key t0 + l (the 32 floats of a kv head sit 32 bytes apart) with 4-byte cp.async into the
    // stage's scale slots and makes them count on the same mbarrier (cp.async.mbarrier.arrive.noinc): the scales travel with
    // their tile, as far ahead as the tile itself, and no warp ever waits for a plain load behind the SM's queue of tile
    // requests (with per-lane loads one tile ahead, `long_scoreboard` was the top stall: 3.1 warps per issued instruction).
    auto issue = [&](int it) {
        const int t0 = kv0 + (warp + it * AM_WARPS) * AM_TILE;
        const uint32_t st = wring + (uint32_t)(it % AM_STAGES) * AM_STAGE_BYTES;
        uint64_t* bar = &full[warp][it % AM_STAGES];
        float* sd = ssm + (it % AM_STAGES) * 2 * AM_TILE + lane;
        const int key = t0 + lane;
        if (key < kv1) {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(sd)), "l"(ksp + (size_t)key * a.n_kv + kvh) : "memory");
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(sd + AM_TILE)), "l"(vsp + (size_t)key * a.n_kv + kvh) : "memory");
        } else {
            sd[0] = 0.f; sd[AM_TILE] = 0.f;
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
        if (lane == 0) {
            mbar_expect_tx(bar, (uint32_t)AM_STAGE_BYTES);                       // rows past the tensor's end are zero-filled and counted
            am_tma_2d(st, km, kvh * AM_HD, t0, bar);
            am_tma_2d(st + AM_TILE_BYTES, vm, kvh * AM_HD, t0, bar);
        }
    };
    for (int it = 0; it < AM_STAGES && it < my_tiles; ++it) issue(it);

    // ── query planes: per head 16-bit fixed point, split into a high and a (signed) low byte ──
    if (warp < G) {
        const int head = kvh * G + warp;
        const __half* qh = a.q + ((size_t)z * a.n_heads + head) * AM_HD + 4 * lane;
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
        reinterpret_cast<uint32_t*>(qpl + (warp * 2 + 0) * AM_HD)[lane] = hi;
        reinterpret_cast<uint32_t*>(qpl + (warp * 2 + 1) * AM_HD)[lane] = lo;
        if (lane == 0) qsc[warp] = dq * a.scale * 1.4426950408889634f;     // scores in units of log2: the softmax below is 2^x
    }
    __syncthreads();
    // B fragments of QK^T: column n = g is (head g>>1, plane g&1); k-bytes = dims 32*ks + 4c.. and +16
    uint32_t bq[4][2];
    {
        const bool live = (g >> 1) < G;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(qpl + ((g >> 1) * 2 + (g & 1)) * AM_HD);
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
        const int t0 = kv0 + (warp + it * AM_WARPS) * AM_TILE;
        const uint32_t Kt = wring + (uint32_t)(it % AM_STAGES) * AM_STAGE_BYTES, Vt = Kt + AM_TILE_BYTES;
        if (!timed_out && !mbar_wait_bounded(&full[warp][it % AM_STAGES], (it / AM_STAGES) & 1)) timed_out = true;
        if (a.nocompute) {                      // diagnostic: how fast do the tiles alone arrive?
            __syncwarp();
            if (it + AM_STAGES < my_tiles) { if (lane == 0) fence_proxy_async(); issue(it + AM_STAGES); }
            continue;
        }
        float ksv[4], vsv[4];
        {
            const float* sd = ssm + (it % AM_STAGES) * 2 * AM_TILE;
            #pragma unroll
            for (int r = 0; r < 4; ++r) { ksv[r] = sd[g + 8 * r]; vsv[r] = sd[AM_TILE + g + 8 * r]; }
        }

        // ── S = K Q^T: rows = keys, columns = (head, plane) ──
        float sc[4];
        #pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            int acc[4] = { 0, 0, 0, 0 };
            const uint32_t r0 = Kt + (uint32_t)(16 * mt + g) * 128u + 4u * c;    // rows 16mt+g and +8 share the swizzle term g
            #pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t o0 = (uint32_t)(((2 * ks) ^ g) << 4), o1 = (uint32_t)(((2 * ks + 1) ^ g) << 4);
                uint32_t af[4];
                af[0] = am_lds32(r0 + o0);
                af[1] = am_lds32(r0 + 8 * 128 + o0);
                af[2] = am_lds32(r0 + o1);
                af[3] = am_lds32(r0 + 8 * 128 + o1);
                am_mma_s8(acc, af, bq[ks][0], bq[ks][1]);
            }
            // thread (g, c): columns 2c, 2c+1 = (head c, hi), (head c, lo)
            sc[2 * mt]     = (float)(acc[0] * 256 + acc[1]) * (sfac * ksv[2 * mt]);
            sc[2 * mt + 1] = (float)(acc[2] * 256 + acc[3]) * (sfac * ksv[2 * mt + 1]);
        }
        #pragma unroll
        for (int r = 0; r < 4; ++r) if (t0 + g + 8 * r >= kv1) sc[r] = -INFINITY;

        // ── online softmax for head c over the tile's 32 keys ──
        float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        #pragma unroll
        for (int o = 4; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, o));
        // The softmax weights of a tile are formed relative to the TILE's maximum, and the products p_j * vs_j are held as
        // 16-bit fixed point relative to the LARGEST product of the tile, so they keep their full precision however far the
        // tile lies below the running maximum and whatever the spread of the V scales; the tile as a whole is then scaled by
        // tfac = 2^{tile max - running max}.  A tile always holds at least one unmasked key, so tmax is finite.
        const float m_new = fmaxf(m_run, tmax);
        const float corr = am_exp2(m_run - m_new), tfac = am_exp2(tmax - m_new);
        m_run = m_new;
        float psum = 0.f, pw[4], wmax = 0.f;
        #pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float pv = am_exp2(sc[r] - tmax);          // masked keys: 2^-inf = 0
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
            wsm[(2 * c) * AM_TILE + key] = (uint8_t)h8;
            wsm[(2 * c + 1) * AM_TILE + key] = (uint8_t)l8;
        }
        l_run = l_run * corr + psum * tfac;
        const float dwt = dw * tfac;
        __syncwarp();
        // B fragments of O = V^T W: column n = g; register kb holds keys 16*kb + {2c, 2c+1, 2c+8, 2c+9}
        uint32_t bw[2];
        #pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint8_t* wr = wsm + g * AM_TILE + 16 * kb + 2 * c;
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
                    const int row = 16 * kb + 2 * c, b = 4 * (g + 8 * hf + 16 * s);
                    am_transpose4x4(am_lds32(am_swz(Vt, row, b)), am_lds32(am_swz(Vt, row + 1, b)),
                                    am_lds32(am_swz(Vt, row + 8, b)), am_lds32(am_swz(Vt, row + 9, b)), T[kb][hf]);
                }
            }
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t af[4] = { T[0][0][j], T[0][1][j], T[1][0][j], T[1][1][j] };
                int acc[4] = { 0, 0, 0, 0 };
                am_mma_s8(acc, af, bw[0], bw[1]);
                // rows g and g+8 of this MMA are dims 4*(g+16s)+j and 4*(g+8+16s)+j; columns 2c, 2c+1 = (head c, hi/lo)
                O[(s * 4 + j) * 2 + 0] = O[(s * 4 + j) * 2 + 0] * corr + dwt * (float)(acc[0] * 256 + acc[1]);
                O[(s * 4 + j) * 2 + 1] = O[(s * 4 + j) * 2 + 1] * corr + dwt * (float)(acc[2] * 256 + acc[3]);
            }
        }
        __syncwarp();
        if (it + AM_STAGES < my_tiles) { if (lane == 0) fence_proxy_async(); issue(it + AM_STAGES); }
    }
    if (timed_out && lane == 0) atomicExch(a.status, JB_ERR_TIMEOUT);

    // ── merge the four warps, write the slice's partial (or the final output when there is one slice) ──
    #pragma unroll
    for (int o = 4; o < 32; o <<= 1) l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, o);
    __syncthreads();                                        // the staging rings are free now
    float* sm_m = reinterpret_cast<float*>(smem);           // [warp][4]
    float* sm_l = sm_m + AM_WARPS * 4;
    float* sm_o = sm_l + AM_WARPS * 4;                      // [warp][4][128]
    if (head_live) {
        if (g == 0) { sm_m[warp * 4 + c] = m_run; sm_l[warp * 4 + c] = l_run; }
        #pragma unroll
        for (int s = 0; s < 2; ++s)
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                sm_o[(warp * 4 + c) * AM_HD + 4 * (g + 16 * s) + j]     = O[(s * 4 + j) * 2 + 0];
                sm_o[(warp * 4 + c) * AM_HD + 4 * (g + 8 + 16 * s) + j] = O[(s * 4 + j) * 2 + 1];
            }
    }
    __syncthreads();
    const int d = tid;                                      // 128 threads = 128 dims
    for (int h = 0; h < G; ++h) {
        float M = -FLT_MAX;
        #pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) M = fmaxf(M, sm_m[w * 4 + h]);
        float L = 0.f, acc = 0.f;
        #pragma unroll
        for (int w = 0; w < AM_WARPS; ++w) {
            const float e = am_exp2(sm_m[w * 4 + h] - M);
            L += sm_l[w * 4 + h] * e;
            acc += sm_o[(w * 4 + h) * AM_HD + d] * e;
        }
        const int head = kvh * G + h;
        if (a.n_splits == 1) {
            a.out[((size_t)z * a.n_heads + head) * AM_HD + d] = __float2half_rn(L > 0.f ? acc / L : 0.f);
        } else {
            float* pb = a.part + (((size_t)z * a.n_heads + head) * a.n_splits + split) * AM_PREC;
            if (d == 0) { pb[0] = ntiles_cta > 0 ? M : -FLT_MAX; pb[1] = L; }
            pb[4 + d] = acc;
        }
    }
    if (a.n_splits == 1) return;

    // ── the last slice of this (sequence, kv head) to finish merges all of them: out = Σ acc_s e^{m_s-M} / Σ l_s e^{m_s-M}
    //    (reference :944-969) ──
    __threadfence();                                        // this CTA's partials are visible device-wide before its ticket
    __syncthreads();
    if (tid == 0) {
        unsigned int* tk = a.tickets + (size_t)z * a.n_kv + kvh;
        const unsigned int t = atomicAdd(tk, 1u);
        s_last = (t == (unsigned int)a.n_splits - 1u);
        if (s_last) *tk = 0u;                               // ready for the next call (stream order separates calls)
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // One warp per head, no CTA barrier: lane l reads (m, l) of slices l and l + 32 (n_splits <= 64), the warp reduces the
    // maximum and the sum, then every lane adds its four dimensions over the slices in order with independent 16-byte loads
    // (a serial pass per head with a barrier and an L2 round trip per batch of slices used to cost 0.3 us per slice: 20 of the
    // 29 us of a 32768-key call).
    if (warp < G) {
        const int head = kvh * G + warp;
        const float* pb = a.part + ((size_t)z * a.n_heads + head) * a.n_splits * AM_PREC;
        const bool in0 = lane < a.n_splits, in1 = lane + 32 < a.n_splits;
        const float m0 = in0 ? __ldcg(pb + (size_t)lane * AM_PREC) : -FLT_MAX, m1 = in1 ? __ldcg(pb + (size_t)(lane + 32) * AM_PREC) : -FLT_MAX;
        const float l0 = in0 ? __ldcg(pb + (size_t)lane * AM_PREC + 1) : 0.f, l1 = in1 ? __ldcg(pb + (size_t)(lane + 32) * AM_PREC + 1) : 0.f;
        const float M = warp_max(fmaxf(m0, m1));
        const float e0 = in0 ? am_exp2(m0 - M) : 0.f, e1 = in1 ? am_exp2(m1 - M) : 0.f;
        const float L = warp_sum(l0 * e0 + l1 * e1);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // sixteen loads in flight per lane: four L2 round trips for the 64 slices a call can have
        for (int s0 = 0; s0 < a.n_splits; s0 += 16) {
            float4 v[16];
            #pragma unroll
            for (int i = 0; i < 16; ++i)
                v[i] = s0 + i < a.n_splits ? __ldcg(reinterpret_cast<const float4*>(pb + (size_t)(s0 + i) * AM_PREC + 4) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            #pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int s = s0 + i;
                const float e = __shfl_sync(0xFFFFFFFFu, s < 32 ? e0 : e1, s & 31);
                acc.x += v[i].x * e; acc.y += v[i].y * e; acc.z += v[i].z * e; acc.w += v[i].w * e;
            }
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        const __half2 o0 = __floats2half2_rn(acc.x * inv, acc.y * inv), o1 = __floats2half2_rn(acc.z * inv, acc.w * inv);
        uint2 st2; st2.x = *reinterpret_cast<const uint32_t*>(&o0); st2.y = *reinterpret_cast<const uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(a.out + ((size_t)z * a.n_heads + head) * AM_HD + 4 * lane) = st2;
    }
}

// ── host side ──────────────────────────────────────────────────────────────
typedef CUresult (*AmEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AmEncodeFn am_encode_fn() {
    static AmEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = (AmEncodeFn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

// Tensor map over one K (or V) cache of `rows` positions: a [rows][n_kv*128] byte matrix, box = 128 bytes x 32 rows.
bool attn_tma_encode(void* map_out, const void* base, int rows, int n_kv) {
    AmEncodeFn fn = am_encode_fn();
    if (!fn || rows <= 0 || ((uintptr_t)base & 15)) return false;
    const cuuint64_t gdim[2] = { (cuuint64_t)n_kv * AM_HD, (cuuint64_t)rows };
    const cuuint64_t gstr[1] = { (cuuint64_t)n_kv * AM_HD };
    const cuuint32_t box[2] = { (cuuint32_t)AM_HD, (cuuint32_t)AM_TILE };
    const cuuint32_t estr[2] = { 1, 1 };
    alignas(64) CUtensorMap m;               // the driver wants a 64-byte aligned object; map_out may be any 128-byte slot
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
    memcpy(map_out, &m, sizeof m);
    return true;
}

static bool am_capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) { cudaGetLastError(); return false; }
    return cs != cudaStreamCaptureStatusNone;
}

// Slices: as many CTAs as fit at once (three per SM, rounded down: a second wave of a few stragglers would double the call);
// one slice below 640 keys (a sliced call pays the partials, a ticket and the merge: ~1.5 us), slices of at least 128 keys up to
// 2048 keys and of at least 512 beyond, at most 64 (the merge reads two slices per lane); a batch: see below.  Measured per call, 300 / 500 / 700 /
// 1024 / 4096 / 8192 / 32768 keys: 5.1 / 6.3 / 6.9 / 6.4 / 9.7 / 12.1 / 20.4 us.
static int am_splits(int seq, int n_kv, int batch, int sm_count) {
    if (seq < 640) return 1;
    // a ragged batch: slices of 1024 keys of the LONGEST sequence the caches can hold (shorter sequences get the same number of
    // shorter slices): without slices the longest sequence's CTA runs 256 tiles on four warps while most SMs have drained —
    // 64 sequences U{256..8192}: 343 us unsliced, 163 / 141 / 164 us with slices of 2048 / 1024 / 512 keys
    if (batch > 1) { const int n = seq / 1024; return n < 1 ? 1 : (n > 16 ? 16 : n); }
    const int want = 3 * sm_count / (n_kv * batch);
    const int by_len = seq < 2048 ? seq / 128 : seq / 512;
    int ns = want < by_len ? want : by_len;
    if (ns > 64) ns = 64;
    return ns < 1 ? 1 : ns;
}

// The TMA path needs to know how many rows a cache holds (the tensor map's extent): a length by value, a device-side
// position together with max_seq, or a plan of prebuilt maps (a host array) for a ragged batch.
bool attention_tma_applies(const AttnCall& c) {
    const int G = c.n_kv > 0 ? c.n_heads / c.n_kv : 0;
    if (!(c.kv_int8 && c.hd == AM_HD && c.chd == AM_HD && c.window == 0 && c.causal_start < 0 && (G == 1 || G == 2 || G == 4) && c.n_heads == G * c.n_kv))
        return false;
    if (c.tma_maps) return c.ks_list && c.vs_list && c.seq_lens;
    if (c.k_list) return false;
    if (!c.k || !c.v || !c.ks || !c.vs || ((uintptr_t)c.k & 15) || ((uintptr_t)c.v & 15)) return false;
    return c.d_pos ? c.max_seq > 0 : c.seq_len > 0;
}

template <int NSEQ>
static int am_launch(const AmMaps<NSEQ>& mp, const AmArgs& a, int G, dim3 grid, DeviceCtx* cx, cudaStream_t st) {
    auto kern = G == 4 ? attn_tma_kernel<4, NSEQ> : (G == 2 ? attn_tma_kernel<2, NSEQ> : attn_tma_kernel<1, NSEQ>);
    const int gi = (G == 4 ? 2 : (G == 2 ? 1 : 0)) + (NSEQ == 1 ? 0 : 3);
    if (!cx->attn_tma_attr[gi]) { JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AM_SMEM)); cx->attn_tma_attr[gi] = true; }
    JB_CUDA(launch_k(kern, grid, dim3(AM_WARPS * 32), (size_t)AM_SMEM, st, pdl_enabled(), mp, a));
    count_launch();
    return JB_OK;
}

int launch_attention_tma(const AttnCall& c, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    const int batch = c.batch > 0 ? c.batch : 1;
    const int rows = c.tma_maps ? c.max_seq : (c.d_pos ? c.max_seq : c.seq_len);
    int n_splits = c.n_splits > 0 ? c.n_splits : am_splits(rows > 0 ? rows : 1, c.n_kv, batch, cx->sm_count);
    if (n_splits > 64) n_splits = 64;                       // the merge holds one slice per thread of the last CTA
    AmArgs a = {};
    a.out = c.out; a.q = c.q; a.ks = c.ks; a.vs = c.vs;
    a.ragged = c.tma_maps ? 1 : 0; a.ks_list = c.ks_list; a.vs_list = c.vs_list; a.seq_lens = c.seq_lens;
    a.n_heads = c.n_heads; a.n_kv = c.n_kv; a.seq_len = c.seq_len; a.d_pos = c.d_pos; a.scale = c.scale; a.status = cx->d_status;
    static const bool nocompute = getenv("JLLM_B200_ATTN_NOCOMPUTE") != nullptr;
    a.nocompute = nocompute ? 1 : 0;
    if (n_splits > 1) {
        // partials in the per-device split buffer; one ticket word per (sequence, kv head) in a per-device array that is zeroed
        // once and that every call leaves at zero
        a.part = (size_t)batch * c.n_kv <= (size_t)ATTN_TICKET_WORDS ? splitk_buffer((size_t)batch * c.n_heads * n_splits * AM_PREC, !am_capturing(st)) : nullptr;
        if (!a.part) n_splits = 1;       // no scratch (or capture in progress): one slice per kv head, still on the GPU
        else a.tickets = cx->attn_tickets;
    }
    a.n_splits = n_splits;
    const int G = c.n_heads / c.n_kv;
    if (!c.tma_maps) {
        alignas(64) AmMaps<1> mp;
        if (!attn_tma_encode(&mp.m[0], c.k, rows, c.n_kv) || !attn_tma_encode(&mp.m[1], c.v, rows, c.n_kv))
            return set_error(JB_ERR_CUDA, "attention: tensor map for the KV cache refused");
        return am_launch<1>(mp, a, G, dim3(c.n_kv, n_splits, 1), cx, st);
    }
    // ragged batch: c.tma_maps is a HOST array of [batch][K, V] maps; groups of AM_BATCH_SEQS sequences per launch
    const CUtensorMap* hm = reinterpret_cast<const CUtensorMap*>(c.tma_maps);
    for (int z0 = 0; z0 < batch; z0 += AM_BATCH_SEQS) {
        const int n = batch - z0 < AM_BATCH_SEQS ? batch - z0 : AM_BATCH_SEQS;
        alignas(64) AmMaps<AM_BATCH_SEQS> mp;
        memcpy(mp.m, hm + 2 * z0, (size_t)n * 2 * sizeof(CUtensorMap));
        for (int i = 2 * n; i < 2 * AM_BATCH_SEQS; ++i) mp.m[i] = mp.m[0];
        a.z0 = z0;
        const int rc = am_launch<AM_BATCH_SEQS>(mp, a, G, dim3(c.n_kv, n_splits, n), cx, st);
        if (rc) return rc;
    }
    return JB_OK;
}

}  // namespace jb
