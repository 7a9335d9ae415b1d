// gemv.cu — streaming K-quant GEMV for B200 (sm_100a).
//
// Replaces the reference's decode GEMV family (src/kernels/gemv_q4.cu:445-683 kernels,
// :1245-1616 dispatch).  The GGUF super-block layout is read unchanged from HBM.
//
// Shape of the kernel
//   * grid = 2 CTAs per SM; every CTA owns one contiguous byte range of the (up to three)
//     weight matrices, split evenly by bytes, so all SMs stream the same amount.
//   * weights travel HBM -> shared memory with 1-D TMA bulk copies (cp.async.bulk +
//     mbarrier complete_tx) through a ring of slots, several copies in flight per CTA;
//     Q6_K rows (210-byte blocks, 2-byte aligned) are copied as the enclosing 16-byte
//     aligned span and re-aligned with funnel shifts when read from shared memory.
//   * the activation vector is quantised by every CTA itself into shared memory (q8_1
//     codes, or 16-bit fixed point for the entry points whose reference path keeps fp16
//     activations), optionally after a fused RMSNorm, laid out so that the 16-byte runs
//     the lanes read are bank-conflict free.
//   * each lane takes one 16-byte run of quants per step, dots it with dp4a, and a warp
//     reduces the rows it owns with shuffles; outputs are deterministic.
//   * launched with programmatic dependent launch: weight copies are issued before
//     griddepcontrol.wait, so they overlap the tail of the kernel that produces x.
#include "gemv.cuh"

namespace jb {

constexpr int GV_WARPS   = 4;
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_MAXSLOT = 8;
constexpr int GV_SMEM_BUDGET = 110 * 1024;     // per CTA, two CTAs per SM

struct GvSegDev {
    const uint8_t* W; void* y; int M; int type;
    int rb;          // row bytes
    int U;           // 16-byte work items per row (Q4_K: 8/block, Q6_K: 4/block)
    int R;           // rows per warp
    int trc;         // rows per chunk
};
struct GvParams {
    GvSegDev seg[3]; int nseg;
    const __half* x; int K;
    int out_mode; const __half* residual;
    int do_norm; const void* norm_w; int norm_w_fp32; float eps;
    int32_t* dbg_dots; int* status;
    int slot_bytes, nslots, needA, needB, paired_rows;
    uint32_t off_xA, off_xB, off_xd, off_xs, off_xsum, off_gate, off_slots;
    long long total_bytes;
};

// ── activation staging ───────────────────────────────────────────────────
// Layout A (read by Q4_K items), per 256 elements: [8 runs of 16 low-nibble partners]
// [8 runs of 16 high-nibble partners]: element e = 32j + 16h + i (sub-block j, half h)
// lands at (j&1)*128 + (2*(j>>1)+h)*16 + i.  Layout B (Q6_K items): plane k (= 32-wide
// quarter of a 128-half) at k*K/4, run (blk*4 + 2n + c)*16.  In 16-bit mode a second
// plane with the low bytes follows at +K.
template <int XM>
__device__ __forceinline__ void stage_x(const GvParams& p, uint8_t* smem, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K;
    float rrms = 1.0f;
    if (p.do_norm) {   // reference: fused_rmsnorm_residual, src/kernels/fused_norm.cu:33-101
        float ss = 0.f;
        for (int g4 = tid; g4 < K / 4; g4 += GV_THREADS) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p.x + 4 * g4);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        #pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) tot += red[w];
        rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
        __syncthreads();
    }
    uint8_t* xA = smem + p.off_xA; uint8_t* xB = smem + p.off_xB;
    float* xd = reinterpret_cast<float*>(smem + p.off_xd);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    int*   xsum = reinterpret_cast<int*>(smem + p.off_xsum);
    for (int g4 = tid; g4 < K / 4; g4 += GV_THREADS) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p.x + 4 * g4);
        float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        float v[4] = { a.x, a.y, b.x, b.y };
        if (p.do_norm) {
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float w = p.norm_w_fp32 ? reinterpret_cast<const float*>(p.norm_w)[4 * g4 + i]
                                              : __half2float(reinterpret_cast<const __half*>(p.norm_w)[4 * g4 + i]);
                v[i] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i], rrms), w)));
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        #pragma unroll
        for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        int q[4]; int qsum = 0; float d; float fsum = 0.f;
        if (XM == 0) {     // q8_1: src/kernels/gemv_q4.cu:445-466
            d = __fdiv_rn(amax, 127.0f);
            const float id = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
            #pragma unroll
            for (int i = 0; i < 4; ++i) { q[i] = max(-127, min(127, __float2int_rn(__fmul_rn(v[i], id)))); qsum += q[i]; }
        } else {           // 16-bit fixed point
            d = __fdiv_rn(amax, 32767.0f);
            const float id = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
            #pragma unroll
            for (int i = 0; i < 4; ++i) { q[i] = max(-32767, min(32767, __float2int_rn(__fmul_rn(v[i], id)))); qsum += q[i]; }
            fsum = (v[0] + v[1]) + (v[2] + v[3]);
        }
        // 16-element code sums (Q6_K subtracts 32*sum instead of re-centring every quant)
        int s16 = qsum;
        s16 += __shfl_xor_sync(0xFFFFFFFFu, s16, 1);
        s16 += __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
        int s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 4);
        if (XM == 1) {
            #pragma unroll
            for (int o = 1; o < 8; o <<= 1) fsum += __shfl_xor_sync(0xFFFFFFFFu, fsum, o);
        }
        const int e0 = 4 * g4, blk = e0 >> 8, r = e0 & 255;
        uint32_t w_hi, w_lo = 0;
        if (XM == 0) {
            w_hi = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
        } else {
            w_hi = (uint32_t)((q[0] >> 8) & 0xFF) | ((uint32_t)((q[1] >> 8) & 0xFF) << 8) | ((uint32_t)((q[2] >> 8) & 0xFF) << 16) | ((uint32_t)((q[3] >> 8) & 0xFF) << 24);
            w_lo = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
        }
        if (p.needA) {
            const int j = r >> 5, wi = r & 31, h = wi >> 4, i = wi & 15;
            const int off = blk * 256 + (j & 1) * 128 + (2 * (j >> 1) + h) * 16 + i;
            *reinterpret_cast<uint32_t*>(xA + off) = w_hi;
            if (XM == 1) *reinterpret_cast<uint32_t*>(xA + K + off) = w_lo;
        }
        if (p.needB) {
            const int n = r >> 7, k = (r & 127) >> 5, c = (r & 31) >> 4, i = r & 15;
            const int off = k * (K >> 2) + (blk * 4 + 2 * n + c) * 16 + i;
            *reinterpret_cast<uint32_t*>(xB + off) = w_hi;
            if (XM == 1) *reinterpret_cast<uint32_t*>(xB + K + off) = w_lo;
            if ((lane & 3) == 0) xsum[e0 >> 4] = s16;
        }
        if ((lane & 7) == 0) {
            if (XM == 0) {
                xd[e0 >> 5] = __half2float(__float2half_rn(d));
                xs[e0 >> 5] = __half2float(__float2half_rn(__fmul_rn(d, (float)s32)));
            } else {
                xd[e0 >> 5] = d;
                xs[e0 >> 5] = fsum;
            }
        }
    }
}

// ── Q4_K: one 16-byte run of quants per lane ─────────────────────────────
// Run u (0..7) of a block holds the low nibbles of sub-block 2*(u>>1) (elements
// 16*(u&1)..+15) and the high nibbles of sub-block 2*(u>>1)+1.  Lanes u and u^1
// exchange one partial so that each ends with the complete 32-element integer dot of
// sub-block u — the same accumulator the reference builds with eight dp4a
// (src/kernels/gemv_q4.cu:487-494) — and applies  dall*sc*(d8*dot) - dmin*m*s8  (:499).
template <int XM>
__device__ __forceinline__ float q4k_item(const uint8_t* sb, int u, int kblk, const GvParams& p,
                                          const uint8_t* smem, int& dot_out) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb);
    const uint4 w = *reinterpret_cast<const uint4*>(sb + 16 + 16 * u);
    const uint8_t* xa = smem + p.off_xA + kblk * 256 + 16 * u;
    const int4 xl = *reinterpret_cast<const int4*>(xa);
    const int4 xh = *reinterpret_cast<const int4*>(xa + 128);
    int dlo, dhi;
    if (XM == 0) {
        dlo = dp4a_us(w.x & 0x0F0F0F0Fu, xl.x, 0); dlo = dp4a_us(w.y & 0x0F0F0F0Fu, xl.y, dlo);
        dlo = dp4a_us(w.z & 0x0F0F0F0Fu, xl.z, dlo); dlo = dp4a_us(w.w & 0x0F0F0F0Fu, xl.w, dlo);
        dhi = dp4a_us(w.x & 0xF0F0F0F0u, xh.x, 0); dhi = dp4a_us(w.y & 0xF0F0F0F0u, xh.y, dhi);
        dhi = dp4a_us(w.z & 0xF0F0F0F0u, xh.z, dhi); dhi = dp4a_us(w.w & 0xF0F0F0F0u, xh.w, dhi);
        dhi >>= 4;      // the masked byte is 16*nibble, the sum is an exact multiple of 16
    } else {
        const uint4 yl = *reinterpret_cast<const uint4*>(xa + p.K);
        const uint4 yh = *reinterpret_cast<const uint4*>(xa + p.K + 128);
        int a = dp4a_us(w.x & 0x0F0F0F0Fu, xl.x, 0); a = dp4a_us(w.y & 0x0F0F0F0Fu, xl.y, a);
        a = dp4a_us(w.z & 0x0F0F0F0Fu, xl.z, a); a = dp4a_us(w.w & 0x0F0F0F0Fu, xl.w, a);
        int b = dp4a_uu(w.x & 0x0F0F0F0Fu, yl.x, 0); b = dp4a_uu(w.y & 0x0F0F0F0Fu, yl.y, b);
        b = dp4a_uu(w.z & 0x0F0F0F0Fu, yl.z, b); b = dp4a_uu(w.w & 0x0F0F0F0Fu, yl.w, b);
        dlo = a * 256 + b;
        a = dp4a_us(w.x & 0xF0F0F0F0u, xh.x, 0); a = dp4a_us(w.y & 0xF0F0F0F0u, xh.y, a);
        a = dp4a_us(w.z & 0xF0F0F0F0u, xh.z, a); a = dp4a_us(w.w & 0xF0F0F0F0u, xh.w, a);
        b = dp4a_uu(w.x & 0xF0F0F0F0u, yh.x, 0); b = dp4a_uu(w.y & 0xF0F0F0F0u, yh.y, b);
        b = dp4a_uu(w.z & 0xF0F0F0F0u, yh.z, b); b = dp4a_uu(w.w & 0xF0F0F0F0u, yh.w, b);
        dhi = (a * 256 + b) >> 4;
    }
    const bool odd = u & 1;
    const int keep = odd ? dhi : dlo, send = odd ? dlo : dhi;
    const int dot = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
    dot_out = dot;
    int sc, mn;
    scale_min_k4(u, hdr.y, hdr.z, hdr.w, sc, mn);
    const float dall = h2f_bits(hdr.x & 0xFFFFu), dmin = h2f_bits(hdr.x >> 16);
    const float d8 = reinterpret_cast<const float*>(smem + p.off_xd)[kblk * 8 + u];
    const float s8 = reinterpret_cast<const float*>(smem + p.off_xs)[kblk * 8 + u];
    return __fsub_rn(__fmul_rn(__fmul_rn(dall, (float)sc), __fmul_rn(d8, (float)dot)),
                     __fmul_rn(__fmul_rn(dmin, (float)mn), s8));
}

// 16 bytes from a 2-byte aligned shared-memory address: five aligned words, funnel-shifted.
__device__ __forceinline__ void lds16_unaligned(const uint8_t* ptr, uint32_t out[4]) {
    const uint32_t a = smem_u32(ptr), base = a & ~3u, sh = (a & 2u) * 8u;
    uint32_t w[5];
    #pragma unroll
    for (int i = 0; i < 5; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(base + 4 * i));
    #pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}

// ── Q6_K: one (half n, column run c) per lane = 64 weights in four 16-element scale
// groups (quarters k = 0..3 at +32k), reference arithmetic src/kernels/gemv_q4.cu:581-618:
// per group  d*sc*(d8*dot)  with dot = Σ(q6-32)·x = Σq6·x - 32·Σx.
template <int XM>
__device__ __forceinline__ float q6k_item(const uint8_t* sb, int n, int c, int kblk, const GvParams& p,
                                          const uint8_t* smem, int dots_out[4]) {
    uint32_t A[4], B[4], H[4];
    lds16_unaligned(sb + 64 * n + 16 * c, A);
    lds16_unaligned(sb + 64 * n + 32 + 16 * c, B);
    lds16_unaligned(sb + 128 + 32 * n + 16 * c, H);
    const float d = h2f_bits(*reinterpret_cast<const unsigned short*>(sb + 208));
    const int8_t* scp = reinterpret_cast<const int8_t*>(sb + 192 + 8 * n + c);
    const uint8_t* xb = smem + p.off_xB + (kblk * 4 + 2 * n + c) * 16;
    const int*   xsum = reinterpret_cast<const int*>(smem + p.off_xsum) + kblk * 16 + 8 * n + c;
    const float* xd   = reinterpret_cast<const float*>(smem + p.off_xd) + kblk * 8 + 4 * n;
    float acc = 0.f;
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int4 xv = *reinterpret_cast<const int4*>(xb + k * (p.K >> 2));
        const int xw[4] = { xv.x, xv.y, xv.z, xv.w };
        uint32_t yw[4] = { 0, 0, 0, 0 };
        if (XM == 1) {
            const uint4 yv = *reinterpret_cast<const uint4*>(xb + p.K + k * (p.K >> 2));
            yw[0] = yv.x; yw[1] = yv.y; yw[2] = yv.z; yw[3] = yv.w;
        }
        int dh = 0, dl = 0;
        #pragma unroll
        for (int w = 0; w < 4; ++w) {
            uint32_t v;
            if (k == 0)      v = (A[w] & 0x0F0F0F0Fu) | ((H[w] << 4) & 0x30303030u);
            else if (k == 1) v = (B[w] & 0x0F0F0F0Fu) | ((H[w] << 2) & 0x30303030u);
            else if (k == 2) v = ((A[w] >> 4) & 0x0F0F0F0Fu) | (H[w] & 0x30303030u);
            else             v = ((B[w] >> 4) & 0x0F0F0F0Fu) | ((H[w] >> 2) & 0x30303030u);
            dh = dp4a_us(v, xw[w], dh);
            if (XM == 1) dl = dp4a_uu(v, yw[w], dl);
        }
        const int dot = (XM == 1 ? dh * 256 + dl : dh) - 32 * xsum[2 * k];
        dots_out[k] = dot;
        const float sc = (float)scp[2 * k];
        acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(d, sc), __fmul_rn(xd[k], (float)dot)));
    }
    return acc;
}

struct GvPiece { int first, last, nch; };

__device__ __forceinline__ void gv_chunk(const GvParams& p, const GvPiece pc[3], int c, int& seg, int& r0, int& nrows) {
    seg = 0;
    #pragma unroll
    for (int i = 0; i < 2; ++i)
        if (seg == i && c >= pc[i].nch && i + 1 < p.nseg) { c -= pc[i].nch; seg = i + 1; }
    const int trc = p.seg[seg].trc;
    r0 = pc[seg].first + c * trc;
    nrows = min(trc, pc[seg].last - r0);
}

__device__ __forceinline__ void gv_issue(const GvParams& p, const GvPiece pc[3], int c, uint8_t* smem, uint64_t* full) {
    int seg, r0, nrows;
    gv_chunk(p, pc, c, seg, r0, nrows);
    const GvSegDev& s = p.seg[seg];
    const uintptr_t g0 = (uintptr_t)s.W + (size_t)r0 * s.rb, g1 = g0 + (size_t)nrows * s.rb;
    const uintptr_t a0 = g0 & ~(uintptr_t)15;
    const uintptr_t endw = ((uintptr_t)s.W + (size_t)s.M * s.rb) & ~(uintptr_t)15;
    uintptr_t a1 = (g1 + 15) & ~(uintptr_t)15;
    if (a1 > endw) a1 = endw;                     // never read past the tensor; the tail comes by plain loads
    const int slot = c % p.nslots;
    const uint32_t bytes = (uint32_t)(a1 - a0);
    mbar_expect_tx(&full[slot], bytes);
    bulk_g2s(smem + p.off_slots + (size_t)slot * p.slot_bytes, (const void*)a0, bytes, &full[slot]);
}

template <int XM>
__global__ void __launch_bounds__(GV_THREADS, 2) gemv_stream_kernel(const __grid_constant__ GvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GV_MAXSLOT];
    __shared__ float red[GV_WARPS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // this CTA's rows in every segment
    GvPiece pc[3];
    int nchunks = 0, pair_first = 0;
    {
        const long long G = gridDim.x, b = blockIdx.x;
        if (p.paired_rows) {      // out_mode 3: the same row range of both matrices
            const int M = p.seg[0].M;
            const int f = (int)((long long)M * b / G), l = (int)((long long)M * (b + 1) / G);
            pair_first = f;
            #pragma unroll
            for (int i = 0; i < 2; ++i) { pc[i].first = f; pc[i].last = l; pc[i].nch = (l - f + p.seg[i].trc - 1) / p.seg[i].trc; nchunks += pc[i].nch; }
            pc[2].first = pc[2].last = pc[2].nch = 0;
        } else {
            const long long lo = p.total_bytes * b / G, hi = p.total_bytes * (b + 1) / G;
            long long cum = 0;
            #pragma unroll
            for (int i = 0; i < 3; ++i) {
                pc[i].first = pc[i].last = pc[i].nch = 0;
                if (i < p.nseg) {
                    const long long rb = p.seg[i].rb, M = p.seg[i].M;
                    long long f = lo - cum <= 0 ? 0 : (lo - cum + rb - 1) / rb;
                    long long l = hi - cum <= 0 ? 0 : (hi - cum + rb - 1) / rb;
                    f = f > M ? M : f; l = l > M ? M : l;
                    pc[i].first = (int)f; pc[i].last = (int)l;
                    pc[i].nch = (int)((l - f + p.seg[i].trc - 1) / p.seg[i].trc);
                    nchunks += pc[i].nch;
                    cum += rb * M;
                }
            }
        }
    }
    if (tid == 0) {
        for (int s = 0; s < p.nslots; ++s) mbar_init(&full[s], 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (tid == 0) {
        const int pre = nchunks < p.nslots ? nchunks : p.nslots;
        for (int c = 0; c < pre; ++c) gv_issue(p, pc, c, smem, full);   // weights do not depend on the previous kernel
    }
    pdl_wait();                  // x (and the residual) come from the kernel before us
    stage_x<XM>(p, smem, red);
    __syncthreads();
    pdl_launch();

    float* gate_s = reinterpret_cast<float*>(smem + p.off_gate);
    bool timed_out = false;
    for (int c = 0; c < nchunks; ++c) {
        const int slot = c % p.nslots;
        // a wait that runs out is recorded and the loop carries on (every thread still
        // reaches every barrier below); later waits are skipped
        if (!timed_out && !mbar_wait_bounded(&full[slot], (c / p.nslots) & 1)) timed_out = true;
        int seg, r0, nrows;
        gv_chunk(p, pc, c, seg, r0, nrows);
        const GvSegDev& s = p.seg[seg];
        const uintptr_t g0 = (uintptr_t)s.W + (size_t)r0 * s.rb;
        uint8_t* sdata = smem + p.off_slots + (size_t)slot * p.slot_bytes + (g0 & 15);
        {   // bytes between the last 16-byte boundary inside the tensor and its end
            const uintptr_t g1 = g0 + (size_t)nrows * s.rb;
            const uintptr_t endw = ((uintptr_t)s.W + (size_t)s.M * s.rb) & ~(uintptr_t)15;
            if (g1 > endw) {     // CTA-uniform
                const int tail = (int)(g1 - endw);
                if (tid < tail) sdata[(endw - g0) + tid] = reinterpret_cast<const uint8_t*>(endw)[tid];
                __syncthreads();
            }
        }
        const int R = s.R, wrow0 = warp * R;
        const int nrw = max(0, min(R, nrows - wrow0));
        if (nrw > 0) {
            const uint8_t* rows = sdata + (size_t)wrow0 * s.rb;
            const int U = s.U, total = nrw * U;
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            for (int base = 0; base < total; base += 32) {
                const int i = base + lane;
                const bool valid = i < total;
                const int ii = valid ? i : 0;
                const int rl = (ii >= U) + (ii >= 2 * U) + (ii >= 3 * U);
                const int j = ii - rl * U;
                float term;
                if (s.type == T_Q4K) {
                    const int blk = j >> 3, u = j & 7;
                    int dot;
                    term = q4k_item<XM>(rows + (size_t)rl * s.rb + blk * Q4K_BYTES, u, blk, p, smem, dot);
                    if (p.dbg_dots && seg == 0 && valid)
                        p.dbg_dots[(size_t)(r0 + wrow0 + rl) * (U) + j] = dot;
                } else {
                    const int blk = j >> 2, n = (j >> 1) & 1, cc = j & 1;
                    int dots[4];
                    term = q6k_item<XM>(rows + (size_t)rl * s.rb + blk * Q6K_BYTES, n, cc, blk, p, smem, dots);
                    if (p.dbg_dots && seg == 0 && valid) {
                        int32_t* o = p.dbg_dots + (size_t)(r0 + wrow0 + rl) * (U * 4) + blk * 16 + 8 * n + cc;
                        o[0] = dots[0]; o[2] = dots[1]; o[4] = dots[2]; o[6] = dots[3];
                    }
                }
                if (!valid) term = 0.f;
                acc[0] += rl == 0 ? term : 0.f; acc[1] += rl == 1 ? term : 0.f;
                acc[2] += rl == 2 ? term : 0.f; acc[3] += rl == 3 ? term : 0.f;
            }
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (r < nrw) {
                    const float v = warp_sum(acc[r]);
                    if (lane == 0) {
                        const int row = r0 + wrow0 + r;
                        if (p.out_mode == 0)      reinterpret_cast<__half*>(s.y)[row] = __float2half_rn(v);
                        else if (p.out_mode == 1) reinterpret_cast<float*>(s.y)[row] = v;
                        else if (p.out_mode == 2) {   // src/kernels/gemv_q4.cu:996-999
                            const __half pr = __float2half_rn(v);
                            reinterpret_cast<__half*>(s.y)[row] = __float2half_rn(__fadd_rn(__half2float(pr), __half2float(p.residual[row])));
                        } else {                      // fused SwiGLU of the gate/up pair (src/kernels/convert.cu:85-104)
                            const float hv = __half2float(__float2half_rn(v));
                            if (seg == 0) gate_s[row - pair_first] = hv;
                            else {
                                const float g = gate_s[row - pair_first];
                                reinterpret_cast<__half*>(p.seg[0].y)[row] =
                                    __float2half_rn(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), hv));
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();                         // every warp is done with this slot
        if (tid == 0 && c + p.nslots < nchunks) { fence_proxy_async(); gv_issue(p, pc, c + p.nslots, smem, full); }
    }
    if (timed_out && tid == 0) atomicExch(p.status, JB_ERR_TIMEOUT);
}

// ── Q5_K (and nothing else): plain warp-per-row kernel with the reference's float
// arithmetic, src/kernels/gemv_q4.cu:318-363.  Q5_K is not in any benchmark shape.
__global__ void gemv_q5k_kernel(__half* y, float* y32, const uint8_t* W, const __half* x, const __half* residual, int M, int K) {
    pdl_wait();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const int nb = K / QK_K;
    float acc = 0.f;
    for (int b = 0; b < nb; ++b) {
        const uint8_t* blk = W + ((size_t)row * nb + b) * Q5K_BYTES;
        const float dall = h2f_bits(blk[0] | (blk[1] << 8)), dmin = h2f_bits(blk[2] | (blk[3] << 8));
        const uint32_t s0 = blk[4] | (blk[5] << 8) | (blk[6] << 16) | ((uint32_t)blk[7] << 24);
        const uint32_t s1 = blk[8] | (blk[9] << 8) | (blk[10] << 16) | ((uint32_t)blk[11] << 24);
        const uint32_t s2 = blk[12] | (blk[13] << 8) | (blk[14] << 16) | ((uint32_t)blk[15] << 24);
        const uint8_t qh = blk[16 + lane];
        for (int il = 0; il < 4; ++il) {
            int sc1, m1, sc2, m2;
            scale_min_k4(2 * il, s0, s1, s2, sc1, m1); scale_min_k4(2 * il + 1, s0, s1, s2, sc2, m2);
            const uint8_t q = blk[48 + 32 * il + lane];
            const float wlo = __fsub_rn(__fmul_rn(__fmul_rn(dall, (float)sc1), (float)((q & 0xF) + ((qh >> (2 * il)) & 1) * 16)), __fmul_rn(dmin, (float)m1));
            const float whi = __fsub_rn(__fmul_rn(__fmul_rn(dall, (float)sc2), (float)((q >> 4) + ((qh >> (2 * il + 1)) & 1) * 16)), __fmul_rn(dmin, (float)m2));
            acc += wlo * __half2float(x[b * QK_K + 64 * il + lane]);
            acc += whi * __half2float(x[b * QK_K + 64 * il + 32 + lane]);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        if (y32) y32[row] = acc;
        else if (residual) y[row] = __float2half_rn(__half2float(__float2half_rn(acc)) + __half2float(residual[row]));
        else y[row] = __float2half_rn(acc);
    }
}

int launch_gemv_q5k(__half* y, float* y32, const void* W, const __half* x, const __half* residual, int M, int K, cudaStream_t st) {
    if (M <= 0) return JB_OK;
    JB_CUDA(launch_k(gemv_q5k_kernel, dim3((M + 3) / 4), dim3(128), 0, st, pdl_enabled(), y, y32,
                     (const uint8_t*)W, x, residual, M, K));
    count_launch();
    return JB_OK;
}

static int pick_rows_per_warp(int U, int rb, int chunk_cap) {
    int best = 1; double best_eff = -1.0;
    for (int R = 1; R <= 4; R *= 2) {
        if ((long long)GV_WARPS * R * rb + 16 > chunk_cap) break;
        const int items = R * U, iters = (items + 31) / 32;
        const double eff = (double)items / (32.0 * iters);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = R; }
    }
    return best;
}

int launch_gemv(const GemvArgs& a, cudaStream_t st) {
    if (a.nseg < 1 || a.nseg > 3) return set_error(JB_ERR_ARG, "gemv: nseg=%d", a.nseg);
    if (a.K <= 0 || a.K % QK_K) return set_error(JB_ERR_ARG, "gemv: K=%d is not a positive multiple of 256", a.K);
    if (a.K > 32768) return set_error(JB_ERR_LIMIT, "gemv: K=%d exceeds the supported 32768", a.K);
    if (!a.x) return set_error(JB_ERR_PTR, "gemv: null activation pointer");
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    GvParams p = {};
    p.nseg = a.nseg; p.x = a.x; p.K = a.K; p.out_mode = a.out_mode; p.residual = a.residual;
    p.do_norm = a.do_norm; p.norm_w = a.norm_w; p.norm_w_fp32 = a.norm_w_fp32; p.eps = a.eps;
    p.dbg_dots = a.dbg_dots; p.status = cx->d_status;
    const int nb = a.K / QK_K;
    long long total_rows = 0;
    for (int i = 0; i < a.nseg; ++i) {
        const GemvSeg& s = a.seg[i];
        if (s.type != T_Q4K && s.type != T_Q6K) return set_error(JB_ERR_TYPE, "gemv: ggml type %d has no streaming path", s.type);
        if (!s.W || !s.y) return set_error(JB_ERR_PTR, "gemv: null weight or output pointer");
        if (s.M < 0) return set_error(JB_ERR_ARG, "gemv: M=%d", s.M);
        if (s.type == T_Q4K && ((uintptr_t)s.W & 15)) return set_error(JB_ERR_PTR, "gemv: Q4_K weights must be 16-byte aligned");
        if (s.type == T_Q6K && ((uintptr_t)s.W & 1))  return set_error(JB_ERR_PTR, "gemv: Q6_K weights must be 2-byte aligned");
        if (s.type == T_Q4K) p.needA = 1; else p.needB = 1;
        total_rows += s.M;
    }
    if (total_rows == 0) return JB_OK;
    if (a.out_mode == 2 && (a.nseg != 1 || !a.residual)) return set_error(JB_ERR_ARG, "gemv: residual epilogue needs one matrix and a residual");
    if (a.out_mode == 3 && (a.nseg != 2 || a.seg[0].M != a.seg[1].M)) return set_error(JB_ERR_ARG, "gemv: SwiGLU epilogue needs two matrices of equal height");
    // shared-memory plan
    const int K = a.K, planes = a.xmode ? 2 : 1;
    uint32_t off = 0;
    p.off_xA = off; off += p.needA ? planes * K : 0;
    p.off_xB = off; off += p.needB ? planes * K : 0;
    p.off_xd = off; off += (K / 32) * 4;
    p.off_xs = off; off += (K / 32) * 4;
    p.off_xsum = off; off += p.needB ? (K / 16) * 4 : 0;
    int grid = cx->sm_count * 2;
    p.paired_rows = a.out_mode == 3;
    {   // rows of one CTA in paired mode: at most max(ceil(M/grid), 16) + 2
        int rows = p.paired_rows ? (a.seg[0].M + grid - 1) / grid : 0;
        rows = rows < 16 ? 16 : rows;
        p.off_gate = off; off += p.paired_rows ? (uint32_t)(rows + 2) * 4 : 0;
    }
    off = (off + 127) & ~127u;
    p.off_slots = off;
    const int ring_budget = GV_SMEM_BUDGET - (int)off;
    const int chunk_cap = ring_budget / 2 - 16;
    int slot = 0;
    for (int i = 0; i < a.nseg; ++i) {
        GvSegDev& d = p.seg[i];
        d.W = (const uint8_t*)a.seg[i].W; d.y = a.seg[i].y; d.M = a.seg[i].M; d.type = a.seg[i].type;
        d.rb = nb * block_bytes(d.type);
        d.U = d.type == T_Q4K ? nb * 8 : nb * 4;
        if (d.rb + 16 > chunk_cap) return set_error(JB_ERR_LIMIT, "gemv: one row (%d B) does not fit a staging slot", d.rb);
        d.R = pick_rows_per_warp(d.U, d.rb, chunk_cap);
        d.trc = GV_WARPS * d.R;
        if ((long long)d.trc * d.rb + 16 > chunk_cap) { d.R = 1; d.trc = (chunk_cap - 16) / d.rb; if (d.trc > GV_WARPS) d.trc = GV_WARPS; }
        const int need = ((d.trc * d.rb + 16 + 127) / 128) * 128;
        slot = need > slot ? need : slot;
        p.total_bytes += (long long)d.rb * d.M;
    }
    p.slot_bytes = slot;
    p.nslots = ring_budget / slot;
    if (p.nslots > GV_MAXSLOT) p.nslots = GV_MAXSLOT;
    if (p.nslots < 2) return set_error(JB_ERR_LIMIT, "gemv: staging ring does not fit (slot %d B)", slot);
    const size_t smem_bytes = (size_t)p.off_slots + (size_t)p.nslots * slot;
    int min_trc = p.seg[0].trc;
    for (int i = 1; i < a.nseg; ++i) min_trc = p.seg[i].trc < min_trc ? p.seg[i].trc : min_trc;
    const long long max_useful = (total_rows + min_trc - 1) / min_trc;
    if (grid > max_useful) grid = (int)max_useful;
    if (grid < 1) grid = 1;
    auto kern = a.xmode ? gemv_stream_kernel<1> : gemv_stream_kernel<0>;
    if (!cx->gemv_attr[a.xmode ? 1 : 0]) {
        JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GV_SMEM_BUDGET));
        cx->gemv_attr[a.xmode ? 1 : 0] = true;
    }
    JB_CUDA(launch_k(kern, dim3(grid), dim3(GV_THREADS), smem_bytes, st, pdl_enabled(), p));
    count_launch();
    return JB_OK;
}

}  // namespace jb
