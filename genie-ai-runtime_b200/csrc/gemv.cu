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

struct GvSegDev {
    const uint8_t* W; void* y; int M; int type;
    int rb;          // row bytes
    int U;           // work items per row: 4 per super-block for both types
    int R;           // rows per warp pass ("row group")
    int trc;         // rows per chunk = GV_WARPS * R
};
struct GvParams {
    GvSegDev seg[3]; int nseg;
    const __half* x; int K;
    int out_mode; const __half* residual;
    int do_norm; const void* norm_w; int norm_w_fp32; float eps;
    int32_t* dbg_dots; int* status;
    int slot_bytes, nslots, needA, needB, paired_rows;
    uint32_t off_xA, off_xB, off_xd, off_xs, off_xsum, off_gate, off_slots;
    long long total_bytes;      // Σ over segments of (row groups x bytes per group)
};

// ── activation staging ───────────────────────────────────────────────────
// Layout A (read by Q4_K items), per 256 elements: the 16-element run r = 2*(j>>1)+h of sub-block j = 2*il + p
// (p = 0: low-nibble partners, p = 1: high-nibble partners) sits at p*128 + (16*r ^ 16*(blk&1)) — the xor keeps
// the 16-byte reads of eight neighbouring lanes (two blocks x four il) on different banks.  Layout B (Q6_K
// items): plane k (= 32-wide quarter of a 128-half) at k*K/4, run (blk*4 + 2n + c)*16.  In 16-bit mode a
// second plane with the low bytes follows at +K.
template <int XM>
__device__ __forceinline__ void stage_x(const GvParams& p, uint8_t* smem, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.K;
    float rrms = 1.0f;
    if (p.do_norm) {   // reference: fused_rmsnorm_residual, src/kernels/fused_norm.cu:33-101
        float ss = 0.f;
        for (int g8 = tid; g8 < K / 8; g8 += GV_THREADS) {
            const uint4 raw = *reinterpret_cast<const uint4*>(p.x + 8 * g8);
            const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
            #pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i])); ss += a.x * a.x + a.y * a.y; }
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        #pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) tot += red[w];
        rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
    }
    uint8_t* xA = smem + p.off_xA; uint8_t* xB = smem + p.off_xB;
    float* xd = reinterpret_cast<float*>(smem + p.off_xd);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    int*   xsum = reinterpret_cast<int*>(smem + p.off_xsum);
    // one thread per 32-element group: no shuffles, one pair of divisions per group
    for (int gi = tid; gi < K / 32; gi += GV_THREADS) {
        float v[32];
        #pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 raw = *reinterpret_cast<const uint4*>(p.x + 32 * gi + 8 * q4);
            const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                v[8 * q4 + 2 * i] = a.x; v[8 * q4 + 2 * i + 1] = a.y;
            }
        }
        if (p.do_norm) {
            float wn[32];
            if (p.norm_w_fp32) {
                #pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    const float4 w4 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + 32 * gi + 4 * q4);
                    wn[4 * q4] = w4.x; wn[4 * q4 + 1] = w4.y; wn[4 * q4 + 2] = w4.z; wn[4 * q4 + 3] = w4.w;
                }
            } else {
                #pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.norm_w) + 32 * gi + 8 * q4);
                    const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
                    #pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                        wn[8 * q4 + 2 * i] = a.x; wn[8 * q4 + 2 * i + 1] = a.y;
                    }
                }
            }
            #pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i], rrms), wn[i])));
        }
        float amax = 0.f;
        #pragma unroll
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const float lim = XM == 0 ? 127.0f : 32767.0f;
        const float d = __fdiv_rn(amax, lim);                      // q8_1: src/kernels/gemv_q4.cu:445-466
        const float id = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
        uint32_t hi[8], lo[8];
        int s16[2] = { 0, 0 };
        float fsum = 0.f;
        #pragma unroll
        for (int w = 0; w < 8; ++w) {
            hi[w] = 0; lo[w] = 0;
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x = v[4 * w + i];
                const int q = max(-(int)lim, min((int)lim, __float2int_rn(__fmul_rn(x, id))));
                s16[w >> 2] += q;
                if (XM == 0) hi[w] |= (uint32_t)(q & 0xFF) << (8 * i);
                else { hi[w] |= (uint32_t)((q >> 8) & 0xFF) << (8 * i); lo[w] |= (uint32_t)(q & 0xFF) << (8 * i); }
            }
        }
        if (XM == 1) {
            // fp32 sum of the group in the order of an 8-lane xor tree over 4-element partial sums
            float ps[8];
            #pragma unroll
            for (int w = 0; w < 8; ++w) ps[w] = (v[4 * w] + v[4 * w + 1]) + (v[4 * w + 2] + v[4 * w + 3]);
            fsum = ((ps[0] + ps[1]) + (ps[2] + ps[3])) + ((ps[4] + ps[5]) + (ps[6] + ps[7]));
        }
        const int blk = gi >> 3, j = gi & 7;
        if (p.needA) {
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int off = blk * 256 + (j & 1) * 128 + (((2 * (j >> 1) + h) * 16) ^ ((blk & 1) << 4));
                *reinterpret_cast<uint4*>(xA + off) = make_uint4(hi[4 * h], hi[4 * h + 1], hi[4 * h + 2], hi[4 * h + 3]);
                if (XM == 1) *reinterpret_cast<uint4*>(xA + K + off) = make_uint4(lo[4 * h], lo[4 * h + 1], lo[4 * h + 2], lo[4 * h + 3]);
            }
        }
        if (p.needB) {
            const int n = j >> 2, k = j & 3;
            #pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int off = k * (K >> 2) + (blk * 4 + 2 * n + c) * 16;
                *reinterpret_cast<uint4*>(xB + off) = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
                if (XM == 1) *reinterpret_cast<uint4*>(xB + K + off) = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
                xsum[2 * gi + c] = s16[c];
            }
        }
        if (XM == 0) {
            xd[gi] = __half2float(__float2half_rn(d));
            xs[gi] = __half2float(__float2half_rn(__fmul_rn(d, (float)(s16[0] + s16[1]))));
        } else {
            xd[gi] = d;
            xs[gi] = fsum;
        }
    }
}

__device__ __forceinline__ int dot16_us(const uint4& w, uint32_t mask, const int4& x) {
    int d = dp4a_us(w.x & mask, x.x, 0); d = dp4a_us(w.y & mask, x.y, d);
    d = dp4a_us(w.z & mask, x.z, d);     return dp4a_us(w.w & mask, x.w, d);
}
__device__ __forceinline__ int dot16_uu(const uint4& w, uint32_t mask, const uint4& x) {
    int d = dp4a_uu(w.x & mask, x.x, 0); d = dp4a_uu(w.y & mask, x.y, d);
    d = dp4a_uu(w.z & mask, x.z, d);     return dp4a_uu(w.w & mask, x.w, d);
}

// ── Q4_K: one 32-byte group of quants per lane ───────────────────────────
// Group il (0..3) of a block holds the low nibbles of sub-block 2*il and the high nibbles of sub-block
// 2*il+1, 32 elements each.  The lane builds both complete 32-element integer dots — the accumulators the
// reference builds with eight dp4a each (src/kernels/gemv_q4.cu:487-494) — and folds them as
//   dall * (sc0*dot0*d8_0 + sc1*dot1*d8_1) - dmin * (m0*s8_0 + m1*s8_1)
// which is the reference's  Σ dall*sc*(d8*dot) - dmin*m*s8  (:499) with the common factors taken out.
template <int XM>
__device__ __forceinline__ float q4k_item(const uint8_t* sb, int il, int kblk, const GvParams& p,
                                          const uint8_t* smem, int& dot0, int& dot1) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb);
    const uint4 w0 = *reinterpret_cast<const uint4*>(sb + 16 + 32 * il);
    const uint4 w1 = *reinterpret_cast<const uint4*>(sb + 32 + 32 * il);
    const int sw = (kblk & 1) << 4;
    const uint8_t* xa = smem + p.off_xA + kblk * 256;
    const int o0 = (32 * il) ^ sw, o1 = (32 * il + 16) ^ sw;
    const int4 xl0 = *reinterpret_cast<const int4*>(xa + o0), xl1 = *reinterpret_cast<const int4*>(xa + o1);
    const int4 xh0 = *reinterpret_cast<const int4*>(xa + 128 + o0), xh1 = *reinterpret_cast<const int4*>(xa + 128 + o1);
    if (XM == 0) {
        dot0 = dot16_us(w0, 0x0F0F0F0Fu, xl0) + dot16_us(w1, 0x0F0F0F0Fu, xl1);
        dot1 = (dot16_us(w0, 0xF0F0F0F0u, xh0) + dot16_us(w1, 0xF0F0F0F0u, xh1)) >> 4;   // exact: every term is a multiple of 16
    } else {
        const uint8_t* xb = xa + p.K;
        const uint4 yl0 = *reinterpret_cast<const uint4*>(xb + o0), yl1 = *reinterpret_cast<const uint4*>(xb + o1);
        const uint4 yh0 = *reinterpret_cast<const uint4*>(xb + 128 + o0), yh1 = *reinterpret_cast<const uint4*>(xb + 128 + o1);
        dot0 = (dot16_us(w0, 0x0F0F0F0Fu, xl0) + dot16_us(w1, 0x0F0F0F0Fu, xl1)) * 256 +
               (dot16_uu(w0, 0x0F0F0F0Fu, yl0) + dot16_uu(w1, 0x0F0F0F0Fu, yl1));
        dot1 = ((dot16_us(w0, 0xF0F0F0F0u, xh0) + dot16_us(w1, 0xF0F0F0F0u, xh1)) * 16 +
                ((dot16_uu(w0, 0xF0F0F0F0u, yh0) + dot16_uu(w1, 0xF0F0F0F0u, yh1)) >> 4));
    }
    // scales / mins of sub-blocks 2*il and 2*il+1 (two adjacent bytes), both halves of get_scale_min_k4 at once
    const int sh = 16 * (il & 1);
    const uint32_t a = (hdr.y >> sh) & 0xFFFFu, b = (hdr.z >> sh) & 0xFFFFu, c = (hdr.w >> sh) & 0xFFFFu;
    const bool hi = il >= 2;
    const uint32_t sc2 = hi ? ((c & 0x0F0Fu) | ((a >> 2) & 0x3030u)) : (a & 0x3F3Fu);
    const uint32_t mn2 = hi ? (((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u)) : (b & 0x3F3Fu);
    const float dall = h2f_bits(hdr.x & 0xFFFFu), dmin = h2f_bits(hdr.x >> 16);
    const float2 d8 = *reinterpret_cast<const float2*>(smem + p.off_xd + (kblk * 8 + 2 * il) * 4);
    const float2 s8 = *reinterpret_cast<const float2*>(smem + p.off_xs + (kblk * 8 + 2 * il) * 4);
    const float pos = (float)((int)(sc2 & 0xFF) * dot0) * d8.x + (float)((int)(sc2 >> 8) * dot1) * d8.y;
    const float neg = (float)(mn2 & 0xFF) * s8.x + (float)(mn2 >> 8) * s8.y;
    return dall * pos - dmin * neg;
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

// ── Q6_K: one (half n, column run c) per lane = 64 weights in four 16-element scale groups (quarters k = 0..3
// at +32k), reference arithmetic src/kernels/gemv_q4.cu:581-618: per group  d*sc*(d8*dot)  with
// dot = Σ(q6-32)·x = Σq6·x - 32·Σx.
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
    const float4 xd4  = *reinterpret_cast<const float4*>(smem + p.off_xd + (kblk * 8 + 4 * n) * 4);
    const float xdv[4] = { xd4.x, xd4.y, xd4.z, xd4.w };
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
        acc += (float)dot * ((float)scp[2 * k] * xdv[k]);
    }
    return d * acc;
}

// One warp, `nrw` (<= 4) consecutive rows in shared memory: lanes stride over the rows' 32-byte items
// (4 per super-block), each lane adds its terms into the accumulator of the row the item belongs to.
template <int XM, int TYPE, bool DBG>
__device__ __forceinline__ void consume_rows(const uint8_t* rows, int nrw, int rb_, int U_, int lane, const GvParams& p,
                                             const uint8_t* smem, float (&acc)[4], int32_t* dbg) {
    const unsigned rb = (unsigned)rb_, U = (unsigned)U_, total = (unsigned)nrw * U;
    constexpr unsigned BB = TYPE == T_Q4K ? Q4K_BYTES : Q6K_BYTES;
    for (unsigned base = 0; base < total; base += 32) {
        const unsigned i = base + lane;
        const bool valid = i < total;
        const unsigned ii = valid ? i : 0u;
        const unsigned rl = (ii >= U) + (ii >= 2 * U) + (ii >= 3 * U);
        const unsigned j = ii - rl * U, blk = j >> 2, sub = j & 3;
        const uint8_t* sb = rows + rl * rb + blk * BB;
        float term;
        if (TYPE == T_Q4K) {
            int d0, d1;
            term = q4k_item<XM>(sb, (int)sub, (int)blk, p, smem, d0, d1);
            if (DBG && dbg && valid) { int32_t* o = dbg + (size_t)rl * (2 * U) + blk * 8 + 2 * sub; o[0] = d0; o[1] = d1; }
        } else {
            int dots[4];
            term = q6k_item<XM>(sb, (int)(sub >> 1), (int)(sub & 1), (int)blk, p, smem, dots);
            if (DBG && dbg && valid) {
                int32_t* o = dbg + (size_t)rl * (4 * U) + blk * 16 + 8 * (sub >> 1) + (sub & 1);
                o[0] = dots[0]; o[2] = dots[1]; o[4] = dots[2]; o[6] = dots[3];
            }
        }
        if (!valid) term = 0.f;
        acc[0] += rl == 0 ? term : 0.f; acc[1] += rl == 1 ? term : 0.f;
        acc[2] += rl == 2 ? term : 0.f; acc[3] += rl == 3 ? term : 0.f;
    }
}

struct GvPiece { int first, last, nch; };   // rows [first, last) of a segment, chunks of trc rows

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

template <int XM, bool DBG>
__global__ void __launch_bounds__(GV_THREADS, 4) gemv_stream_kernel(const __grid_constant__ GvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GV_MAXSLOT];
    __shared__ float red[GV_WARPS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // this CTA's rows in every segment: an even split of the row groups by bytes
    GvPiece pc[3];
    int nchunks = 0, pair_first = 0;
    {
        const long long G = gridDim.x, b = blockIdx.x;
        if (p.paired_rows) {      // out_mode 3: the same row range of both matrices
            const int R = p.seg[0].R, M = p.seg[0].M, groups = (M + R - 1) / R;
            const int f = min(M, (int)((long long)groups * b / G) * R), l = min(M, (int)((long long)groups * (b + 1) / G) * R);
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
                    const long long R = p.seg[i].R, M = p.seg[i].M, gb = R * p.seg[i].rb, groups = (M + R - 1) / R;
                    long long f = lo - cum <= 0 ? 0 : (lo - cum + gb - 1) / gb;
                    long long l = hi - cum <= 0 ? 0 : (hi - cum + gb - 1) / gb;
                    f = f > groups ? groups : f; l = l > groups ? groups : l;
                    pc[i].first = (int)min(M, f * R); pc[i].last = (int)min(M, l * R);
                    pc[i].nch = (pc[i].last - pc[i].first + p.seg[i].trc - 1) / p.seg[i].trc;
                    nchunks += pc[i].nch;
                    cum += gb * groups;
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
        uint8_t* sdata = smem + p.off_slots + (unsigned)slot * (unsigned)p.slot_bytes + (unsigned)(g0 & 15);
        {   // bytes between the last 16-byte boundary inside the tensor and its end
            const uintptr_t g1 = g0 + (size_t)nrows * s.rb;
            const uintptr_t endw = ((uintptr_t)s.W + (size_t)s.M * s.rb) & ~(uintptr_t)15;
            if (g1 > endw) {     // CTA-uniform
                const int tail = (int)(g1 - endw);
                if (tid < tail) sdata[(endw - g0) + tid] = reinterpret_cast<const uint8_t*>(endw)[tid];
                __syncthreads();
            }
        }
        const int R = s.R, wrow0 = warp * R, type = s.type;
        const int nrw = max(0, min(R, nrows - wrow0));
        if (nrw > 0) {
            const uint8_t* rows = sdata + (unsigned)wrow0 * (unsigned)s.rb;
            float acc[4] = { 0.f, 0.f, 0.f, 0.f };
            int32_t* dbg = (DBG && seg == 0) ? p.dbg_dots + (size_t)(r0 + wrow0) * (type == T_Q4K ? 2 * s.U : 4 * s.U) : nullptr;
            if (type == T_Q4K) consume_rows<XM, T_Q4K, DBG>(rows, nrw, s.rb, s.U, lane, p, smem, acc, dbg);
            else               consume_rows<XM, T_Q6K, DBG>(rows, nrw, s.rb, s.U, lane, p, smem, acc, dbg);
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

// rows per warp pass: the count of 32-byte items of a row group should fill whole warps
static double lane_eff(int R, int U) { const int items = R * U, iters = (items + 31) / 32; return (double)items / (32.0 * iters); }

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
    if (a.out_mode == 3 && (a.nseg != 2 || a.seg[0].M != a.seg[1].M || a.seg[0].type != a.seg[1].type))
        return set_error(JB_ERR_ARG, "gemv: SwiGLU epilogue needs two matrices of equal height and type");
    p.paired_rows = a.out_mode == 3;
    const int K = a.K, planes = a.xmode ? 2 : 1;
    // Try 4, 2, then 1 CTA per SM: the shared-memory budget per CTA decides how many row groups fit a slot.
    const int smem_sm = cx->max_smem_optin + 1024;           // per-SM shared memory (per-CTA opt-in limit + 1 KB reserve)
    for (int cps = 4; cps >= 1; cps >>= 1) {
        int budget = smem_sm / cps - 1024 - 256;              // 1 KB system reserve per CTA, 256 B for static shared memory
        if (budget > cx->max_smem_optin - 1024) budget = cx->max_smem_optin - 1024;
        uint32_t off = 0;
        p.off_xA = off; off += p.needA ? planes * K : 0;
        p.off_xB = off; off += p.needB ? planes * K : 0;
        p.off_xd = off; off += (K / 32) * 4;
        p.off_xs = off; off += (K / 32) * 4;
        p.off_xsum = off; off += p.needB ? (K / 16) * 4 : 0;
        int grid = cx->sm_count * cps;
        {   // rows of one CTA in paired mode: at most max(ceil(M/grid), 16) + 8
            int rows = p.paired_rows ? (a.seg[0].M + grid - 1) / grid : 0;
            rows = rows < 16 ? 16 : rows;
            p.off_gate = off; off += p.paired_rows ? (uint32_t)(rows + 8) * 4 : 0;
        }
        off = (off + 127) & ~127u;
        p.off_slots = off;
        const int ring = budget - (int)off;
        const int chunk_cap = ring / 2 - 16;                  // at least two slots
        bool fits = chunk_cap > 0;
        int slot = 0;
        p.total_bytes = 0;
        double worst_eff = 1.0;
        for (int i = 0; i < a.nseg && fits; ++i) {
            GvSegDev& d = p.seg[i];
            d.W = (const uint8_t*)a.seg[i].W; d.y = a.seg[i].y; d.M = a.seg[i].M; d.type = a.seg[i].type;
            d.rb = nb * block_bytes(d.type);
            d.U = nb * 4;
            int best = 0; double be = -1.0;
            for (int R = 1; R <= 4; R *= 2) {
                if ((long long)GV_WARPS * R * d.rb + 16 > chunk_cap) break;
                const double e = lane_eff(R, d.U);
                if (e > be + 1e-9) { be = e; best = R; }
            }
            if (!best) { fits = false; break; }
            d.R = best; d.trc = GV_WARPS * best;
            worst_eff = be < worst_eff ? be : worst_eff;
            const int need = ((d.trc * d.rb + 16 + 127) / 128) * 128;
            slot = need > slot ? need : slot;
            const long long groups = (d.M + d.R - 1) / d.R;
            p.total_bytes += groups * d.R * d.rb;
        }
        if (!fits) {
            if (cps == 1) return set_error(JB_ERR_LIMIT, "gemv: one row group does not fit the staging ring (K=%d)", K);
            continue;
        }
        (void)worst_eff;
        p.slot_bytes = slot;
        p.nslots = ring / slot;
        if (p.nslots > GV_MAXSLOT) p.nslots = GV_MAXSLOT;
        if (p.nslots < 2) { if (cps == 1) return set_error(JB_ERR_LIMIT, "gemv: staging ring does not fit (slot %d B)", slot); continue; }
        const size_t smem_bytes = (size_t)p.off_slots + (size_t)p.nslots * slot;
        long long groups_total = 0;
        for (int i = 0; i < a.nseg; ++i) groups_total += (p.seg[i].M + p.seg[i].R - 1) / p.seg[i].R;
        if (p.paired_rows) groups_total /= 2;
        if (grid > groups_total) grid = (int)groups_total;
        if (grid < 1) grid = 1;
        auto kern = a.dbg_dots ? (a.xmode ? gemv_stream_kernel<1, true> : gemv_stream_kernel<0, true>)
                               : (a.xmode ? gemv_stream_kernel<1, false> : gemv_stream_kernel<0, false>);
        const int ki = (a.xmode ? 1 : 0) + (a.dbg_dots ? 2 : 0);
        if (!cx->gemv_attr[ki]) {
            JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cx->max_smem_optin - 1024));
            cx->gemv_attr[ki] = true;
        }
        JB_CUDA(launch_k(kern, dim3(grid), dim3(GV_THREADS), smem_bytes, st, pdl_enabled(), p));
        count_launch();
        return JB_OK;
    }
    return set_error(JB_ERR_LIMIT, "gemv: no launch configuration fits (K=%d)", K);
}

}  // namespace jb
