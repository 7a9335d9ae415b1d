// mmq_stream.cu — batched K-quant GEMM for FEW tokens (2..64): the weights are streamed once, as in the GEMV.
//
// y[N x M] = x[N x K] . W^T with the arithmetic of the tensor-core prefill kernel (mmq_tc.cu: fp16 operands built from
// the reference's quantised values — half(d*sc)*(q-8) and half(d8*q8), min term and centring constant as 16 extra K
// columns per super-block, mmq_q4k_llama.cu:159-163, :383-404; mmq_q6k_llama.cu:424-438), so the two kernels give the
// same numbers up to the order of the fp32 accumulation and the existing oracle is the checker.
//
// With N <= 64 the product is bound by HBM (every weight byte is used N times, against ~300 needed to fill the tensor
// pipe), and the 128 x 256 tiles of the prefill kernel leave most of the machine idle.  Here:
//   * a CTA owns 16*RG weight rows (RG row groups of one 16-row MMA tile) and a range of super-blocks; per super-block
//     ONE stage of a CTA-wide ring receives the rows' blocks (16-byte cp.async copies spread over all threads) and the
//     activation operand of ALL tokens for that super-block (one bulk copy: the quantise pre-kernel writes it
//     block-major, [K/256][tokens][288 halves], so that is a contiguous 36 KB at 64 tokens);
//   * FOUR warps share a row group, each taking a quarter of every super-block (two 32-weight sub-blocks): a warp alone
//     runs ~1100 dependent-ish instructions per super-block, and with one warp per row group an SM held 5 warps and issued
//     on a quarter of its cycles; the four partial accumulators are added in a fixed order through shared memory at the end;
//   * a warp dequantises its weights straight into mma.sync.m16n8k16 A fragments in registers (no trip through shared
//     memory) and multiplies them against the 8-token B fragments of all token tiles, read with one 16-byte shared load
//     per (sub-block, token tile); lane c of a quad takes weights 8c..8c+7 of every 32-weight sub-block on both
//     operands, which is a permutation of K inside an MMA and leaves the sums unchanged;
//   * K ranges of one row tile (when the row tiles alone would not fill the SMs) write fp32 partials that a second
//     kernel adds in a fixed order.
// Waits on the stage barriers are bounded; a wait that runs out sets the device status word.
#include "mmq.cuh"
#include <cstdio>
#include <cstdlib>

namespace jb {

constexpr int MS_XROW   = 288;                    // halves per (token, super-block): 256 products, 8 group sums, 8 centring sums, pad
constexpr int MS_XROWB  = MS_XROW * 2;            // 576 B = 144 words = 16 mod 32: the 16-byte reads of a quarter-warp hit 32 banks
constexpr int MS_W4SLOT = 160;                    // Q4_K block slot: 144 B + 16 (40 words = 8 mod 32: conflict-free 8-byte reads of 4 rows)
constexpr int MS_W6SLOT = 240;                    // Q6_K block slot: 210 B at any even offset below 16, rounded to 16
constexpr int MS_MAXRG = 4;                        // row groups per CTA
constexpr int MS_KS = 4;                           // warps per row group (quarters of a super-block)

struct MsArgs {
    __half* y; float* part;                       // output, or fp32 partials [split][N][M] when nsplit > 1
    const __half* res;                            // optional residual [N][M]: y = half(float(res) + float(half(product)))
    const uint8_t* W; const __half* xb;           // weights; activation operand, block-major
    int M, N, NP, K, nb;                          // NP = tokens padded to a multiple of 8
    int rg, nsplit, blocks_per_split, nstage;
    int* status;
};

__device__ __forceinline__ void ms_mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ms_lds128(uint32_t a) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ uint2 ms_lds64(uint32_t a) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ uint32_t ms_lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }

// four codes (one per byte, already masked) -> (q - bias) * s as two half2 words; 0x6400 | q is the half 1024 + q
__device__ __forceinline__ void ms_codes4(uint32_t q4, __half2 kbias, __half2 s, uint32_t& lo, uint32_t& hi) {
    const uint32_t a = __byte_perm(q4, 0x64646464u, 0x4140), b = __byte_perm(q4, 0x64646464u, 0x4342);
    const __half2 ha = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&a), kbias), s);
    const __half2 hb = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&b), kbias), s);
    lo = *reinterpret_cast<const uint32_t*>(&ha); hi = *reinterpret_cast<const uint32_t*>(&hb);
}
// the same with the scale given as an fp16 (hi, lo) split of an fp32 product, so each weight is rounded to fp16 once
__device__ __forceinline__ void ms_codes4_split(uint32_t q4, __half2 kbias, __half2 shi, __half2 slo, uint32_t& lo, uint32_t& hi) {
    const uint32_t a = __byte_perm(q4, 0x64646464u, 0x4140), b = __byte_perm(q4, 0x64646464u, 0x4342);
    const __half2 qa = __hsub2(*reinterpret_cast<const __half2*>(&a), kbias), qb = __hsub2(*reinterpret_cast<const __half2*>(&b), kbias);
    const __half2 ra = __hfma2(qa, shi, __hmul2(qa, slo)), rb = __hfma2(qb, shi, __hmul2(qb, slo));
    lo = *reinterpret_cast<const uint32_t*>(&ra); hi = *reinterpret_cast<const uint32_t*>(&rb);
}

// ── activation operand ────────────────────────────────────────────────────
// One warp per 32-element group of one token (the quantiser of mmq_tc_quantize_kernel, mmq_q4k_llama.cu:383-404 /
// mmq_q6k_llama.cu:424-438), written block-major: xb[(kb * NP + token) * 288 + ...]: 256 products half(d*q) in K order,
// then for Q4_K the 8 group sums half(Σx) and the 8 centring sums half(d*Σq); zero elsewhere and for padded tokens.
__global__ void mms_quantize_kernel(const __half* x, __half* xb, int N, int NP, int K, int ds4) {
    pdl_wait();
    const long long g = (long long)blockIdx.x * blockDim.y + threadIdx.y;
    const int lane = threadIdx.x, G = K / 32;
    if (g >= (long long)NP * G) return;
    const int t = (int)(g / G), gi = (int)(g - (long long)t * G), kb = gi >> 3, j = gi & 7;
    __half* row = xb + ((size_t)kb * NP + t) * MS_XROW;
    if (t >= N) {                                      // padded token: zeros
        row[32 * j + lane] = __float2half_rn(0.f);
        if (lane < 4) row[256 + 4 * j + lane] = __float2half_rn(0.f);
        return;
    }
    const float v = __half2float(x[(size_t)t * K + (size_t)gi * 32 + lane]);
    const float amax = warp_max(fabsf(v));
    float sum = v;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    float d = __fdiv_rn(amax, 127.0f);
    const float dinv = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    const int q = __float2int_rn(__fmul_rn(v, dinv));
    int qsum = q;
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, o);
    if (ds4) d = __half2float(__float2half_rn(d));
    row[32 * j + lane] = __float2half_rn(__fmul_rn(d, (float)q));
    if (lane == 0) {
        row[256 + j] = __float2half_rn(ds4 ? sum : 0.f);
        row[264 + j] = __float2half_rn(ds4 ? __fmul_rn(d, (float)qsum) : 0.f);
    }
    if (lane >= 16 && j < 4) row[272 + 4 * j + (lane - 16) % 4] = __float2half_rn(0.f);      // pad halves 272..287
}

// ── the product ───────────────────────────────────────────────────────────
template <int TYPE, int NT>
__global__ void __launch_bounds__(MS_MAXRG * MS_KS * 32, 1) mms_kernel(const MsArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[4];
    constexpr int BB = TYPE == T_Q4K ? Q4K_BYTES : Q6K_BYTES, WSLOT = TYPE == T_Q4K ? MS_W4SLOT : MS_W6SLOT;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, c = lane & 3;
    const int rows_cta = 16 * a.rg, row0 = blockIdx.x * rows_cta;
    const int rgi = warp >> 2, ks = warp & 3;            // this warp's row group and its quarter of every super-block
    const int kb0 = blockIdx.y * a.blocks_per_split, kb1 = min(a.nb, kb0 + a.blocks_per_split), nk = kb1 - kb0;
    const uint32_t x_bytes = (uint32_t)a.NP * MS_XROWB;
    const uint32_t stage_bytes = x_bytes + (uint32_t)rows_cta * WSLOT;
    const size_t rb = (size_t)a.nb * BB;
    const uintptr_t wend = (uintptr_t)a.W + (size_t)a.M * rb;                         // no copy reads past the tensor

    // A stage is complete when thread 0's bulk copy of the activation chunk has landed and every thread's 16-byte copies of
    // the weight blocks have (cp.async + cp.async.mbarrier.arrive.noinc: one arrival per thread, none of them counted as
    // pending before it is made).  The rows' blocks are 144 / 210 bytes, 16 * WPC of them per super-block: as bulk copies
    // they would be that many tiny TMA transfers per stage, as per-thread 16-byte copies they are five to eight
    // instructions per thread.
    const int live_rows = min(rows_cta, a.M - row0);
    constexpr int CPR = WSLOT / 16;                       // 16-byte pieces per block slot
    if (tid == 0) { for (int s = 0; s < a.nstage; ++s) mbar_init(&full[s], 1u + blockDim.x); fence_mbar_init(); }
    __syncthreads();
    pdl_launch();

    auto issue = [&](int i) {            // chunk i (super-block kb0 + i) -> stage i % nstage; called by every thread
        const int st = i % a.nstage, kb = kb0 + i;
        uint8_t* sx = smem + (size_t)st * stage_bytes;
        uint8_t* sw = sx + x_bytes;
        if (tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(&full[st], x_bytes);
            bulk_g2s(sx, reinterpret_cast<const uint8_t*>(a.xb) + (size_t)kb * x_bytes, x_bytes, &full[st]);
        }
        for (int idx = tid; idx < live_rows * CPR; idx += blockDim.x) {
            const int r = idx / CPR, pc = idx - r * CPR;
            const uintptr_t src = (uintptr_t)a.W + (size_t)(row0 + r) * rb + (size_t)kb * BB;
            const uintptr_t p16 = (src & ~(uintptr_t)15) + 16u * (uintptr_t)pc;
            if (p16 >= src + BB) continue;                                   // a spare piece of the slot
            uint8_t* dst = sw + (size_t)r * WSLOT + 16 * pc;
            if (p16 + 16 <= wend) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"((const void*)p16) : "memory");
            } else {                                                         // the tensor's last bytes: nothing is read past its end
                const uintptr_t tend = (uintptr_t)a.W + (size_t)a.M * rb;
                for (uintptr_t q = p16; q < tend; ++q) dst[q - p16] = *reinterpret_cast<const uint8_t*>(q);
            }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[st])) : "memory");
    };
    // weights do not depend on the producer kernel, the activation operand does: the whole first ring waits for it
    pdl_wait();
    for (int i = 0; i < a.nstage && i < nk; ++i) issue(i);
    __syncthreads();                    // plain stores of a tensor's last bytes (see issue) are visible to every reader from here on

    float acc[NT][4];
    #pragma unroll
    for (int t = 0; t < NT; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
    const bool warp_live = rgi < a.rg && row0 + 16 * rgi < a.M;
    bool timed_out = false;

    for (int i = 0; i < nk; ++i) {
        const int st = i % a.nstage;
        if (!timed_out && !mbar_wait_bounded(&full[st], (uint32_t)(i / a.nstage) & 1u)) timed_out = true;
        const uint32_t sx = smem_u32(smem + (size_t)st * stage_bytes), sw = sx + x_bytes;
        if (warp_live) {
            // this lane's two rows (g and g + 8 of the warp's tile); a row past M reads row 0's slot and is never stored
            const int rA = 16 * rgi + g, rB = rA + 8;
            const bool liveA = row0 + rA < a.M, liveB = row0 + rB < a.M;
            uint32_t pA = sw + (uint32_t)(liveA ? rA : 16 * rgi) * WSLOT, pB = sw + (uint32_t)(liveB ? rB : 16 * rgi) * WSLOT;
            const uint32_t xq = sx + (uint32_t)g * MS_XROWB + (uint32_t)c * 16u;     // token g of tile 0, this lane's 8 halves of sub-block 0
            if (TYPE == T_Q4K) {
                const uint4 hA = ms_lds128(pA), hB = ms_lds128(pB);
                const __half dhA = __ushort_as_half((unsigned short)(hA.x & 0xFFFFu)), dhB = __ushort_as_half((unsigned short)(hB.x & 0xFFFFu));
                const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));      // 1024 + 8
                {
                    const int il = ks;                    // this warp's 64 weights of the block: sub-blocks 2ks (low nibbles), 2ks+1 (high)
                    const uint2 wA = ms_lds64(pA + 16 + 32 * il + 8 * c), wB = ms_lds64(pB + 16 + 32 * il + 8 * c);
                    #pragma unroll
                    for (int sub = 0; sub < 2; ++sub) {
                        const int j = 2 * il + sub;
                        int scA, mnA, scB, mnB;
                        scale_min_k4(j, hA.y, hA.z, hA.w, scA, mnA);
                        scale_min_k4(j, hB.y, hB.z, hB.w, scB, mnB);
                        const __half2 sA = __half2half2(__hmul(dhA, __int2half_rn(scA))), sB = __half2half2(__hmul(dhB, __int2half_rn(scB)));
                        uint32_t k0[4], k1[4];           // A fragments of the sub-block's two k-steps
                        ms_codes4((wA.x >> (4 * sub)) & 0x0F0F0F0Fu, k1032, sA, k0[0], k0[2]);
                        ms_codes4((wA.y >> (4 * sub)) & 0x0F0F0F0Fu, k1032, sA, k1[0], k1[2]);
                        ms_codes4((wB.x >> (4 * sub)) & 0x0F0F0F0Fu, k1032, sB, k0[1], k0[3]);
                        ms_codes4((wB.y >> (4 * sub)) & 0x0F0F0F0Fu, k1032, sB, k1[1], k1[3]);
                        uint4 b[NT];
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) b[t] = ms_lds128(xq + (uint32_t)t * 8u * MS_XROWB + (uint32_t)j * 64u);
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) ms_mma_f16(acc[t], k0, b[t].x, b[t].y);      // NT independent accumulators between
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) ms_mma_f16(acc[t], k1, b[t].z, b[t].w);      // two MMAs into the same one
                    }
                }
                // the extra k-step (first warp of the row group): columns 0..7 = half(-dmin) * half(m_j) against the group sums, 8..15 = 8 * half(d*sc_j)
                // against the centring sums; this lane holds columns 2c, 2c+1 (a0/a1) and 8+2c, 9+2c (a2/a3)
                if (ks == 0) {
                    const __half mhA = __hneg(__ushort_as_half((unsigned short)(hA.x >> 16))), mhB = __hneg(__ushort_as_half((unsigned short)(hB.x >> 16)));
                    const __half eight = __ushort_as_half((unsigned short)0x4800);
                    uint32_t e[4];
                    int s0, m0, s1, m1;
                    scale_min_k4(2 * c, hA.y, hA.z, hA.w, s0, m0); scale_min_k4(2 * c + 1, hA.y, hA.z, hA.w, s1, m1);
                    { const __half2 mn = __halves2half2(__hmul(mhA, __int2half_rn(m0)), __hmul(mhA, __int2half_rn(m1)));
                      const __half2 ce = __halves2half2(__hmul(eight, __hmul(dhA, __int2half_rn(s0))), __hmul(eight, __hmul(dhA, __int2half_rn(s1))));
                      e[0] = *reinterpret_cast<const uint32_t*>(&mn); e[2] = *reinterpret_cast<const uint32_t*>(&ce); }
                    scale_min_k4(2 * c, hB.y, hB.z, hB.w, s0, m0); scale_min_k4(2 * c + 1, hB.y, hB.z, hB.w, s1, m1);
                    { const __half2 mn = __halves2half2(__hmul(mhB, __int2half_rn(m0)), __hmul(mhB, __int2half_rn(m1)));
                      const __half2 ce = __halves2half2(__hmul(eight, __hmul(dhB, __int2half_rn(s0))), __hmul(eight, __hmul(dhB, __int2half_rn(s1))));
                      e[1] = *reinterpret_cast<const uint32_t*>(&mn); e[3] = *reinterpret_cast<const uint32_t*>(&ce); }
                    const uint32_t xe = sx + (uint32_t)g * MS_XROWB + 512u + (uint32_t)c * 4u;
                    #pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const uint32_t b0 = ms_lds32(xe + (uint32_t)t * 8u * MS_XROWB), b1 = ms_lds32(xe + (uint32_t)t * 8u * MS_XROWB + 16u);
                        ms_mma_f16(acc[t], e, b0, b1);
                    }
                }
            } else {
                // Q6_K: blocks are 2-byte aligned; a block starts `dl` bytes into its slot (the copy brought the enclosing
                // 16-byte aligned range).  Every 8-byte field is read as three aligned words and funnel-shifted.
                const uintptr_t srcA = (uintptr_t)a.W + (size_t)(row0 + (liveA ? rA : 16 * rgi)) * rb + (size_t)(kb0 + i) * BB;
                const uintptr_t srcB = (uintptr_t)a.W + (size_t)(row0 + (liveB ? rB : 16 * rgi)) * rb + (size_t)(kb0 + i) * BB;
                pA += (uint32_t)(srcA & 15); pB += (uint32_t)(srcB & 15);
                const __half2 k1056 = __half2half2(__ushort_as_half((unsigned short)0x6420));      // 1024 + 32
                {
                    const int n = ks >> 1, qt0 = 2 * (ks & 1);   // this warp's half of the block and its two quarters
                    uint32_t frag[2][2][4];             // [quarter - qt0][k-step][a0..a3]
                    #pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        const uint32_t p = rs ? pB : pA;
                        const uint32_t al = p & ~3u, sh = (p & 2u) * 8u;
                        auto field8 = [&](uint32_t off, uint32_t& w0, uint32_t& w1) {     // 8 bytes at block offset `off`
                            const uint32_t x0 = ms_lds32(al + off), x1 = ms_lds32(al + off + 4), x2 = ms_lds32(al + off + 8);
                            w0 = __funnelshift_r(x0, x1, sh); w1 = __funnelshift_r(x1, x2, sh);
                        };
                        uint32_t la0, la1, lb0, lb1, h0, h1;
                        field8(64 * n + 8 * c, la0, la1);            // ql[64n + l]:      quarters 0 (low nibble) and 2 (high)
                        field8(64 * n + 32 + 8 * c, lb0, lb1);       // ql[64n + 32 + l]: quarters 1 and 3
                        field8(128 + 32 * n + 8 * c, h0, h1);        // qh[32n + l]: bit pairs of the four quarters
                        // scales 8n + 2*quarter + (l >= 16): one int8 per quarter for this lane
                        const float d = h2f_bits(ms_lds32((p + 208) & ~3u) >> (((p + 208) & 2u) * 8u));
                        #pragma unroll
                        for (int qq = 0; qq < 2; ++qq) {
                            const int qt = qt0 + qq;
                            const uint32_t sa = p + 192 + 8 * n + 2 * qt + (c >> 1);
                            const int sc = (int)(int8_t)((ms_lds32(sa & ~3u) >> ((sa & 3u) * 8u)) & 0xFFu);
                            const float ds = __fmul_rn(d, (float)sc);
                            const __half hs = __float2half_rn(ds);
                            const __half2 shi = __half2half2(hs), slo = __half2half2(__float2half_rn(ds - __half2float(hs)));
                            const uint32_t L0 = (((qt & 1) ? lb0 : la0) >> (4 * (qt >> 1))) & 0x0F0F0F0Fu;
                            const uint32_t L1 = (((qt & 1) ? lb1 : la1) >> (4 * (qt >> 1))) & 0x0F0F0F0Fu;
                            const uint32_t q0 = L0 | (((h0 >> (2 * qt)) & 0x03030303u) << 4), q1 = L1 | (((h1 >> (2 * qt)) & 0x03030303u) << 4);
                            ms_codes4_split(q0, k1056, shi, slo, frag[qq][0][rs], frag[qq][0][2 + rs]);
                            ms_codes4_split(q1, k1056, shi, slo, frag[qq][1][rs], frag[qq][1][2 + rs]);
                        }
                    }
                    #pragma unroll
                    for (int qq = 0; qq < 2; ++qq) {
                        const int j = 4 * n + qt0 + qq;
                        uint4 b[NT];
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) b[t] = ms_lds128(xq + (uint32_t)t * 8u * MS_XROWB + (uint32_t)j * 64u);
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) ms_mma_f16(acc[t], frag[qq][0], b[t].x, b[t].y);
                        #pragma unroll
                        for (int t = 0; t < NT; ++t) ms_mma_f16(acc[t], frag[qq][1], b[t].z, b[t].w);
                    }
                }
            }
        }
        __syncthreads();                                 // every warp is done with this stage
        if (i + a.nstage < nk) issue(i + a.nstage);
    }
    if (timed_out && lane == 0) atomicExch(a.status, JB_ERR_TIMEOUT);
    // The four warps of a row group hold partial sums over their quarters of K: warps 1..3 leave theirs in shared memory (the
    // stages are free: the loop ended with a CTA barrier), warp 0 adds them in the order 0, 1, 2, 3 and stores.
    float* red = reinterpret_cast<float*>(smem);             // [row group][ks - 1][NT * 4][32 lanes]
    if (warp_live && ks > 0) {
        float* dst = red + ((size_t)(rgi * 3 + ks - 1) * NT * 4) * 32 + lane;
        #pragma unroll
        for (int t = 0; t < NT; ++t)
            #pragma unroll
            for (int e = 0; e < 4; ++e) dst[(t * 4 + e) * 32] = acc[t][e];
    }
    __syncthreads();
    if (!warp_live || ks != 0) return;
    #pragma unroll
    for (int k = 0; k < 3; ++k) {
        const float* src = red + ((size_t)(rgi * 3 + k) * NT * 4) * 32 + lane;
        #pragma unroll
        for (int t = 0; t < NT; ++t)
            #pragma unroll
            for (int e = 0; e < 4; ++e) acc[t][e] += src[(t * 4 + e) * 32];
    }
    // D fragment: rows g / g+8 of the row group, tokens 8t + 2c and 8t + 2c + 1
    #pragma unroll
    for (int t = 0; t < NT; ++t) {
        #pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = row0 + 16 * rgi + g + 8 * (e >> 1), tok = 8 * t + 2 * c + (e & 1);
            if (row < a.M && tok < a.N) {
                if (a.nsplit == 1) {
                    const size_t o = (size_t)tok * a.M + row;
                    const __half pr = __float2half_rn(acc[t][e]);
                    a.y[o] = a.res ? __float2half_rn(__fadd_rn(__half2float(a.res[o]), __half2float(pr))) : pr;
                }
                else a.part[((size_t)blockIdx.y * a.N + tok) * a.M + row] = acc[t][e];
            }
        }
    }
}

__global__ void mms_reduce_kernel(__half* y, const float* part, const __half* res, long long n, int nsplit) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int k = 0; k < nsplit; ++k) s += part[(size_t)k * n + i];      // fixed order: the result does not depend on timing
    const __half pr = __float2half_rn(s);
    y[i] = res ? __float2half_rn(__fadd_rn(__half2float(res[i]), __half2float(pr))) : pr;
}

// ── host side ─────────────────────────────────────────────────────────────
bool mmq_stream_applies(const void* W, int type, int M, int N, int K) {
    static const bool off = [] { const char* e = getenv("JLLM_B200_MMQ_STREAM"); return e && e[0] == '0'; }();
    if (off || N < 2 || N > 64 || M < 16 || K % QK_K) return false;
    // the largest matrices at more than 48 tokens: the tensor-core kernel is faster (64 tokens, Q4_K 9728 x 2560: 29.5 against
    // 36.6 us; Q6_K 2560 x 9728: 30.7 against 35.7 us; equal at 32 tokens, and the smaller matrices stay faster here)
    if (N > 48 && (long long)M * K >= (1ll << 24) && mmq_tc_applies(W, type, M, N, K)) return false;
    if (type == T_Q4K) return ((uintptr_t)W & 15) == 0;
    return type == T_Q6K && ((uintptr_t)W & 1) == 0;
}

struct MsShape { int rg, nsplit, bps, nstage; size_t smem; };

static MsShape ms_shape(int type, int M, int NP, int nb, int sm_count, size_t smem_max) {
    const int wslot = type == T_Q4K ? MS_W4SLOT : MS_W6SLOT;
    MsShape best = {}; double best_cost = 1e30;
    for (int rg = MS_MAXRG; rg >= 1; --rg) {
        const size_t stage = (size_t)NP * MS_XROWB + (size_t)16 * rg * wslot;
        int nstage = (int)((smem_max - 1024) / stage);
        if (nstage < 2) continue;
        if (nstage > 4) nstage = 4;
        const size_t red_bytes = (size_t)rg * 3 * (NP / 8) * 4 * 32 * sizeof(float);      // partial sums of the k-slice warps
        if (red_bytes > stage * nstage) continue;
        const int tiles = (M + 16 * rg - 1) / (16 * rg);
        for (int ns = 1; ns <= nb && ns <= 32; ++ns) {
            const int bps = (nb + ns - 1) / ns;
            if ((nb + bps - 1) / bps != ns) continue;
            const long long ctas = (long long)tiles * ns;
            // time ~ (CTAs an SM runs one after the other) x (super-blocks of a CTA + pipeline fill) x (its row groups + a share
            // for the activation chunk every CTA fetches per super-block); partial sums cost a second pass over N x M floats
            const long long per_sm = (ctas + sm_count - 1) / sm_count;
            const double cost = (double)per_sm * (bps + 1.5) * (rg + 0.5) + (ns > 1 ? 2.0 + 0.5 * ns : 0.0);
            if (cost < best_cost - 1e-9) { best_cost = cost; best = { rg, ns, bps, nstage, stage * nstage + 256 }; }
        }
    }
    return best;
}

static int ms_tiles(int N) { return N <= 8 ? 1 : (N <= 16 ? 2 : (N <= 32 ? 4 : 8)); }     // 8-token MMA tiles the kernel is built for

size_t mmq_stream_scratch_bytes(int type, int M, int N, int K) {
    (void)type;
    const int NPk = 8 * ms_tiles(N), nb = K / QK_K;
    return (((size_t)nb * NPk * MS_XROWB + 255) & ~(size_t)255) + (size_t)32 * N * M * sizeof(float);   // operand + partials of up to 32 K ranges
}

// `residual` (optional, [N][M]): the residual exit of a layer fused in (add_half arithmetic: the product is rounded to fp16
// first).  `reuse_operand`: the caller multiplies the SAME activations by another matrix of the same weight type right after
// the previous call on this stream (Q and K, gate and up): the quantised operand in `scratch` is still valid and the quantise
// launch is skipped; the library checks pointer, shape, flavour and scratch address and quantises again if anything differs.
int launch_mmq_stream(__half* y, const void* W, int type, const __half* x, void* scratch, int M, int N, int K, const __half* residual,
                      bool reuse_operand, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    const int nb = K / QK_K, NT = ms_tiles(N);
    const int NPk = NT * 8;                               // tokens the kernel multiplies (padded ones are zero columns)
    __half* xb = reinterpret_cast<__half*>(scratch);
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + (((size_t)nb * NPk * MS_XROWB + 255) & ~(size_t)255));
    const MsShape sh = ms_shape(type, M, NPk, nb, cx->sm_count, (size_t)cx->max_smem_optin);
    if (!sh.rg) return set_error(JB_ERR_LIMIT, "batched gemm: no launch shape for N=%d", N);
    const long long groups = (long long)NPk * (K / 32);
    const int ds4 = type == T_Q4K;
    const bool same = reuse_operand && cx->mms_op_x == (const void*)x && cx->mms_op_scratch == scratch && cx->mms_op_n == N && cx->mms_op_k == K &&
                      cx->mms_op_ds4 == ds4 && cx->mms_op_stream == (void*)st;
    if (!same) {
        JB_CUDA(launch_k(mms_quantize_kernel, dim3((unsigned)((groups + 3) / 4)), dim3(32, 4), 0, st, pdl_enabled(), x, xb, N, NPk, K, ds4));
        count_launch();
        cx->mms_op_x = x; cx->mms_op_scratch = scratch; cx->mms_op_n = N; cx->mms_op_k = K; cx->mms_op_ds4 = ds4; cx->mms_op_stream = (void*)st;
    }
    MsArgs a = {};
    a.y = y; a.part = part; a.res = residual; a.W = (const uint8_t*)W; a.xb = xb; a.M = M; a.N = N; a.NP = NPk; a.K = K; a.nb = nb;
    a.rg = sh.rg; a.nsplit = sh.nsplit; a.blocks_per_split = sh.bps; a.nstage = sh.nstage; a.status = cx->d_status;
    void (*kern)(MsArgs);
    #define MS_PICK(T) (NT == 1 ? mms_kernel<T, 1> : (NT == 2 ? mms_kernel<T, 2> : (NT == 4 ? mms_kernel<T, 4> : mms_kernel<T, 8>)))
    kern = type == T_Q4K ? MS_PICK(T_Q4K) : MS_PICK(T_Q6K);
    #undef MS_PICK
    const int ki = (type == T_Q4K ? 0 : 4) + (NT == 1 ? 0 : (NT == 2 ? 1 : (NT == 4 ? 2 : 3)));
    if (!cx->mms_attr[ki]) {
        JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cx->max_smem_optin - 1024));
        cx->mms_attr[ki] = true;
    }
    const int tiles = (M + 16 * sh.rg - 1) / (16 * sh.rg);
    static const bool verbose = getenv("JLLM_B200_MMQ_DEBUG") != nullptr;
    if (verbose) fprintf(stderr, "[mmq_stream] type %d M=%d N=%d K=%d: %d x %d CTAs of %d row groups, %d blocks per CTA, %d stages, smem %zu\n",
                         type, M, N, K, tiles, sh.nsplit, sh.rg, sh.bps, sh.nstage, sh.smem);
    JB_CUDA(launch_k(kern, dim3(tiles, sh.nsplit), dim3(sh.rg * MS_KS * 32), sh.smem, st, pdl_enabled(), a));
    count_launch();
    if (sh.nsplit > 1) {
        const long long n = (long long)N * M;
        JB_CUDA(launch_k(mms_reduce_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, pdl_enabled(), y, (const float*)part, residual, n, sh.nsplit));
        count_launch();
    }
    return JB_OK;
}

}  // namespace jb
