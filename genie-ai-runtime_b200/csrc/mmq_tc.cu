// mmq_tc.cu — batched K-quant GEMM (prefill) on the 5th-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, the activation operand staged by TMA, for sm_100a.
//
// Replaces the reference's default prefill path (gemm_quant_batched -> mul_mat_q_llama, src/kernels/gemv_q4.cu:2478-2495,
// mmq_q4k_llama.cu:408-512).  The reference multiplies int8 codes per 32-element sub-block and rescales every
// partial sum on the CUDA cores (sum += dmA.x*dsB.x*C + dmA.y*dsB.y, mmq_q4k_llama.cu:321-322): on B200 that
// epilogue, not the tensor pipe, would set the speed, because scales change every 32 elements.  Here the same
// numbers are produced by ONE accumulation over the whole K range:
//     y[t][r] = Σ_k  half(dA[r,sb(k)] * (q4[r,k]-8)) * half(d8[t,sb(k)] * q8[t,k])
//             + Σ_sb half(-dmin*m)[r,sb] * half(Σx)[t,sb]  +  Σ_sb (8*dA[r,sb]) * half(d8*Σq8)[t,sb]
// i.e. an fp16 x fp16 -> fp32 GEMM over K + 2K/32 columns whose A operand is dequantised on the fly from the GGUF
// blocks with the reference's own half-precision scale products (mmq_q4k_llama.cu:159-163) and whose B operand is
// the reference's quantised activation (codes x scale, and the per-group sums of the DS4 layout, :383-404).
// The only difference from the reference's arithmetic is the rounding of the two operand products to fp16
// (2^-11 relative each, independent from term to term); the codes are centred (q4-8) so that this rounding acts on
// zero-mean values and does not grow with the cancellation between the scale and the min terms.
//
// Shape of the kernel: one persistent CTA per SM; output tile 128 (rows) x 256 (tokens), K tiles of 64, four
// operand stages, two accumulators in tensor memory; 14 warps:
//   warp 0      TMA producer of the activation tile (cp.async.bulk.tensor.2d, 128-byte swizzle)
//   warp 1      issues tcgen05.mma (one elected lane), commits stages back to the producers
//   warps 2-9   dequantise the weight tile (two threads per row) into the 128-byte-swizzled K-major layout
//   warps 10-13 drain the finished accumulator (tcgen05.ld) and store fp16 results token-major while the
//               other accumulator is being filled.
// The grid walks a list of work: whole output tiles first (a multiple of the grid), then the leftover tiles cut into K
// ranges that fill one more short round (fp32 partials, summed by a second kernel); the row tiles of a second weight
// matrix over the same activations (gate and up) can follow the first's in the same list.
// Every mbarrier wait is bounded; a wait that runs out sets the device status word, the kernel still frees
// its tensor memory and returns.
#include "mmq.cuh"
#include <cuda.h>
#include <type_traits>
#include <cstdlib>

namespace jb {

constexpr int TC_M = 128, TC_N = 256, TC_K = 64, TC_STAGES = 4;
constexpr int TC_A_BYTES = TC_M * TC_K * 2;       // 16 KB
constexpr int TC_B_BYTES = TC_N * TC_K * 2;       // 32 KB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024;    // + alignment slack
constexpr int TC_PRODUCERS = 256;      // two dequantising threads per weight row
constexpr int TC_THREADS = 64 + TC_PRODUCERS + 128;   // TMA warp, MMA warp, 8 dequantising warps, 4 draining warps
constexpr uint32_t TC_WAIT_LIMIT = 1u << 24;

struct TcArgs {
    __half* y; const uint8_t* W; int type; int M, N, K;
    __half* y2; const uint8_t* W2; int M2;   // optional second weight matrix of the same type and K over the same activations (its own output): row tiles after the first's
    int n_main, n_min;        // K tiles of weights, K tiles of the min and centring terms (Q4_K)
    int* status;
    int n_full, ksplit;       // output tiles [0, n_full) are computed whole; each later one ("tail" tile) as `ksplit` K ranges whose
    float* part;              // fp32 partials [ksplit][tail tile][token of the tile][128 rows] a second kernel sums
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait without a sleep between polls: in this kernel every wait sits on the critical path between the
// tensor pipe and the warps that feed it, and a sleeping warp wakes up far later than the barrier flips.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t ok;
#ifdef JB_TC_SPIN
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
#else
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
#endif
        if (ok) return true;
        if ((i & 1023u) == 1023u) {           // a poll may block for a hardware-defined interval: bound the wait in time as well
            const unsigned long long t = global_ns();
            if (!t0) t0 = t; else if (t - t0 > 2000000000ull) return false;
        }
    }
    return false;
}
__device__ __forceinline__ void tc_fail(volatile int* fail, int* status) { *fail = 1; atomicExch(status, JB_ERR_TIMEOUT); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// K-major operand tile, 128-byte rows, 128-byte swizzle, 8-row atoms 1024 bytes apart
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 bytes = 8 fp16 weights of row `rl` written at K-chunk `c` (0..7) of a swizzled 128-byte row
__device__ __forceinline__ void tc_store_chunk(uint8_t* a_tile, int rl, int c, uint4 v) {
    *reinterpret_cast<uint4*>(a_tile + rl * 128 + ((c ^ (rl & 7)) << 4)) = v;
}
// four nibbles (already masked to 0x0F0F0F0F) -> four halves (q - 8) * dA, as two half2 words.  The codes are
// centred so that the fp16 rounding of the products acts on values of half the magnitude and zero mean; the
// constant 8 * dA comes back through an extra K column per sub-block (see tc_dequant_q4k_extra).
__device__ __forceinline__ void tc_nib4(uint32_t n4, __half2 dA, uint32_t& lo, uint32_t& hi) {
    const __half2 k1024 = __half2half2(__ushort_as_half((unsigned short)0x6408));    // 1024 + 8
    const uint32_t a = __byte_perm(n4, 0x64646464u, 0x4140), b = __byte_perm(n4, 0x64646464u, 0x4342);      // 0x6400 | q = the half 1024 + q
    const __half2 ha = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&a), k1024), dA);
    const __half2 hb = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&b), k1024), dA);
    lo = *reinterpret_cast<const uint32_t*>(&ha); hi = *reinterpret_cast<const uint32_t*>(&hb);
}

// Two threads share a weight row: thread `h` (0/1) of a row owns bytes 16h..16h+15 of every 32-byte run of
// packed codes, i.e. elements 16h..16h+15 of each 32-element sub-block or quarter.  Raw bytes are fetched one
// whole group of K tiles ahead (Q4_K: a block = 4 tiles; Q6_K: half a block = 2 tiles), so the global-load
// latency overlaps the dequantisation of the group before.
struct RawQ4 { uint4 hdr; uint4 q[4]; };                     // header + this thread's 16 bytes of each tile
struct RawQ6 { uint32_t ql[2][5], qh[5], sc[3], d; };        // aligned words around this thread's bytes

__device__ __forceinline__ void tc_load_q4k(RawQ4& r, const uint8_t* b, int h) {
    r.hdr = __ldg(reinterpret_cast<const uint4*>(b));
    #pragma unroll
    for (int il = 0; il < 4; ++il) r.q[il] = __ldg(reinterpret_cast<const uint4*>(b + 16 + 32 * il + 16 * h));
}
// tile il of the block: low nibbles -> sub-block 2il (tile columns 16h..), high nibbles -> sub-block 2il+1 (32+16h..)
__device__ __forceinline__ void tc_dequant_q4k(uint8_t* a_tile, int rl, const RawQ4& r, int il, int h) {
    int sc0, mn0, sc1, mn1;
    scale_min_k4(2 * il, r.hdr.y, r.hdr.z, r.hdr.w, sc0, mn0);
    scale_min_k4(2 * il + 1, r.hdr.y, r.hdr.z, r.hdr.w, sc1, mn1);
    const __half dh = __ushort_as_half((unsigned short)(r.hdr.x & 0xFFFFu));
    const __half2 dA0 = __half2half2(__hmul(dh, __int2half_rn(sc0)));      // half product, mmq_q4k_llama.cu:159-163
    const __half2 dA1 = __half2half2(__hmul(dh, __int2half_rn(sc1)));
    const uint32_t w[4] = {r.q[il].x, r.q[il].y, r.q[il].z, r.q[il].w};
    #pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint4 lo, hi;
        tc_nib4(w[2 * c] & 0x0F0F0F0Fu, dA0, lo.x, lo.y);
        tc_nib4(w[2 * c + 1] & 0x0F0F0F0Fu, dA0, lo.z, lo.w);
        tc_nib4((w[2 * c] >> 4) & 0x0F0F0F0Fu, dA1, hi.x, hi.y);
        tc_nib4((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, dA1, hi.z, hi.w);
        tc_store_chunk(a_tile, rl, 2 * h + c, lo);
        tc_store_chunk(a_tile, rl, 4 + 2 * h + c, hi);
    }
}

// Q4_K extra K tiles: 8 columns per chunk = the 8 sub-blocks of one block.  Chunks [0, nb) hold the min term
// half(-dmin) * half(m) (multiplied by the per-group sums of x, as in the reference); chunks [nb, 2nb) hold
// 8 * half(d * sc), which multiplied by the per-group sums of the quantised activations restores the centring of
// the codes.  Thread h writes chunks 4h..4h+3 of tile `tm`: the four block headers they are made of are fetched
// together (tc_extra_load), ahead of the wait for the stage, so one L2 latency is exposed per tile at most.
__device__ __forceinline__ void tc_extra_load(uint4 (&hd)[4], const uint8_t* row_blocks, int nb, int tm, int h) {
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int bi = 8 * tm + 4 * h + i;
        hd[i] = make_uint4(0, 0, 0, 0);
        if (row_blocks && bi < 2 * nb) hd[i] = __ldg(reinterpret_cast<const uint4*>(row_blocks + (size_t)(bi >= nb ? bi - nb : bi) * Q4K_BYTES));
    }
}
__device__ __forceinline__ void tc_dequant_q4k_extra(uint8_t* a_tile, int rl, const uint4 (&hd)[4], bool have_row, int nb, int tm, int h) {
    const __half eight = __ushort_as_half((unsigned short)0x4800);
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = 4 * h + i, bi = 8 * tm + c;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (have_row && bi < 2 * nb) {
            const bool centre = bi >= nb;
            const __half dh = __ushort_as_half((unsigned short)(hd[i].x & 0xFFFFu));
            const __half mh = __hneg(__ushort_as_half((unsigned short)(hd[i].x >> 16)));
            unsigned short o[8];
            #pragma unroll
            for (int j = 0; j < 8; ++j) {
                int sc, mn; scale_min_k4(j, hd[i].y, hd[i].z, hd[i].w, sc, mn);
                o[j] = __half_as_ushort(centre ? __hmul(eight, __hmul(dh, __int2half_rn(sc))) : __hmul(mh, __int2half_rn(mn)));
            }
            v = make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16));
        }
        tc_store_chunk(a_tile, rl, c, v);
    }
}

// Q6_K: K tile q4 (0..3) of a block = half n = q4>>1, quarters 2kp and 2kp+1 (kp = q4&1): low (kp=0) or high
// (kp=1) nibbles of ql[64n .. 64n+63], bits 4kp..4kp+3 of qh[32n .. 32n+31], scales 8n+4kp .. +3.  Both tiles of a
// half use the same bytes, so one fetch serves two tiles.  Blocks are 210 bytes, hence only 2-byte aligned:
// every field is read as aligned words around it and re-aligned with a funnel shift (all fields of a block share
// its misalignment).  The word past a field is fetched only when the block is misaligned, so nothing beyond the
// block is touched.
__device__ __forceinline__ void tc_load_q6k(RawQ6& r, const uint8_t* b, int n, int h) {
    const bool mis = ((uintptr_t)b & 2) != 0;
    const uint32_t* base = reinterpret_cast<const uint32_t*>((uintptr_t)b & ~(uintptr_t)3);
    #pragma unroll
    for (int qq = 0; qq < 2; ++qq) {
        const uint32_t* pl = base + 16 * n + 8 * qq + 4 * h;
        #pragma unroll
        for (int i = 0; i < 4; ++i) r.ql[qq][i] = __ldg(pl + i);
        r.ql[qq][4] = mis ? __ldg(pl + 4) : 0u;
    }
    const uint32_t* ph = base + 32 + 8 * n + 4 * h;
    #pragma unroll
    for (int i = 0; i < 4; ++i) r.qh[i] = __ldg(ph + i);
    r.qh[4] = mis ? __ldg(ph + 4) : 0u;
    const uint32_t* ps = base + 48 + 2 * n;
    r.sc[0] = __ldg(ps); r.sc[1] = __ldg(ps + 1); r.sc[2] = mis ? __ldg(ps + 2) : 0u;
    r.d = __ldg(reinterpret_cast<const unsigned short*>(b + 208));
}
// Values d*sc*(q-32) are formed as q * hi + q * lo with (hi, lo) the fp16 split of the fp32 product d*sc,
// so each weight is rounded to fp16 once.
__device__ __forceinline__ void tc_dequant_q6k(uint8_t* a_tile, int rl, const RawQ6& r, int kp, int h, uint32_t sh) {
    const float d = h2f_bits(r.d);
    const uint32_t s0 = __funnelshift_r(r.sc[0], r.sc[1], sh), s1 = __funnelshift_r(r.sc[1], r.sc[2], sh);
    const uint32_t sc4 = kp ? s1 : s0;                     // scales 8n+4kp .. +3; this thread uses 2qq + h
    const __half2 k1056 = __half2half2(__ushort_as_half((unsigned short)0x6420));   // 1024 + 32
    #pragma unroll
    for (int qq = 0; qq < 2; ++qq) {           // quarter 2kp + qq: tile columns 32qq + 16h .. +15
        const float ds = __fmul_rn(d, (float)(int)(int8_t)((sc4 >> (8 * (2 * qq + h))) & 0xFF));
        const __half hs = __float2half_rn(ds);
        const __half2 shi = __half2half2(hs), slo = __half2half2(__float2half_rn(ds - __half2float(hs)));
        #pragma unroll
        for (int c = 0; c < 2; ++c) {          // chunk of 8 elements = two ql words
            uint32_t out[4];
            #pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int wi = 2 * c + e;
                const uint32_t L = (__funnelshift_r(r.ql[qq][wi], r.ql[qq][wi + 1], sh) >> (4 * kp)) & 0x0F0F0F0Fu;
                const uint32_t H = __funnelshift_r(r.qh[wi], r.qh[wi + 1], sh) >> (4 * kp + 2 * qq);
                const uint32_t q6 = L | ((H & 0x03030303u) << 4);
                const uint32_t a = __byte_perm(q6, 0x64646464u, 0x4140), bb = __byte_perm(q6, 0x64646464u, 0x4342);
                const __half2 qa = __hsub2(*reinterpret_cast<const __half2*>(&a), k1056);
                const __half2 qb = __hsub2(*reinterpret_cast<const __half2*>(&bb), k1056);
                const __half2 ra = __hfma2(qa, shi, __hmul2(qa, slo));
                const __half2 rb = __hfma2(qb, shi, __hmul2(qb, slo));
                out[2 * e] = *reinterpret_cast<const uint32_t*>(&ra);
                out[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&rb);
            }
            tc_store_chunk(a_tile, rl, 4 * qq + 2 * h + c, make_uint4(out[0], out[1], out[2], out[3]));
        }
    }
}

// activation operand: X'[t][0..K) = half(d*q) (codes x scale of the reference's quantiser, mmq_q4k_llama.cu:383-404,
// mmq_q6k_llama.cu:424-438); for Q4_K also X'[t][K + g] = half(sum of x over group g) (the reference's DS4 sum)
// and X'[t][K + K/32 + g] = half(d * sum of codes of group g); zero up to the padded width Kp.
__global__ void mmq_tc_quantize1_kernel(const __half* x, __half* xq, int N, int K, int Kp, int ds4) {
    pdl_wait();
    const long long g = (long long)blockIdx.x * blockDim.y + threadIdx.y;
    const int lane = threadIdx.x, G = K / 32;
    if (g >= (long long)N * G) return;
    const long long t = g / G; const int gi = (int)(g - t * G);
    const float v = __half2float(x[g * 32 + lane]);
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
    __half* row = xq + t * Kp;
    row[gi * 32 + lane] = __float2half_rn(__fmul_rn(d, (float)q));
    if (ds4 && lane == 0) {
        row[K + gi] = __float2half_rn(sum);
        row[K + G + gi] = __float2half_rn(__fmul_rn(d, (float)qsum));
    }
    if (gi == 0) for (int c = K + (ds4 ? 2 * G : 0) + lane; c < Kp; c += 32) row[c] = __float2half_rn(0.f);
}

// The same operand, one warp per (token, super-block of 256): lane 4j + c holds elements 8c..8c+7 of group j, read and
// written as 16 bytes (the form above moves 2 bytes per lane and needs eight times the warps; on a 2048 x 9728 operand it
// took as long as half the product).  The sum of x is taken in the order of the 32-lane xor-shuffle tree of that form
// (partners 16, 8, 4, 2, 1 apart), so both forms, and the CPU restatement of the reference's quantiser, give the same bits.
// Needs x 16-byte aligned.
__global__ void mmq_tc_quantize_kernel(const __half* x, __half* xq, int N, int K, int Kp, int ds4) {
    pdl_wait();
    const long long wi = (long long)blockIdx.x * blockDim.y + threadIdx.y;
    const int lane = threadIdx.x, nsb = K / QK_K, G = K / 32;
    if (wi >= (long long)N * nsb) return;
    const long long t = wi / nsb; const int sb = (int)(wi - t * nsb);
    const int c = lane & 3, gi = sb * 8 + (lane >> 2);
    const uint4 raw = *reinterpret_cast<const uint4*>(x + t * K + (size_t)gi * 32 + 8 * c);
    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8], s[8];
    float amax = 0.f;
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&rw[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    #pragma unroll
    for (int i = 0; i < 8; ++i) { s[i] = v[i] + __shfl_xor_sync(0xFFFFFFFFu, v[i], 2); }       // elements 16 apart
    #pragma unroll
    for (int i = 0; i < 8; ++i) { s[i] = s[i] + __shfl_xor_sync(0xFFFFFFFFu, s[i], 1); }       // 8 apart
    const float sum = __fadd_rn(__fadd_rn(__fadd_rn(s[0], s[4]), __fadd_rn(s[2], s[6])), __fadd_rn(__fadd_rn(s[1], s[5]), __fadd_rn(s[3], s[7])));   // 4, 2, 1 apart
    float d = __fdiv_rn(amax, 127.0f);
    const float dinv = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    int q[8], qsum = 0;
    #pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = __float2int_rn(__fmul_rn(v[i], dinv)); qsum += q[i]; }
    qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, 1);
    qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, 2);
    if (ds4) d = __half2float(__float2half_rn(d));
    uint32_t ow[4];
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 h = __halves2half2(__float2half_rn(__fmul_rn(d, (float)q[2 * i])), __float2half_rn(__fmul_rn(d, (float)q[2 * i + 1])));
        ow[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    __half* row = xq + t * Kp;
    *reinterpret_cast<uint4*>(row + (size_t)gi * 32 + 8 * c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    if (ds4 && c == 0) {
        row[K + gi] = __float2half_rn(sum);
        row[K + G + gi] = __float2half_rn(__fmul_rn(d, (float)qsum));
    }
    if (sb == 0) for (int z = K + (ds4 ? 2 * G : 0) + lane; z < Kp; z += 32) row[z] = __float2half_rn(0.f);
}

// Persistent kernel: one CTA per SM walks output tiles (token tile fastest, so the CTAs running at one time
// share a few weight row tiles and the whole activation panel in L2).  Four operand stages; two accumulators of
// 256 tensor-memory columns each, so the drain of one tile overlaps the K loop of the next.
//
// The thread that issues the MMAs is the scarce resource: it must start a 128x256x16 MMA every 128 cycles, and a
// single thread retires only a few dozen instructions in that time.  So its loop holds one barrier wait per K
// tile (weights and activations complete the same barrier), descriptors formed by one addition, and nothing else;
// and the other warps stay off the shared-memory pipe while they wait: one lane per role polls an mbarrier, the
// rest of the role sleeps in a hardware named barrier.
template <int TYPE>
__global__ void __launch_bounds__(TC_THREADS, 1) mmq_tc_kernel(const __grid_constant__ CUtensorMap xmap, TcArgs a, int n_tile) {
    extern __shared__ uint8_t tc_smem_raw[];
    __shared__ uint64_t full[TC_STAGES], empty[TC_STAGES], acc_full[2], acc_empty[2], drain_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int fail;
    __shared__ volatile int drain_go[2];     // verdict of the draining role's polling lane, double-buffered across tiles
    uint8_t* smem = tc_smem_raw + ((1024u - (smem_u32(tc_smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (a.N + n_tile - 1) / n_tile, tiles_m1 = (a.M + TC_M - 1) / TC_M, tiles_m = tiles_m1 + (a.M2 + TC_M - 1) / TC_M;
    const int n_tail = tiles_n * tiles_m - a.n_full;
    const int n_work = a.n_full + n_tail * a.ksplit;
    const int n_tiles = a.n_main + a.n_min;
    // Work item w = (output tile, K range).  The first n_full items are whole output tiles, a multiple of the grid, so every
    // CTA gets the same number of them; the tiles left over would occupy a fraction of the SMs for a whole tile time, so
    // each is cut into ksplit K ranges that together fill one more, short, round.  A range holds main K tiles [t0, t1)
    // (whole fetch groups), and the last range of a tile the extra tiles.
    constexpr int GTILES = TYPE == T_Q4K ? 4 : 2;
    auto k_range = [&](int w, int& tile, int& sp, int& t0, int& t1, bool& extra) {
        int ks = 1;
        tile = w; sp = 0;
        if (w >= a.n_full) { const int v = w - a.n_full; ks = a.ksplit; tile = a.n_full + v / ks; sp = v - (v / ks) * ks; }
        const int ng = a.n_main / GTILES;
        t0 = (int)((long long)ng * sp / ks) * GTILES;
        t1 = (int)((long long)ng * (sp + 1) / ks) * GTILES;
        extra = sp == ks - 1;
    };
    const uint32_t b_bytes = (uint32_t)n_tile * TC_K * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full[s], TC_PRODUCERS / 32 + 1); mbar_init(&empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        mbar_init(&drain_bar, 1);
        fence_mbar_init();
        fail = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // activation tiles by TMA; the quantised activations are the previous kernel's output
        pdl_wait();
        if (lane == 0) {
            uint32_t it = 0;
            for (int w = blockIdx.x; w < n_work && !fail; w += gridDim.x) {
                int tile, sp, t0, t1; bool extra;
                k_range(w, tile, sp, t0, t1, extra);
                const int n0 = (tile % tiles_n) * n_tile;
                for (int t = t0; t < n_tiles; ++t, ++it) {
                    if (t == t1) { if (!extra) break; t = a.n_main; if (t >= n_tiles) break; }
                    const int s = it % TC_STAGES;
                    if (!tc_wait(&empty[s], ((it / TC_STAGES) & 1) ^ 1) || fail) { tc_fail(&fail, a.status); break; }
                    mbar_expect_tx(&full[s], b_bytes);
                    tma_load_2d(smem + s * TC_STAGE_BYTES + TC_A_BYTES, &xmap, t * TC_K, n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // fp16 x fp16 -> fp32, both operands K-major, M = 128, N = n_tile
            const uint32_t idesc = (1u << 4) | ((uint32_t)(n_tile >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
            const uint64_t ad0 = tc_smem_desc(smem_u32(smem)), bd0 = tc_smem_desc(smem_u32(smem + TC_A_BYTES));
            uint32_t it = 0, j = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x, ++j) {
                const uint32_t d_tmem = tmem + (j & 1) * 256u;
                if (!tc_wait(&acc_empty[j & 1], ((j >> 1) & 1) ^ 1)) { ok = false; break; }
                tc_fence_after();
                int tile, sp, t0, t1; bool extra;
                k_range(w, tile, sp, t0, t1, extra);
                const int count = (t1 - t0) + (extra ? a.n_min : 0);
                for (int t = 0; t < count; ++t, ++it) {
                    const uint32_t s = it % TC_STAGES;
                    if (!tc_wait(&full[s], (it / TC_STAGES) & 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t ad = ad0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4)), bd = bd0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4));
                    tc_mma_f16(d_tmem, ad, bd, idesc, (uint32_t)(t != 0));
                    tc_mma_f16(d_tmem, ad + 2, bd + 2, idesc, 1u);
                    tc_mma_f16(d_tmem, ad + 4, bd + 4, idesc, 1u);
                    tc_mma_f16(d_tmem, ad + 6, bd + 6, idesc, 1u);
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[j & 1]);
            }
            if (!ok) tc_fail(&fail, a.status);
            // nothing of this CTA may still be running on the tensor pipe when the columns are freed
            tc_commit(&drain_bar);
            tc_wait(&drain_bar, 0);
        }
    } else if (warp < 2 + TC_PRODUCERS / 32) {
        // weight tiles: thread (rl, h) dequantises its half of row rl of every K tile
        const int pw = warp - 2, rl = (pw & 3) * 32 + lane, h = pw >> 2;
        const int nb = a.K / QK_K;
        constexpr int BB = TYPE == T_Q4K ? Q4K_BYTES : Q6K_BYTES;
        constexpr int GT = GTILES;                              // K tiles per fetched group
        typename std::conditional<TYPE == T_Q4K, RawQ4, RawQ6>::type cur, nxt;
        uint32_t it = 0;
        bool ok = true;
        // stage s is free again: every producer thread watches the mbarrier itself (an extra hop through one polling
        // lane and a named barrier measured slower: the wake-up latency sits on the critical path)
        auto stage_free = [&](uint32_t it_) -> bool {
            return tc_wait(&empty[it_ % TC_STAGES], ((it_ / TC_STAGES) & 1) ^ 1) && !fail;
        };
        auto stage_done = [&](uint32_t it_) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[it_ % TC_STAGES]);
        };
        for (int w = blockIdx.x; w < n_work && ok; w += gridDim.x) {
            int tile, sp, kt0, kt1; bool extra;
            k_range(w, tile, sp, kt0, kt1, extra);
            const int rt = tile / tiles_n;
            const bool second = rt >= tiles_m1;
            const int row = (second ? rt - tiles_m1 : rt) * TC_M + rl;
            const uint8_t* rowp = row < (second ? a.M2 : a.M) ? (second ? a.W2 : a.W) + (size_t)row * nb * BB : nullptr;
            const int g_first = kt0 / GT, g_last = kt1 / GT;
            auto fetch = [&](decltype(cur)& r, int g) {
                if (!rowp || g >= g_last) return;
                if constexpr (TYPE == T_Q4K) tc_load_q4k(r, rowp + (size_t)g * Q4K_BYTES, h);
                else                         tc_load_q6k(r, rowp + (size_t)(g >> 1) * Q6K_BYTES, g & 1, h);
            };
            fetch(cur, g_first);
            int t = kt0;
            for (int g = g_first; g < g_last && ok; ++g) {
                fetch(nxt, g + 1);
                #pragma unroll
                for (int u = 0; u < GT; ++u, ++t, ++it) {
                    if (!stage_free(it)) { ok = false; break; }
                    uint8_t* at = smem + (it % TC_STAGES) * TC_STAGE_BYTES;
                    if (!rowp) {
                        #pragma unroll
                        for (int c = 0; c < 4; ++c) tc_store_chunk(at, rl, (c & 1) + 2 * h + 4 * (c >> 1), make_uint4(0, 0, 0, 0));
                    } else if constexpr (TYPE == T_Q4K) {
                        tc_dequant_q4k(at, rl, cur, u, h);
                    } else {
                        tc_dequant_q6k(at, rl, cur, u, h, (uint32_t)(((uintptr_t)(rowp + (size_t)(g >> 1) * Q6K_BYTES)) & 2) * 8);
                    }
                    stage_done(it);
                }
                cur = nxt;
            }
            if constexpr (TYPE == T_Q4K) {                               // the min-term and centring tiles
                uint4 xh[4];
                if (extra && a.n_main < n_tiles && ok) tc_extra_load(xh, rowp, nb, 0, h);
                for (t = a.n_main; extra && t < n_tiles && ok; ++t, ++it) {
                    if (!stage_free(it)) { ok = false; break; }
                    tc_dequant_q4k_extra(smem + (it % TC_STAGES) * TC_STAGE_BYTES, rl, xh, rowp != nullptr, nb, t - a.n_main, h);
                    if (t + 1 < n_tiles) tc_extra_load(xh, rowp, nb, t + 1 - a.n_main, h);      // the next one, in flight across the hand-over
                    stage_done(it);
                }
            }
        }
        if (!ok) tc_fail(&fail, a.status);
    } else {
        // drain: warp e owns TMEM lanes 32*(warp%4) .. +31 = tile rows; results go out token-major as fp16.
        // Other kernels may still read or write y until the previous kernel in the stream has finished.
        pdl_wait();
        const int rl = (warp & 3) * 32 + lane, dw = warp - 2 - TC_PRODUCERS / 32;
        uint32_t j = 0;
        for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++j) {
            const uint32_t acc = j & 1;
            int tile, sp, t0_, t1_; bool extra_;
            k_range(w, tile, sp, t0_, t1_, extra_);
            const int rt = tile / tiles_n;
            const bool second = rt >= tiles_m1;
            const int n0 = (tile % tiles_n) * n_tile, row = (second ? rt - tiles_m1 : rt) * TC_M + rl, m_out = second ? a.M2 : a.M;
            __half* y_out = second ? a.y2 : a.y;
            float* part = w >= a.n_full ? a.part + ((size_t)sp * n_tail + (size_t)(tile - a.n_full)) * n_tile * TC_M : nullptr;
            if (dw == 0 && lane == 0) {
                const bool good = tc_wait(&acc_full[acc], (j >> 1) & 1) && !fail;
                if (!good) tc_fail(&fail, a.status);
                drain_go[j & 1] = good;
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (!drain_go[j & 1]) break;
            tc_fence_after();
            for (int cb = 0; cb < n_tile; cb += 32) {
                uint32_t r[32];
                tc_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + acc * 256u + (uint32_t)cb, r);
                if (row < m_out) {
                    #pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int tok = n0 + cb + c;
                        if (tok < a.N) {
                            if (part) part[(size_t)(cb + c) * TC_M + rl] = __uint_as_float(r[c]);
                            else y_out[(size_t)tok * m_out + row] = __float2half_rn(__uint_as_float(r[c]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// sum of the K-range partials of the tail tiles in a fixed order, rounded once to fp16; a thread takes four consecutive rows
// of one token (16-byte loads; the rows of a tile start at a multiple of 128, so with M a multiple of 4 a group of four
// is inside the tensor or outside it as a whole)
__global__ void mmq_tc_reduce_kernel(__half* y, __half* y2, const float* part, int M, int M2, int N, int n_tile, int tiles_n, int n_full, int n_tail, int ksplit) {
    pdl_wait();
    const long long total = (long long)n_tail * n_tile * TC_M;
    const long long e = 4 * ((long long)blockIdx.x * blockDim.x + threadIdx.x);
    if (e >= total) return;
    const int rl = (int)(e % TC_M), tl = (int)((e / TC_M) % n_tile), tile = n_full + (int)(e / ((long long)TC_M * n_tile));
    int rt = tile / tiles_n;
    const int tiles_m1 = (M + TC_M - 1) / TC_M, tok = (tile % tiles_n) * n_tile + tl;
    if (rt >= tiles_m1) { rt -= tiles_m1; y = y2; M = M2; }          // a tile of the second matrix
    const int row = rt * TC_M + rl;
    if (row >= M || tok >= N) return;
    float4 sum = *reinterpret_cast<const float4*>(part + e);
    for (int k = 1; k < ksplit; ++k) {
        const float4 v = *reinterpret_cast<const float4*>(part + (long long)k * total + e);
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    __half* dst = y + (size_t)tok * M + row;
    if ((M & 3) == 0 && ((uintptr_t)y & 7) == 0) {
        const __half2 lo = __floats2half2_rn(sum.x, sum.y), hi = __floats2half2_rn(sum.z, sum.w);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        const float v[4] = {sum.x, sum.y, sum.z, sum.w};
        for (int i = 0; i < 4 && row + i < M; ++i) dst[i] = __float2half_rn(v[i]);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

// Token-tile width, the number of whole output tiles and the K ranges of each remaining ("tail") tile, chosen together.
// The whole tiles are the largest multiple of the grid; the tail is cut into as many K ranges as fill the grid once more
// (every range keeps at least eight K tiles, and its partial sums cost a tile of fp32 traffic each way).  Cost of a
// choice, in tile times of the full width = (whole rounds + 1 / ranges + a little per range) x (tile width / 256,
// floored at 0.65 for the MMA-issue and dequantisation floor of a K tile).
static void tc_pick(int tiles_m, int N, int n_main_tiles, int sm_count, int& n_tile, int& ksplit, int& n_full) {
    float best = 1e30f;
    n_tile = 256; ksplit = 1; n_full = tiles_m * ((N + 255) / 256);
    for (int cand = 256; cand >= 32; cand >>= 1) {
        if (cand < 256 && cand >= 2 * N) continue;
        const int tiles = tiles_m * ((N + cand - 1) / cand);
        const float w = cand / 256.f, wt = w > 0.65f ? w : 0.65f;
        const int rounds = tiles / sm_count, tail = tiles - rounds * sm_count;
        int ks = 1;
        if (tail > 0) {
            ks = sm_count / tail;
            if (ks > n_main_tiles / 8) ks = n_main_tiles / 8;
            if (ks > 16) ks = 16;
            if (ks < 1) ks = 1;
        }
        const float cost = tail == 0 ? rounds * wt : (rounds + 1.0f / ks + (ks > 1 ? 0.04f + 0.01f * ks : 0.f)) * wt;
        if (cost < best - 1e-6f) { best = cost; n_tile = cand; ksplit = ks; n_full = ks > 1 ? rounds * sm_count : tiles; }
    }
}
size_t mmq_tc_scratch_bytes(int type, int M, int N, int K) { return mmq_tc_scratch_bytes_pair(type, M, 0, N, K); }
size_t mmq_tc_scratch_bytes_pair(int type, int M, int M2, int N, int K) {
    DeviceCtx* c = ctx();
    const int sm = c ? c->sm_count : 148;
    const int n_min = type == T_Q4K ? (2 * (K / 32) + TC_K - 1) / TC_K : 0;
    size_t b = (((size_t)N * (size_t)(K + n_min * TC_K) * sizeof(__half)) + 255) & ~(size_t)255;
    int n_tile, ks, n_full;
    const int tiles_m = (M + TC_M - 1) / TC_M + (M2 + TC_M - 1) / TC_M;
    tc_pick(tiles_m, N, K / TC_K, sm, n_tile, ks, n_full);
    const int tiles = ((N + n_tile - 1) / n_tile) * tiles_m;
    if (ks > 1) b += (size_t)ks * (size_t)(tiles - n_full) * n_tile * TC_M * sizeof(float);
    return b + 256;
}

bool mmq_tc_applies(const void* W, int type, int M, int N, int K) {
    if (type != T_Q4K && type != T_Q6K) return false;
    if (type == T_Q4K && ((uintptr_t)W & 15)) return false;      // 16-byte loads of the nibble words
    if (type == T_Q6K && ((uintptr_t)W & 1)) return false;
    return N >= 2 && M >= 1 && K % QK_K == 0 && encode_tiled_fn() != nullptr;
}

int launch_mmq_tc(__half* y, const void* W, int type, const __half* x, __half* xq, int M, int N, int K, bool same_x, cudaStream_t st) {
    return launch_mmq_tc_pair(y, nullptr, W, nullptr, type, x, xq, M, 0, N, K, same_x, st);
}
// y = x . W^T and, when W2 is given, y2 = x . W2^T in the same launch: the row tiles of both matrices are one list of work, so
// two products that share their activations (gate and up) fill the grid together instead of one after the other.
int launch_mmq_tc_pair(__half* y, __half* y2, const void* W, const void* W2, int type, const __half* x, __half* xq, int M, int M2, int N, int K,
                       bool same_x, cudaStream_t st) {
    DeviceCtx* c = ctx();
    if (!c) return set_error(JB_ERR_STATE, "batched gemm: library not initialised");
    TcArgs a;
    a.y = y; a.W = (const uint8_t*)W; a.type = type; a.M = M; a.N = N; a.K = K;
    a.y2 = y2; a.W2 = (const uint8_t*)W2; a.M2 = W2 ? M2 : 0;
    a.n_main = K / TC_K;
    a.n_min = type == T_Q4K ? (2 * (K / 32) + TC_K - 1) / TC_K : 0;
    a.status = c->d_status;
    const int Kp = (a.n_main + a.n_min) * TC_K;
    int n_tile;
    const int tiles_m = (M + TC_M - 1) / TC_M + (a.M2 + TC_M - 1) / TC_M;
    tc_pick(tiles_m, N, a.n_main, c->sm_count, n_tile, a.ksplit, a.n_full);
    const int tiles_n = (N + n_tile - 1) / n_tile, tiles = tiles_n * tiles_m;
    a.part = a.ksplit > 1 ? reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xq) + ((((size_t)N * Kp * sizeof(__half)) + 255) & ~(size_t)255)) : nullptr;

    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)Kp, (cuuint64_t)N};
    const cuuint64_t gstr[1] = {(cuuint64_t)Kp * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)TC_K, (cuuint32_t)n_tile};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xq, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(JB_ERR_CUDA, "batched gemm: tensor map for the activation tile refused (driver code %d)", (int)r);

    static bool attr_done[2] = {false, false};
    const int ti = type == T_Q4K ? 0 : 1;
    if (!attr_done[ti]) {
        if (ti == 0) JB_CUDA(cudaFuncSetAttribute(mmq_tc_kernel<T_Q4K>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
        else         JB_CUDA(cudaFuncSetAttribute(mmq_tc_kernel<T_Q6K>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
        attr_done[ti] = true;
    }
    // The operand of the previous call is still in the scratch when the caller says x has not changed since and everything
    // that shapes it (tokens, K, the Q4_K extras) is the same: the products that share an input quantise it once.
    const int ds4 = (int)(type == T_Q4K);
    const bool reuse = same_x && c->tc_op_x == x && c->tc_op_xq == xq && c->tc_op_stream == (void*)st && c->tc_op_n == N && c->tc_op_k == K && c->tc_op_ds4 == ds4;
    if (!reuse) {
        if (((uintptr_t)x & 15) == 0) {
            const long long warps = (long long)N * (K / QK_K);
            JB_CUDA(launch_k(mmq_tc_quantize_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(32, 4), 0, st, pdl_enabled(), x, xq, N, K, Kp, ds4));
        } else {
            const long long groups = (long long)N * (K / 32);
            JB_CUDA(launch_k(mmq_tc_quantize1_kernel, dim3((unsigned)((groups + 3) / 4)), dim3(32, 4), 0, st, pdl_enabled(), x, xq, N, K, Kp, ds4));
        }
        count_launch();
        c->tc_op_x = x; c->tc_op_xq = xq; c->tc_op_stream = (void*)st; c->tc_op_n = N; c->tc_op_k = K; c->tc_op_ds4 = ds4;
    }
    const int n_work = a.n_full + (tiles - a.n_full) * a.ksplit;
    const dim3 grid(n_work < c->sm_count ? n_work : c->sm_count);
    if (ti == 0) JB_CUDA(launch_k(mmq_tc_kernel<T_Q4K>, grid, dim3(TC_THREADS), TC_SMEM, st, pdl_enabled(), map, a, n_tile));
    else         JB_CUDA(launch_k(mmq_tc_kernel<T_Q6K>, grid, dim3(TC_THREADS), TC_SMEM, st, pdl_enabled(), map, a, n_tile));
    count_launch();
    if (a.ksplit > 1) {
        const int n_tail = tiles - a.n_full;
        const long long n = (long long)n_tail * n_tile * TC_M / 4;
        JB_CUDA(launch_k(mmq_tc_reduce_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, pdl_enabled(), y, y2, (const float*)a.part, M, a.M2, N, n_tile, tiles_n, a.n_full, n_tail, a.ksplit));
        count_launch();
    }
    return JB_OK;
}

}  // namespace jb
