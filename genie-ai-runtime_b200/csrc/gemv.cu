// gemv.cu — streaming K-quant GEMV for B200 (sm_100a).
//
// Replaces the reference's decode GEMV family (src/kernels/gemv_q4.cu:445-683 kernels,
// :1245-1616 dispatch).  The GGUF super-block layout is read unchanged from HBM.
//
// Shape of the kernel
//   * ONE kernel function serves every GEMV entry point, both weight types and both activation formats: the launches of
//     a decode step alternate between as few functions as possible and the code stays small (70 KB), because every launch
//     fetches whatever the instruction cache has lost of it behind its own weight stream.
//   * grid = one or two CTAs per SM, half an SM each (8 warps at 128 registers, 111 KB of shared memory); every CTA owns
//     one contiguous range of row groups of the (up to three) weight matrices, split evenly by bytes.  Consuming warps,
//     rows per task and K chunks of long rows are chosen per launch so that the longest chain of work any warp runs is
//     shortest (gv_configure); further warps of the CTA only help to stage the activations.
//   * weights travel HBM -> shared memory with 1-D TMA bulk copies (cp.async.bulk + mbarrier complete_tx); every
//     warp runs its own ring of slots with one mbarrier per slot, no CTA-wide barrier in the loop; Q6_K rows
//     (210-byte blocks, 2-byte aligned) are copied as the enclosing 16-byte aligned span and re-aligned with funnel
//     shifts when read from shared memory.  Half of every ring is requested before griddepcontrol.wait, the other half
//     right after the loads of the activation vector (requests leave an SM in order).
//   * the activation vector is quantised once per CTA by all its threads (four threads per 32-element group) into shared
//     memory (q8_1 codes, or 16-bit fixed point for the entry points whose reference path keeps fp16 activations),
//     optionally after a fused RMSNorm, laid out so that the 16-byte runs the lanes read are bank-conflict free.
//   * Q4_K: a lane owns one super-block column of three consecutive rows (the activations of the column are read once for
//     the three rows, which are independent instruction streams); Q6_K: a lane owns 64 weights of one row; integer dots
//     with dp4a, rows reduced with shuffles; outputs are deterministic.
//   * launched with programmatic dependent launch (launch_dependents first thing).
//   * the same body runs as one phase of an optional chained launch (gemv_chain_kernel), and an instantiation of its own
//     carries the tensor-parallel hooks: activations polled as {value, epoch} packets, results pushed to every rank.
#include "gemv.cuh"
#include <cstdio>
#include <cstdlib>

namespace jb {

// Stream kernel: a CTA takes HALF an SM.  A product whose share per SM fits one ring launches one CTA per SM, and the other
// half is where the CTAs of the NEXT kernel in the stream become resident as soon as this one has issued
// griddepcontrol.launch_dependents: they set up their barriers and start their bulk copies while this kernel is still
// computing.  A larger product launches two CTAs per SM.
constexpr int GV_MAXWARPS = 8;                 // 8 warps at 128 registers (rows-deep columns keep many values live)
constexpr int GV_CHAINWARPS = 16;              // the chain kernel keeps a whole SM per CTA (its phases overlap inside one launch)
constexpr int GV_CHAINTHREADS = GV_CHAINWARPS * 32;
constexpr int GV_MAXSLOT = 8;
constexpr int GV_NTRACE = 16;                  // time stamps per CTA of a traced launch

struct GvSegDev {
    const uint8_t* W; void* y; int M; int type;
    int rb;          // row bytes
    int U;           // work items per row: 4 per super-block for both types
    int R;           // rows per task ("row group")
    // Q4_K lane map of a task: the warp is cut into `lg` groups of `lw` lanes; lane c of group g owns super-block column
    // c (and c + lw, ... when a row has more than lw blocks) of the `rl` rows g*rl .. g*rl + rl - 1, so R = lg * rl.
    uint8_t lw, lg, rl, pad_;
};
struct GvParams {
    GvSegDev seg[3]; int nseg;
    const __half* x; int K;
    int out_mode; const __half* residual;
    const uint2* residual_pk;   // residual as packets of this rank's own region (tensor-parallel chain), else null
    int do_norm; const void* norm_w; int norm_w_fp32; float eps;
    int32_t* dbg_dots; int* status;
    unsigned long long* trace;  // diagnostic launches only: GV_NTRACE time stamps per CTA
    int trace_nocompute;        // diagnostic: stream the weights but skip the dot products
    int slot_bytes, nslots, needA, needB, paired_rows, nwarps;
    int early_slots;            // slots of every ring whose copies are issued before the wait for the producer kernel
    int nchunk, chunk_blocks;   // a row group is streamed as nchunk tasks of chunk_blocks super-blocks per row (nchunk > 1 only with R = 1)
    uint32_t off_xA, off_xB, off_xd, off_xs, off_xsum, off_gate, off_slots;
    long long total_bytes;      // Σ over segments of (row groups x bytes per group)
    uint32_t gw[3], ng[3];      // per matrix: weight of a row group in the split over CTAs, number of groups
    uint32_t split_q, split_r;  // Σ gw*ng / grid and % grid
    int tp_wait_on, tp_push_on;
    int xmode;                  // 0 q8_1 activations, 1 16-bit activations
    int chained;                // phase of a chain kernel: activations may have been written by other SMs in this launch
    GemvTpWait tpw;
    GemvTpPush tpp;
};

static thread_local unsigned long long* g_trace = nullptr;    // diagnostic: time stamps of the next launch (gemv_set_trace)
void gemv_set_trace(unsigned long long* t) { g_trace = t; }
static thread_local bool g_tp_wait_set = false, g_tp_push_set = false;
static thread_local GemvTpWait g_tp_wait;
static thread_local GemvTpPush g_tp_push;
void gemv_set_tp_hooks(const GemvTpWait* w, const GemvTpPush* q) {
    g_tp_wait_set = w != nullptr; if (w) g_tp_wait = *w;
    g_tp_push_set = q != nullptr; if (q) g_tp_push = *q;
}

// ── activation staging ───────────────────────────────────────────────────
// Eight consecutive activations as floats: a 16-byte load of the plain fp16 vector, or, for a vector that arrives from
// the other ranks, 64 bytes of packets polled (bounded) until every epoch word matches; the packets are read past L1.
template <bool TP>
__device__ __forceinline__ void gv_load8(const GvParams& p, int it, uint32_t epoch, float (&v)[8]) {
    if (!(TP && p.tp_wait_on)) {
        // inside a chain the vector was written earlier in this launch: read it past L1, which may hold older lines
        const uint4 raw = (TP && p.chained) ? __ldcg(reinterpret_cast<const uint4*>(p.x + 8 * it)) : *reinterpret_cast<const uint4*>(p.x + 8 * it);
        const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = a.x; v[2 * i + 1] = a.y;
        }
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(p.x) + 4 * it;
    uint4 q[4];
    PollGuard guard(p.status);
    for (;;) {
        bool ok = true;
        #pragma unroll
        for (int i = 0; i < 4; ++i) { q[i] = __ldcv(src + i); ok = ok && q[i].y == epoch && q[i].w == epoch; }
        if (ok || !guard.again(p.status)) break;
    }
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i]     = __half2float(__ushort_as_half((unsigned short)(q[i].x & 0xFFFFu)));
        v[2 * i + 1] = __half2float(__ushort_as_half((unsigned short)(q[i].z & 0xFFFFu)));
    }
}

// The eight norm weights of staging item `it` (eight consecutive activations).
__device__ __forceinline__ void gv_norm_w8(const GvParams& p, int it, float (&wn)[8]) {
    if (p.norm_w_fp32) {
        #pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float4 w4 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + 8 * it + 4 * h);
            wn[4 * h] = w4.x; wn[4 * h + 1] = w4.y; wn[4 * h + 2] = w4.z; wn[4 * h + 3] = w4.w;
        }
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.norm_w) + 8 * it);
        const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            wn[2 * i] = a.x; wn[2 * i + 1] = a.y;
        }
    }
}

// Sixteen bytes (eight fp16 activations) of the plain vector.
template <bool TP>
__device__ __forceinline__ uint4 gv_raw8(const GvParams& p, int it) {
    // inside a chain the vector was written earlier in this launch: read it past L1, which may hold older lines
    return (TP && p.chained) ? __ldcg(reinterpret_cast<const uint4*>(p.x + 8 * it)) : *reinterpret_cast<const uint4*>(p.x + 8 * it);
}
__device__ __forceinline__ void gv_unpack8(const uint4& raw, float (&v)[8]) {
    const uint32_t w[4] = { raw.x, raw.y, raw.z, raw.w };
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = a.x; v[2 * i + 1] = a.y;
    }
}

constexpr int GV_PRE = 2;           // staging items whose norm weights a thread loads before it waits for the producer
constexpr int GV_STAGE_REGS = 5;    // staging items (16 bytes each) a thread fetches up front and keeps in registers

// Activation image in shared memory.  Layout A (Q4_K): the int8 codes of super-block b in natural order, cut into
// sixteen 16-byte chunks j and stored chunk-major, chunk j of block b at (j * nb + b) * 16 — the lanes of a warp work
// on consecutive super-blocks, so their 16-byte reads are consecutive.  Layout B (Q6_K): plane k (= 32-wide quarter of
// a 128-half) at k*K/4, run (blk*4 + 2n + c)*16.  In 16-bit mode a second plane with the low bytes follows at +K.
// Group scales xd / xs: four floats of half h of block b at ((h * nb + b) * 4).
//
// `wpre`: the norm weights of this thread's first `npre` staging items, loaded by the caller before it waited for the
// producer kernel (they do not depend on it), so their trip to L2 is off the critical path.
struct GvRange { int gf[3], gl[3]; };   // row groups [gf, gl) of each segment owned by this CTA
__device__ __forceinline__ void gv_prefetch(const GvParams& p, const GvRange& rg, uint8_t* smem, uint64_t (*full)[GV_MAXSLOT], int warp, int lane, bool later,
                                            int u0, int u1);

// `late`: slots [p.early_slots, p.nslots) of every warp's ring are still empty; their bulk copies are issued here, right
// after the loads of the activation vector.  Requests leave an SM in order: a load issued behind the requests of a full
// ring waits for all of them (measured 1.4 us for the 5 KB vector against 0.6 behind half a ring).
template <bool DBG, bool TP>
__device__ __forceinline__ void stage_x(const GvParams& p, uint8_t* smem, float* red, const float (&wpre)[GV_PRE][8], int npre,
                                        const GvRange& rg, uint64_t (*full)[GV_MAXSLOT], bool late) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x, nw_cta = blockDim.x >> 5;
    const int K = p.K, nitems = K / 8, nb = K / QK_K;
    const uint32_t epoch = (TP && p.tp_wait_on) ? p.tpw.seq[0] * (uint32_t)p.tpw.epochs_per_step + (uint32_t)p.tpw.layer + 1u : 0u;
    const bool direct = !(TP && p.tp_wait_on);
    const bool xm = p.xmode != 0;             // 16-bit activations in two int8 planes instead of q8_1 codes (one copy of the code serves both)
    // every item of this thread is requested before any is used: one trip to L2, not one per item
    uint4 raw[GV_STAGE_REGS];
    #pragma unroll
    for (int k = 0; k < GV_STAGE_REGS; ++k) {
        const int it = tid + k * nthreads;
        raw[k] = (direct && it < nitems) ? gv_raw8<TP>(p, it) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (late) gv_prefetch(p, rg, smem, full, warp, lane, false, p.early_slots, p.nslots);
    float rrms = 1.0f;
    if (p.do_norm) {   // reference: fused_rmsnorm_residual, src/kernels/fused_norm.cu:33-101
        float ss = 0.f;
        if (direct) {
            #pragma unroll
            for (int k = 0; k < GV_STAGE_REGS; ++k) {      // lanes past the end hold zeros
                float a[8];
                gv_unpack8(raw[k], a);
                #pragma unroll
                for (int i = 0; i < 4; ++i) ss += a[2 * i] * a[2 * i] + a[2 * i + 1] * a[2 * i + 1];
            }
        }
        for (int g8 = tid + (direct ? GV_STAGE_REGS * nthreads : 0); g8 < nitems; g8 += nthreads) {
            float a[8];
            gv_load8<TP>(p, g8, epoch, a);
            #pragma unroll
            for (int i = 0; i < 4; ++i) ss += a[2 * i] * a[2 * i] + a[2 * i + 1] * a[2 * i + 1];
        }
        if (DBG && p.trace && tid == 0) p.trace[(size_t)blockIdx.x * GV_NTRACE + 12] = global_ns() + (ss == -1.f);
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < nw_cta; ++w) tot += red[w];
        rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.eps)));
        if (DBG && p.trace && tid == 0) p.trace[(size_t)blockIdx.x * GV_NTRACE + 13] = global_ns() + (rrms == -1.f);
    }
    uint8_t* xA = smem + p.off_xA; uint8_t* xB = smem + p.off_xB;
    float* xd = reinterpret_cast<float*>(smem + p.off_xd);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    int*   xsum = reinterpret_cast<int*>(smem + p.off_xsum);
    // Four threads per 32-element group, eight elements each; the group's absmax and sums are combined with two
    // xor-shuffles inside the quad.  K is a multiple of 256, so K/8 is a multiple of 32 and a warp is either entirely
    // inside an iteration or entirely outside: the shuffles are always between live lanes.
    auto quantise = [&](int it, float (&v)[8], int pre) {             // pre: index into wpre, or -1
        const int gi = it >> 2, q4 = it & 3;
        if (p.do_norm) {
            float wn[8];
            if (pre >= 0) {
                #pragma unroll
                for (int i = 0; i < 8; ++i) wn[i] = pre == 0 ? wpre[0][i] : wpre[1][i];
            } else {
                gv_norm_w8(p, it, wn);
            }
            #pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(v[i], rrms), wn[i])));
        }
        float amax = 0.f;
        #pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
        const float lim = xm ? 32767.0f : 127.0f;
        const int ilim = xm ? 32767 : 127, hshift = xm ? 8 : 0;
        const float d = __fdiv_rn(amax, lim);                      // q8_1: src/kernels/gemv_q4.cu:445-466
        const float id = d > 0.f ? __fdiv_rn(1.0f, d) : 0.f;
        uint32_t hi[2] = { 0, 0 }, lo[2] = { 0, 0 };
        int s8 = 0;
        #pragma unroll
        for (int w = 0; w < 2; ++w) {
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x = v[4 * w + i];
                const int q = max(-ilim, min(ilim, __float2int_rn(__fmul_rn(x, id))));
                s8 += q;
                hi[w] |= (uint32_t)((q >> hshift) & 0xFF) << (8 * i);
                lo[w] |= (uint32_t)(q & 0xFF) << (8 * i);          // second plane, 16-bit mode only
            }
        }
        const int s16 = s8 + __shfl_xor_sync(0xFFFFFFFFu, s8, 1);          // code sum of this thread's 16-element half
        const int s32 = s16 + __shfl_xor_sync(0xFFFFFFFFu, s16, 2);
        // fp32 sum of the group in the order of an 8-lane xor tree over 4-element partial sums (16-bit mode)
        const float t = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
        const float t2 = t + __shfl_xor_sync(0xFFFFFFFFu, t, 1);
        const float fsum = t2 + __shfl_xor_sync(0xFFFFFFFFu, t2, 2);
        const int blk = gi >> 3, j = gi & 7, h = q4 >> 1, e8 = (q4 & 1) * 8;    // 16-element half h, byte offset inside its run
        if (p.needA) {
            const int off = ((2 * j + h) * nb + blk) * 16 + e8;
            *reinterpret_cast<uint2*>(xA + off) = make_uint2(hi[0], hi[1]);
            if (xm) *reinterpret_cast<uint2*>(xA + K + off) = make_uint2(lo[0], lo[1]);
        }
        if (p.needB) {
            const int n = j >> 2, k = j & 3;
            const int off = k * (K >> 2) + (blk * 4 + 2 * n + h) * 16 + e8;
            *reinterpret_cast<uint2*>(xB + off) = make_uint2(hi[0], hi[1]);
            if (xm) *reinterpret_cast<uint2*>(xB + K + off) = make_uint2(lo[0], lo[1]);
            if ((q4 & 1) == 0) xsum[2 * gi + h] = s16;
        }
        if (q4 == 0) {
            const int si = ((j >> 2) * nb + blk) * 4 + (j & 3);
            if (!xm) {
                xd[si] = __half2float(__float2half_rn(d));
                xs[si] = __half2float(__float2half_rn(__fmul_rn(d, (float)s32)));
            } else {
                xd[si] = d;
                xs[si] = fsum;
            }
        }
    };
    // ONE copy of the quantiser in a loop that is not unrolled.  Code size matters here: in a decode step every launch
    // meets a cold instruction cache (four different kernels have run since its last launch) and fetches its code behind
    // the weight stream; an unrolled staging phase alone was 20 KB of straight-line code on the path to the first dot.
    #pragma unroll 1
    for (int k = 0, it = tid; it < nitems; ++k, it += nthreads) {      // warp-uniform trip count: nitems is a multiple of 32
        float v[8];
        if (direct && k < GV_STAGE_REGS) {
            uint4 r = raw[0];
            #pragma unroll
            for (int j = 1; j < GV_STAGE_REGS; ++j)
                if (k == j) r = raw[j];
            gv_unpack8(r, v);
        } else {
            gv_load8<TP>(p, it, epoch, v);
        }
        quantise(it, v, k < npre ? k : -1);
    }
    if (DBG && p.trace && tid == 0) p.trace[(size_t)blockIdx.x * GV_NTRACE + 14] = global_ns();
}

// ── shared-memory reads by 32-bit shared address (no generic-pointer arithmetic in the inner loop) ──
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) { uint32_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ int lds_s8(uint32_t a) { int v; asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }

__device__ __forceinline__ int dot16_us(const uint4& w, uint32_t mask, const uint4& x) {
    int d = dp4a_us(w.x & mask, (int)x.x, 0); d = dp4a_us(w.y & mask, (int)x.y, d);
    d = dp4a_us(w.z & mask, (int)x.z, d);     return dp4a_us(w.w & mask, (int)x.w, d);
}
__device__ __forceinline__ int dot16_uu(const uint4& w, uint32_t mask, const uint4& x) {
    int d = dp4a_uu(w.x & mask, x.x, 0); d = dp4a_uu(w.y & mask, x.y, d);
    d = dp4a_uu(w.z & mask, x.z, d);     return dp4a_uu(w.w & mask, x.w, d);
}

// shared addresses of the staged activation image
struct GvX { uint32_t xA, xB, xd, xs, xsum; int K, nb; };

// ── Q6_K: one (half n, column run c) per lane = 64 weights in four 16-element scale groups (quarters k = 0..3
// at +32k), reference arithmetic src/kernels/gemv_q4.cu:581-618: per group  d*sc*(d8*dot)  with
// dot = Σ(q6-32)·x = Σq6·x - 32·Σx.  Blocks are 2-byte aligned: each 16-byte run is read as five aligned words
// and funnel-shifted.  n and c are fixed per lane.
template <int XM>
__device__ __forceinline__ float q6k_item(uint32_t sb, int n, int c, int kblk, const GvX& X, int dots_out[4]) {
    const uint32_t al = sb & ~3u, sh = (sb & 2u) * 8u;
    uint32_t A[4], B[4], H[4];
    {
        const uint32_t pa = al + 64 * n + 16 * c, ph = al + 128 + 32 * n + 16 * c;
        uint32_t wa[5], wb[5], wh[5];
        #pragma unroll
        for (int i = 0; i < 5; ++i) { wa[i] = lds32(pa + 4 * i); wb[i] = lds32(pa + 32 + 4 * i); wh[i] = lds32(ph + 4 * i); }
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            A[i] = __funnelshift_r(wa[i], wa[i + 1], sh); B[i] = __funnelshift_r(wb[i], wb[i + 1], sh); H[i] = __funnelshift_r(wh[i], wh[i + 1], sh);
        }
    }
    const float d = h2f_bits(lds_u16(sb + 208));
    const uint32_t sca = sb + 192 + 8 * n + c;
    const uint32_t xb = X.xB + (kblk * 4 + 2 * n + c) * 16;
    const uint32_t xsa = X.xsum + (kblk * 16 + 8 * n + c) * 4;
    const uint4 xdr = lds128(X.xd + (uint32_t)(n * X.nb + kblk) * 16u);
    const float xdv[4] = { __uint_as_float(xdr.x), __uint_as_float(xdr.y), __uint_as_float(xdr.z), __uint_as_float(xdr.w) };
    // high bit pairs of the four quarters, already in place (bits 4-5 of every byte)
    uint32_t Hq[4][4];
    #pragma unroll
    for (int w = 0; w < 4; ++w) {
        Hq[0][w] = (H[w] << 4) & 0x30303030u; Hq[1][w] = (H[w] << 2) & 0x30303030u;
        Hq[2][w] = H[w] & 0x30303030u;        Hq[3][w] = (H[w] >> 2) & 0x30303030u;
    }
    float acc = 0.f;
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint4 xv = lds128(xb + k * (X.K >> 2));
        const uint32_t xw[4] = { xv.x, xv.y, xv.z, xv.w };
        uint32_t yw[4] = { 0, 0, 0, 0 };
        if (XM == 1) { const uint4 yv = lds128(xb + X.K + k * (X.K >> 2)); yw[0] = yv.x; yw[1] = yv.y; yw[2] = yv.z; yw[3] = yv.w; }
        int dh = 0, dl = 0;
        #pragma unroll
        for (int w = 0; w < 4; ++w) {
            const uint32_t src = (k & 1) ? B[w] : A[w];
            const uint32_t v = (((k & 2) ? (src >> 4) : src) & 0x0F0F0F0Fu) | Hq[k][w];
            dh = dp4a_us(v, (int)xw[w], dh);
            if (XM == 1) dl = dp4a_uu(v, yw[w], dl);
        }
        const int dot = (XM == 1 ? dh * 256 + dl : dh) - 32 * (int)lds32(xsa + 8 * k);
        dots_out[k] = dot;
        acc += (float)dot * ((float)lds_s8(sca + 2 * k) * xdv[k]);
    }
    return d * acc;
}

// ── Q4_K: one super-block COLUMN per lane, RL rows deep ──────────────────
// The warp is cut into groups of `lw` lanes; lane c of group g owns super-block column c of the RL consecutive rows
// g*RL .. g*RL + RL - 1 of the task (a row with more than lw blocks is walked in passes c, c + lw, ...).  The 256
// activation codes and eight group scales of a column are read from shared memory ONCE and multiplied against all RL
// rows, so a block costs 9 sixteen-byte shared loads (its own 144 bytes) plus 20 / RL for the activations, instead of
// 29: the kernel is bound by shared-memory bandwidth once all its weights are in flight, and this is what halves it.
// Arithmetic per (row, block) is that of the reference (src/kernels/gemv_q4.cu:487-499): eight 32-element dp4a dots,
// folded as  dall * Σ_j sc_j*dot_j*d8_j  -  dmin * Σ_j m_j*s8_j  with the scales unpacked four at a time by word-wide
// masks (get_scale_min_k4, :185-195); it does not depend on RL, so every launch shape gives the same bits per row.
// `nrw` rows are present (the last task of a matrix may hold fewer than lg*RL); acc[r] collects row g*RL + r.
template <int XM, int RL, bool DBG>
__device__ __forceinline__ void q4k_columns(uint32_t rows, int nrw, unsigned rb, int nbc, int kb0, int Ufull, int lane, const GvX& X,
                                            unsigned lw, unsigned lg, float (&acc)[4], int32_t* dbg) {
    const unsigned g = (unsigned)lane / lw, c = (unsigned)lane - g * lw;
    const int rbase = (int)g * RL;
    const int nr = min(RL, nrw - rbase);
    if (g >= lg || nr <= 0) return;
    const uint32_t step = (uint32_t)X.nb * 16u;                 // bytes between consecutive 16-byte chunks of one block's codes
    for (unsigned blk = c; blk < (unsigned)nbc; blk += lw) {
        const int kblk = kb0 + (int)blk;
        const uint32_t sb0 = rows + (uint32_t)rbase * rb + blk * Q4K_BYTES;
        uint32_t sclo[RL], schi[RL];       // 6-bit scales of sub-blocks 0..3 / 4..7, a byte each
        float dall[RL], pos[RL], fixed[RL];
        {
            const uint4 sA = lds128(X.xs + (uint32_t)kblk * 16u), sB = lds128(X.xs + (uint32_t)(X.nb + kblk) * 16u);
            const float s8[8] = { __uint_as_float(sA.x), __uint_as_float(sA.y), __uint_as_float(sA.z), __uint_as_float(sA.w),
                                  __uint_as_float(sB.x), __uint_as_float(sB.y), __uint_as_float(sB.z), __uint_as_float(sB.w) };
            #pragma unroll
            for (int r = 0; r < RL; ++r) {
                const uint4 hdr = lds128(sb0 + (uint32_t)min(r, nr - 1) * rb);
                sclo[r] = hdr.y & 0x3F3F3F3Fu;
                schi[r] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t mn03 = hdr.z & 0x3F3F3F3Fu, mn47 = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                float neg = 0.f;
                #pragma unroll
                for (int il = 0; il < 4; ++il) {
                    const uint32_t mnw = il < 2 ? mn03 : mn47;
                    const int sh = 16 * (il & 1);
                    neg += (float)(int)((mnw >> sh) & 0xFFu) * s8[2 * il] + (float)(int)((mnw >> (sh + 8)) & 0xFFu) * s8[2 * il + 1];
                }
                const float2 dm = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));      // (d, dmin)
                dall[r] = dm.x; fixed[r] = dm.y * neg; pos[r] = 0.f;
            }
        }
        const uint32_t xa = X.xA + (uint32_t)kblk * 16u;
        #pragma unroll 1                                            // kept rolled: a quarter of the code, and the RL rows give the parallelism
        for (int il = 0; il < 4; ++il) {
            const uint32_t xc = xa + (uint32_t)(4 * il) * step;     // chunks 4il, 4il+1: sub-block 2il; 4il+2, 4il+3: sub-block 2il+1
            const uint4 xl0 = lds128(xc), xl1 = lds128(xc + step), xh0 = lds128(xc + 2 * step), xh1 = lds128(xc + 3 * step);
            uint4 yl0, yl1, yh0, yh1;
            if (XM == 1) {                                          // second plane: low bytes of the 16-bit activations
                const uint32_t yc = xc + (uint32_t)X.K;
                yl0 = lds128(yc); yl1 = lds128(yc + step); yh0 = lds128(yc + 2 * step); yh1 = lds128(yc + 3 * step);
            }
            // scales of the two 32-element groups of this quarter: floats 2il, 2il+1 of the block's eight
            const uint2 dq = lds64(X.xd + (uint32_t)((il >> 1) * X.nb + kblk) * 16u + (uint32_t)(il & 1) * 8u);
            const float d8a = __uint_as_float(dq.x), d8b = __uint_as_float(dq.y);
            const int sh = 16 * (il & 1);
            #pragma unroll
            for (int r = 0; r < RL; ++r) {
                const uint32_t sbr = sb0 + (uint32_t)min(r, nr - 1) * rb;
                const uint4 w0 = lds128(sbr + 16 + 32 * il), w1 = lds128(sbr + 32 + 32 * il);
                int dot0, dot1;
                if (XM == 0) {
                    dot0 = dot16_us(w0, 0x0F0F0F0Fu, xl0) + dot16_us(w1, 0x0F0F0F0Fu, xl1);
                    dot1 = (dot16_us(w0, 0xF0F0F0F0u, xh0) + dot16_us(w1, 0xF0F0F0F0u, xh1)) >> 4;   // exact: every term is a multiple of 16
                } else {
                    dot0 = (dot16_us(w0, 0x0F0F0F0Fu, xl0) + dot16_us(w1, 0x0F0F0F0Fu, xl1)) * 256 +
                           (dot16_uu(w0, 0x0F0F0F0Fu, yl0) + dot16_uu(w1, 0x0F0F0F0Fu, yl1));
                    dot1 = ((dot16_us(w0, 0xF0F0F0F0u, xh0) + dot16_us(w1, 0xF0F0F0F0u, xh1)) * 16 +
                            ((dot16_uu(w0, 0xF0F0F0F0u, yh0) + dot16_uu(w1, 0xF0F0F0F0u, yh1)) >> 4));
                }
                if (DBG && dbg && r < nr) {
                    int32_t* o = dbg + (size_t)(rbase + r) * (2 * Ufull) + (size_t)kblk * 8;
                    o[2 * il] = dot0; o[2 * il + 1] = dot1;
                }
                const uint32_t scw = il < 2 ? sclo[r] : schi[r];
                const int sc0 = (int)((scw >> sh) & 0xFFu), sc1 = (int)((scw >> (sh + 8)) & 0xFFu);
                pos[r] += (float)(sc0 * dot0) * d8a + (float)(sc1 * dot1) * d8b;
            }
        }
        #pragma unroll
        for (int r = 0; r < RL; ++r)
            if (r < nr) acc[r] += dall[r] * pos[r] - fixed[r];
    }
}

// One warp, `nrw` consecutive rows in shared memory.  Q4_K: q4k_columns with the segment's lane map.  Q6_K (nrw <= 4):
// lanes stride over 32-byte items (4 per super-block); 32 and U are multiples of 4, so a lane's sub-item never changes;
// each lane adds its terms into the accumulator of the row the item belongs to.
// `rb_` = bytes between consecutive rows in shared memory, `U_` = 4 x the super-blocks per row held there (a chunk of
// the row when the row is streamed in several tasks: its first super-block is kb0), `Ufull` = 4 x those of a whole row.
template <int XM, int TYPE, bool DBG>
__device__ __forceinline__ void consume_rows(uint32_t rows, int nrw, int rb_, int U_, int kb0, int Ufull, int lane, const GvX& X,
                                             const GvSegDev& sg, float (&acc)[4], int32_t* dbg) {
    const unsigned rb = (unsigned)rb_;
    if (TYPE == T_Q4K) {
        const int nbc = U_ >> 2;
        switch (sg.rl) {
            case 1:  q4k_columns<XM, 1, DBG>(rows, nrw, rb, nbc, kb0, Ufull, lane, X, sg.lw, sg.lg, acc, dbg); break;
            default: q4k_columns<XM, 3, DBG>(rows, nrw, rb, nbc, kb0, Ufull, lane, X, sg.lw, sg.lg, acc, dbg); break;
        }
        return;
    }
    const unsigned U = (unsigned)U_, total = (unsigned)nrw * U;
    const int sub = lane & 3;
    for (unsigned base = 0; base < total; base += 32) {
        const unsigned i = base + lane;
        const bool valid = i < total;
        const unsigned ii = valid ? i : (unsigned)sub;
        const unsigned rl = (ii >= U) + (ii >= 2 * U) + (ii >= 3 * U);
        const unsigned blk = (ii - rl * U) >> 2;
        const uint32_t sb = rows + rl * rb + blk * Q6K_BYTES;
        int dots[4];
        float term = q6k_item<XM>(sb, sub >> 1, sub & 1, kb0 + (int)blk, X, dots);
        if (DBG && dbg && valid) {
            int32_t* o = dbg + (size_t)rl * (4 * Ufull) + (kb0 + blk) * 16 + 8 * (sub >> 1) + (sub & 1);
            o[0] = dots[0]; o[2] = dots[1]; o[4] = dots[2]; o[6] = dots[3];
        }
        if (!valid) term = 0.f;
        acc[0] += rl == 0 ? term : 0.f; acc[1] += rl == 1 ? term : 0.f;
        acc[2] += rl == 2 ? term : 0.f; acc[3] += rl == 3 ? term : 0.f;
    }
}

// A warp's unit of work is one row group (R consecutive rows of one matrix).  Every warp runs its own
// pipeline: its lane 0 issues the bulk copy of a group into one of the warp's slots, the warp waits on that
// slot's mbarrier, consumes the rows and moves on — no CTA-wide barrier in the loop, so dot products start
// as soon as the first group lands while the rest of the CTA's bytes are still in flight.
// task `u` of warp `warp` -> segment, first row, number of rows
struct GvTask { int seg, row0, nrows, kb0, kb1; bool last; };   // rows [row0, row0+nrows) x super-blocks [kb0, kb1); last chunk of the rows

__device__ __forceinline__ bool gv_task(const GvParams& p, const GvRange& rg, int warp, int u_, GvTask& t) {
    int g;
    int& seg = t.seg; int& row0 = t.row0; int& nrows = t.nrows;
    const int c = p.nchunk > 1 ? u_ % p.nchunk : 0, u = p.nchunk > 1 ? u_ / p.nchunk : u_;
    const int nb = p.K / QK_K;
    t.kb0 = c * p.chunk_blocks; t.kb1 = min(nb, t.kb0 + p.chunk_blocks); t.last = c == p.nchunk - 1;
    if (p.paired_rows) {               // (gate group, up group) of the same rows, back to back on one warp
        seg = u & 1;
        g = rg.gf[0] + warp + p.nwarps * (u >> 1);
        if (g >= rg.gl[0]) return false;
    } else {
        int k = warp + p.nwarps * u;
        seg = -1;
        #pragma unroll
        for (int i = 0; i < 3; ++i) {
            const int cnt = rg.gl[i] - rg.gf[i];
            if (seg < 0 && i < p.nseg) { if (k < cnt) { seg = i; g = rg.gf[i] + k; } else k -= cnt; }
        }
        if (seg < 0) return false;
    }
    const int R = p.seg[seg].R;
    row0 = g * R;
    nrows = min(R, p.seg[seg].M - row0);
    return nrows > 0;
}

// global byte range of a task: whole rows, or (one row only) the super-blocks [kb0, kb1) of it
__device__ __forceinline__ void gv_span(const GvParams& p, const GvTask& t, uintptr_t& g0, uintptr_t& g1) {
    const GvSegDev& s = p.seg[t.seg];
    const int bb = s.type == T_Q4K ? Q4K_BYTES : Q6K_BYTES;
    g0 = (uintptr_t)s.W + (size_t)t.row0 * s.rb + (size_t)(p.nchunk > 1 ? t.kb0 * bb : 0);
    g1 = p.nchunk > 1 ? g0 + (size_t)(t.kb1 - t.kb0) * bb : g0 + (size_t)t.nrows * s.rb;
}

__device__ __forceinline__ void gv_issue(const GvParams& p, const GvTask& t, uint8_t* slot, uint64_t* bar) {
    const GvSegDev& s = p.seg[t.seg];
    uintptr_t g0, g1;
    gv_span(p, t, g0, g1);
    const uintptr_t a0 = g0 & ~(uintptr_t)15;
    const uintptr_t endw = ((uintptr_t)s.W + (size_t)s.M * s.rb) & ~(uintptr_t)15;
    uintptr_t a1 = (g1 + 15) & ~(uintptr_t)15;
    if (a1 > endw) a1 = endw;                     // never read past the tensor; the tail comes by plain loads
    const uint32_t bytes = (uint32_t)(a1 - a0);
    mbar_expect_tx(bar, bytes);
    bulk_g2s(slot, (const void*)a0, bytes, bar);
}

// first tasks of a phase: start the bulk copies of this warp's first row groups.  The slot barriers are created once
// per kernel and live through all phases of a chain; `later` = not the first phase of the launch.
__device__ __forceinline__ void gv_prefetch(const GvParams& p, const GvRange& rg, uint8_t* smem, uint64_t (*full)[GV_MAXSLOT], int warp, int lane, bool later,
                                            int u0, int u1) {
    if (warp >= p.nwarps) return;
    uint8_t* ring = smem + p.off_slots + (unsigned)warp * (unsigned)(p.nslots * p.slot_bytes);
    if (lane == 0) {
        if (later) fence_proxy_async();       // the slots were read with ordinary loads in the phase before
        for (int u = u0; u < u1; ++u) {
            GvTask t;
            if (!gv_task(p, rg, warp, u, t)) break;
            gv_issue(p, t, ring + (unsigned)u * (unsigned)p.slot_bytes, &full[warp][u]);
        }
    }
    __syncwarp();
}

// one GEMV launch, or one phase of a chain (then the caller has prefetched and synchronised the grid)
__device__ __forceinline__ void gv_stamp(const GvParams& p, int k) {
    p.trace[(size_t)blockIdx.x * GV_NTRACE + k] = global_ns();
}

// Q4: the launch may hold Q4_K matrices (false: Q6_K only — the Q4_K code, which wants 128 registers, is left out of the
// 80-register instantiation).
template <bool DBG, bool Q4, bool TP>
__device__ __forceinline__ void gv_phase(const GvParams& p, uint8_t* smem, uint64_t (*full)[GV_MAXSLOT], float* red, const GvRange& rg, uint32_t& par,
                                         const float (&wpre)[GV_PRE][8], int npre, bool late) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    uint8_t* ring = smem + p.off_slots + (unsigned)warp * (unsigned)(p.nslots * p.slot_bytes);
    // the activation format (p.xmode) is a run-time switch inside the quantiser and around the dot products; everything else
    // exists once
    stage_x<DBG, TP>(p, smem, red, wpre, npre, rg, full, late);
    __syncthreads();
    if (DBG && p.trace && tid == 0) gv_stamp(p, 3);
    if (warp >= p.nwarps) return;            // chain phases may use fewer warps than the CTA has (larger staging rings)

    const uint32_t sm0 = smem_u32(smem);
    const GvX X = { sm0 + p.off_xA, sm0 + p.off_xB, sm0 + p.off_xd, sm0 + p.off_xs, sm0 + p.off_xsum, p.K, p.K / QK_K };
    const uint32_t push_epoch = (TP && p.tp_push_on) ? p.tpp.seq[0] * (uint32_t)p.tpp.epochs_per_step + (uint32_t)p.tpp.layer + 1u : 0u;
    bool timed_out = false;
    float gate_keep[4] = { 0.f, 0.f, 0.f, 0.f };
    float acc[4] = { 0.f, 0.f, 0.f, 0.f };       // lives across the chunks of a row
    for (int u = 0;; ++u) {
        GvTask t;
        if (!gv_task(p, rg, warp, u, t)) break;
        const int seg = t.seg, row0 = t.row0, nrows = t.nrows;
        const int slot = u % p.nslots;
        // a wait that runs out is recorded and the loop carries on; later waits are skipped.  `par` holds, per slot
        // barrier, the parity of the phase its next copy completes (barriers live across the phases of a chain).
        if (!timed_out && !mbar_wait_bounded(&full[warp][slot], (par >> slot) & 1u)) timed_out = true;
        par ^= 1u << slot;
        if (DBG && p.trace && tid == 0 && u == 0) gv_stamp(p, 4);
        if (DBG && p.trace && tid == 0 && u < 4) gv_stamp(p, 8 + 2 * u);          // warp 0: task u has landed
        const GvSegDev& s = p.seg[seg];
        uintptr_t g0, g1;
        gv_span(p, t, g0, g1);
        uint8_t* rows = ring + (unsigned)slot * (unsigned)p.slot_bytes + (unsigned)(g0 & 15);
        {   // bytes between the last 16-byte boundary inside the tensor and its end
            const uintptr_t endw = ((uintptr_t)s.W + (size_t)s.M * s.rb) & ~(uintptr_t)15;
            if (g1 > endw) {     // warp-uniform
                const int tail = (int)(g1 - endw);
                if (lane < tail) rows[(endw - g0) + lane] = reinterpret_cast<const uint8_t*>(endw)[lane];
                __syncwarp();
            }
        }
        int32_t* dbg = (DBG && seg == 0 && p.dbg_dots) ? p.dbg_dots + (size_t)row0 * (s.type == T_Q4K ? 2 * s.U : 4 * s.U) : nullptr;
        const int Uc = p.nchunk > 1 ? 4 * (t.kb1 - t.kb0) : s.U, kb0 = p.nchunk > 1 ? t.kb0 : 0;
        if (!(DBG && p.trace && p.trace_nocompute)) {
            if (Q4 && s.type == T_Q4K) {
                if (p.xmode) consume_rows<1, T_Q4K, DBG>(smem_u32(rows), nrows, s.rb, Uc, kb0, s.U, lane, X, s, acc, dbg);
                else         consume_rows<0, T_Q4K, DBG>(smem_u32(rows), nrows, s.rb, Uc, kb0, s.U, lane, X, s, acc, dbg);
            } else {
                if (p.xmode) consume_rows<1, T_Q6K, DBG>(smem_u32(rows), nrows, s.rb, Uc, kb0, s.U, lane, X, s, acc, dbg);
                else         consume_rows<0, T_Q6K, DBG>(smem_u32(rows), nrows, s.rb, Uc, kb0, s.U, lane, X, s, acc, dbg);
            }
        }
        __syncwarp();                            // the warp is done reading this slot
        if (DBG && p.trace && tid == 0 && u < 4) gv_stamp(p, 9 + 2 * u);          // warp 0: task u has been multiplied
        if (lane == 0) {
            GvTask t2;
            if (gv_task(p, rg, warp, u + p.nslots, t2)) {
                fence_proxy_async();
                gv_issue(p, t2, ring + (unsigned)slot * (unsigned)p.slot_bytes, &full[warp][slot]);
            }
        }
        if (!t.last) continue;                   // more super-blocks of these rows follow in the next task
        float mine = 0.f;
        bool has_row; int row_local;
        if (Q4 && s.type == T_Q4K) {
            // Lane c of group g holds partial sums of rows g*rl + r in acc[r]: a guarded shuffle-down tree over the lw lanes of
            // the group (any width) leaves the totals in the group's first lane, which hands total r to lane r of the group.
            const unsigned lw = s.lw, g = (unsigned)lane / lw, c = (unsigned)lane - g * lw;
            #pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                if ((unsigned)off < lw) {
                    #pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float o = __shfl_down_sync(0xFFFFFFFFu, acc[r], off);
                        if (c + (unsigned)off < lw) acc[r] += o;
                    }
                }
            }
            const int first = g < s.lg ? (int)(g * lw) : lane;
            #pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float o = __shfl_sync(0xFFFFFFFFu, acc[r], first);
                if (c == (unsigned)r) mine = o;
            }
            row_local = (int)(g * s.rl + c);
            has_row = g < s.lg && c < s.rl && row_local < nrows;
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        } else {
            // Row sums in six shuffles instead of twenty: the halves of the warp take over two rows each (xor 16), the quarters
            // one row each (xor 8), then three steps inside the octet.  Every lane of octet r ends with the sum of row r; its
            // first lane finishes the row.
            const bool hi16 = lane & 16, hi8 = lane & 8;
            float k0 = hi16 ? acc[2] : acc[0], k1 = hi16 ? acc[3] : acc[1];
            const float g0 = hi16 ? acc[0] : acc[2], g1 = hi16 ? acc[1] : acc[3];
            k0 += __shfl_xor_sync(0xFFFFFFFFu, g0, 16);
            k1 += __shfl_xor_sync(0xFFFFFFFFu, g1, 16);
            float v = hi8 ? k1 : k0;
            v += __shfl_xor_sync(0xFFFFFFFFu, hi8 ? k0 : k1, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            mine = v;
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            row_local = lane >> 3;               // the row of this lane's octet
            has_row = (lane & 7) == 0 && row_local < nrows;
        }
        if (p.out_mode == 3 && seg == 0) {       // gate values stay in registers until the matching up rows arrive
            gate_keep[0] = __half2float(__float2half_rn(mine));      // the lane that will finish row r keeps its gate value
            continue;
        }
        if (has_row) {
            const int row = row0 + row_local;
            if (p.out_mode == 0)      reinterpret_cast<__half*>(s.y)[row] = __float2half_rn(mine);
            else if (p.out_mode == 1) reinterpret_cast<float*>(s.y)[row] = mine;
            else if (p.out_mode == 2) {   // src/kernels/gemv_q4.cu:996-999
                const __half pr = __float2half_rn(mine);
                float res;
                if (TP && p.residual_pk) {    // written earlier in this launch by another CTA of this rank: valid once its epoch matches
                    uint2 q;
                    PollGuard guard(p.status);
                    for (;;) {
                        q = __ldcv(p.residual_pk + row);
                        if (q.y == push_epoch || !guard.again(p.status)) break;
                    }
                    res = __half2float(__ushort_as_half((unsigned short)(q.x & 0xFFFFu)));
                } else {
                    res = __half2float((TP && p.chained) ? __ldcg(p.residual + row) : p.residual[row]);
                }
                reinterpret_cast<__half*>(s.y)[row] = __float2half_rn(__fadd_rn(__half2float(pr), res));
            } else {                      // fused SwiGLU of the gate/up pair (src/kernels/convert.cu:85-104)
                const float hv = __half2float(__float2half_rn(mine));
                const float g = gate_keep[0];
                reinterpret_cast<__half*>(p.seg[0].y)[row] = __float2half_rn(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), hv));
            }
            if (TP && p.tp_push_on) {     // the value just stored, as a packet to every rank (this one included)
                const unsigned short bits = __half_as_ushort(reinterpret_cast<const __half*>(p.out_mode == 3 ? p.seg[0].y : s.y)[row]);
                const uint2 pkt = make_uint2((uint32_t)bits, push_epoch);
                #pragma unroll 1
                for (int r = 0; r < p.tpp.world; ++r)
                    reinterpret_cast<uint2*>(p.tpp.peer[r] + p.tpp.buf_off)[p.tpp.row_off + row] = pkt;
            }
        }
    }
    if (timed_out && lane == 0) atomicExch(p.status, JB_ERR_TIMEOUT);
    if (DBG && p.trace && lane == 0) {
        if (warp == 0) gv_stamp(p, 5);
        atomicMax(&p.trace[(size_t)blockIdx.x * GV_NTRACE + 6], global_ns());       // last warp of the CTA to finish
    }
}


// this CTA's row groups in every segment: an even split of all groups by weight (bytes per group, scaled by the host so
// that the total fits 31 bits; 1 per group of the first matrix for a gate/up pair).  The arithmetic runs on the path from
// CTA entry to the first bulk copy: 32-bit only, total * b / grid as q*b + r*b/grid with q, r from the host.
__device__ __forceinline__ GvRange gv_range(const GvParams& p) {
    GvRange rg;
    const unsigned G = gridDim.x, b = blockIdx.x;
    const unsigned lo = p.split_q * b + (p.split_r * b) / G, hi = p.split_q * (b + 1u) + (p.split_r * (b + 1u)) / G;
    unsigned cum = 0;
    #pragma unroll
    for (int i = 0; i < 3; ++i) {
        rg.gf[i] = rg.gl[i] = 0;
        if (i < p.nseg && p.gw[i]) {
            const unsigned w = p.gw[i], n = p.ng[i];
            const unsigned f = lo <= cum ? 0u : (lo - cum + w - 1u) / w, l = hi <= cum ? 0u : (hi - cum + w - 1u) / w;
            rg.gf[i] = (int)(f > n ? n : f); rg.gl[i] = (int)(l > n ? n : l);
            cum += w * n;
        }
    }
    if (p.paired_rows) { rg.gf[1] = rg.gf[0]; rg.gl[1] = rg.gl[0]; }      // out_mode 3: the same groups of both matrices
    return rg;
}

// TP: with the tensor-parallel hooks (activations and residuals as polled packets, results pushed to the peers); the
// single-GPU instantiation leaves that code out.
template <bool DBG, bool TP>
__global__ void __launch_bounds__(GV_MAXWARPS * 32, 2) gemv_stream_kernel(const __grid_constant__ GvParams p) {
    constexpr int MW = GV_MAXWARPS;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[MW][GV_MAXSLOT];
    __shared__ float red[MW];
    {   // Touch every 128-byte line of the argument block at once: the first read of each line after a launch misses the
        // constant cache, and the path to the first bulk copy would otherwise take those misses one after the other.
        const int* pw = reinterpret_cast<const int*>(&p);
        int touched = 0;
        #pragma unroll
        for (int i = 0; i < (int)(sizeof(GvParams) / 4); i += 32) touched |= pw[i];
        if (touched == 0x7F7F7F7F && p.nseg == 99) red[0] = 0.f;       // never true; keeps the loads
    }
    if (DBG && p.trace && threadIdx.x == 0) { gv_stamp(p, 0); p.trace[(size_t)blockIdx.x * GV_NTRACE + 6] = 0ull; }
    pdl_launch();                // the next kernel's CTAs may take the free half of every SM now; they wait for our completion
                                 // before they touch our outputs
    const GvRange rg = gv_range(p);
    if (DBG && p.trace && threadIdx.x == 0) p.trace[(size_t)blockIdx.x * GV_NTRACE + 7] = global_ns() + (rg.gf[0] == -7);
    if ((threadIdx.x & 31) == 0) {
        for (int s = 0; s < p.nslots; ++s) mbar_init(&full[threadIdx.x >> 5][s], 1);
        fence_mbar_init();
    }
    __syncwarp();
    if (DBG && p.trace && threadIdx.x == 0) gv_stamp(p, 15);
    gv_prefetch(p, rg, smem, full, threadIdx.x >> 5, threadIdx.x & 31, false, 0, p.early_slots);   // weights do not depend on the previous kernel
    float wpre[GV_PRE][8];
    int npre = 0;
    #pragma unroll
    for (int k = 0; k < GV_PRE; ++k) {                                            // nor do the norm weights
        const int it = (int)threadIdx.x + k * (int)blockDim.x;
        #pragma unroll
        for (int i = 0; i < 8; ++i) wpre[k][i] = 0.f;
        if (p.do_norm && it < p.K / 8) { gv_norm_w8(p, it, wpre[k]); npre = k + 1; }
    }
    if (DBG && p.trace && threadIdx.x == 0) gv_stamp(p, 1);
    pdl_wait();                  // x (and the residual) come from the kernel before us
    if (DBG && p.trace && threadIdx.x == 0) gv_stamp(p, 2);
    uint32_t par = 0;
    gv_phase<DBG, true, TP>(p, smem, full, red, rg, par, wpre, npre, p.early_slots < p.nslots);
}

// ── chain: up to four GEMVs that feed one another (Wo -> gate/up -> W_down -> next layer's Q/K/V) in ONE launch ──
// One persistent CTA per SM runs the phases in order with a grid-wide barrier between them.  Against separate
// launches this removes the kernel boundary (drain, launch, first bulk-copy round trip) three times per layer: the
// first weight copies of the next phase are issued before the CTA enters the barrier, so they fly while it waits.
// The barrier is a ticket counter plus a generation word in global memory; the wait is bounded and a timeout is
// recorded in the status word (the phase then runs on whatever has arrived).  All CTAs must be resident at the same
// time: the grid never exceeds the number of SMs and a CTA takes a whole SM.
struct GvChain { int n; unsigned int* bar; GvParams ph[4]; };
static_assert(sizeof(GvChain) <= 4000, "kernel parameter space");

__device__ __forceinline__ void gv_grid_barrier(unsigned int* bar, int* status) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int gen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
        const unsigned int ticket = atomicAdd(bar, 1u);
        if (ticket == gridDim.x - 1) {
            *bar = 0u;
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen + 1u) : "memory");
        } else {
            unsigned int g, i = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(bar + 1) : "memory");
                if (g != gen) break;
                if (++i > (1u << 22)) { atomicExch(status, JB_ERR_TIMEOUT); break; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(GV_CHAINTHREADS, 1) gemv_chain_kernel(const __grid_constant__ GvChain c) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full[GV_CHAINWARPS][GV_MAXSLOT];
    __shared__ float red[GV_CHAINWARPS];
    const float wpre[GV_PRE][8] = {};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {                          // slot barriers of every warp, for all phases
        for (int s = 0; s < GV_MAXSLOT; ++s) mbar_init(&full[warp][s], 1);
        fence_mbar_init();
    }
    __syncwarp();
    uint32_t par = 0;                         // per slot barrier: parity of the phase its next copy completes
    GvRange rg = gv_range(c.ph[0]);
    gv_prefetch(c.ph[0], rg, smem, full, warp, lane, false, 0, c.ph[0].nslots);
    pdl_launch();
    pdl_wait();
    for (int i = 0; i < c.n; ++i) {
        const GvParams& p = c.ph[i];
        if (i > 0) {
            __syncthreads();                  // every warp of this CTA is done with the rings of the phase before
            rg = gv_range(p);
            gv_prefetch(p, rg, smem, full, warp, lane, true, 0, p.nslots);
            if (c.bar) gv_grid_barrier(c.bar, p.status); // ... and every CTA with its rows: the next activation vector is complete
            // (no barrier when every input of the phase arrives as packets: each element carries its own arrival mark)
        }
        gv_phase<false, true, true>(p, smem, full, red, rg, par, wpre, 0, false);
    }
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

// the split of the row groups over `grid` CTAs (gv_range)
static void gv_set_split(GvParams& p, int grid) {
    unsigned long long tot = 0;
    for (int shift = 0;; ++shift) {
        tot = 0;
        for (int i = 0; i < 3; ++i) {
            p.gw[i] = 0; p.ng[i] = 0;
            if (i >= p.nseg || (p.paired_rows && i > 0)) continue;
            const unsigned long long gb = (unsigned long long)p.seg[i].R * p.seg[i].rb >> shift;
            p.gw[i] = p.paired_rows ? 1u : (uint32_t)(gb ? gb : 1);
            p.ng[i] = (uint32_t)((p.seg[i].M + p.seg[i].R - 1) / p.seg[i].R);
            tot += (unsigned long long)p.gw[i] * p.ng[i];
        }
        if (tot < (1ull << 31)) break;
    }
    p.split_q = (uint32_t)(tot / grid); p.split_r = (uint32_t)(tot % grid);
}


// Fills the device-side argument block for one GEMV.  max_warps caps the warps per CTA (a chain runs all its phases
// with one block size); on return smem_bytes / grid hold what this GEMV wants.
// `budget` = dynamic shared memory a CTA may take; `two_per_sm`: a large product may put two of its own CTAs on every SM
// (stream kernel only), small ones leave the second half of the SM to the next kernel.
static int gv_configure(const GemvArgs& a, GvParams& p, int max_warps, int budget, bool two_per_sm, size_t& smem_bytes, int& grid, bool& empty) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    empty = false;
    if (a.nseg < 1 || a.nseg > 3) return set_error(JB_ERR_ARG, "gemv: %d matrices", a.nseg);
    if (a.K <= 0 || a.K % QK_K) return set_error(JB_ERR_ARG, "gemv: K=%d is not a positive multiple of 256", a.K);
    if (!a.x) return set_error(JB_ERR_PTR, "gemv: null activation pointer");
    p = GvParams{};
    p.nseg = a.nseg; p.x = a.x; p.K = a.K; p.out_mode = a.out_mode; p.residual = a.residual; p.residual_pk = (const uint2*)a.residual_pk;
    p.do_norm = a.do_norm; p.norm_w = a.norm_w; p.norm_w_fp32 = a.norm_w_fp32; p.eps = a.eps;
    p.dbg_dots = a.dbg_dots; p.status = cx->d_status; p.xmode = a.xmode ? 1 : 0;
    p.tp_wait_on = a.tp_wait != nullptr; p.tp_push_on = a.tp_push != nullptr;
    if (a.tp_wait) p.tpw = *a.tp_wait;
    if (a.tp_push) p.tpp = *a.tp_push;
    if (p.tp_push_on && (a.out_mode == 1 || a.nseg > 2 || (a.nseg == 2 && a.out_mode != 3)))
        return set_error(JB_ERR_ARG, "gemv: a pushed result must be one fp16 vector");
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
    if (total_rows == 0) { empty = true; return JB_OK; }
    if (a.residual_pk && !a.tp_push) return set_error(JB_ERR_ARG, "gemv: a packet residual needs the push epoch");
    if (a.out_mode == 2 && (a.nseg != 1 || (!a.residual && !a.residual_pk))) return set_error(JB_ERR_ARG, "gemv: residual epilogue needs one matrix and a residual");
    if (a.out_mode == 3 && (a.nseg != 2 || a.seg[0].M != a.seg[1].M || a.seg[0].type != a.seg[1].type))
        return set_error(JB_ERR_ARG, "gemv: SwiGLU epilogue needs two matrices of equal height and type");
    p.paired_rows = a.out_mode == 3;
    const int K = a.K, planes = a.xmode ? 2 : 1;
    // One CTA per SM.  The activation vector is staged once per SM by all the CTA's threads; what is left of the shared
    // memory is split into one staging ring per warp.  Warps per CTA and rows per group are chosen together to
    // minimise the longest chain of work any warp has to run: (row groups of its CTA / warps, rounded up) x
    // (32-lane rounds a group takes, plus half a round of per-group overhead).  Ties go to more warps, larger groups.
    const int U = nb * 4;
    // CTAs of this launch (half an SM each).  A product whose share per SM fits one CTA's rings (Wo, Q/K/V, a 14 MB matrix)
    // launches ONE CTA per SM: the other half of every SM then takes the NEXT kernel's CTAs, which set up and prefetch all
    // their rows while this kernel computes, and few tasks per warp keep the launch short (measured: Wo 4.7 against 6.6 µs,
    // Q/K/V 7.2 against 8.2).  A larger product (gate/up, W_down, logits) launches TWO CTAs per SM: its warps each run
    // several row groups one after the other, and twice the warps shorten that chain more than the overlap would save
    // (gate/up 10.8 against 11.0 µs, W_down 13.2 against 13.9, logits 95 against 116).  JLLM_B200_GEMV_CTAS = 1 / 2 forces either.
    long long all_bytes = 0;
    for (int i = 0; i < a.nseg; ++i) all_bytes += (long long)a.seg[i].M * nb * block_bytes(a.seg[i].type);
    static const int ctas_env = [] { const char* v = getenv("JLLM_B200_GEMV_CTAS"); return v ? atoi(v) : 0; }();
    const bool two = ctas_env ? ctas_env == 2 : all_bytes > (long long)cx->sm_count * (budget - 8192);
    const int ncta = (two_per_sm && two) ? 2 * cx->sm_count : cx->sm_count;
    uint32_t off = 0;
    p.off_xA = off; off += p.needA ? planes * K : 0;
    p.off_xB = off; off += p.needB ? planes * K : 0;
    p.off_xd = off; off += (K / 32) * 4;
    p.off_xs = off; off += (K / 32) * 4;
    p.off_xsum = off; off += p.needB ? (K / 16) * 4 : 0;
    p.off_gate = off;
    off = (off + 127) & ~127u;
    p.off_slots = off;
    static const int warp_choices[] = { 20, 19, 18, 17, 16, 14, 13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2 };
    // Per candidate (warps per CTA, depth): a Q4_K matrix takes `depth` rows per lane — lanes in groups of lw = the row's
    // blocks spread over the fewest passes, lg = 32 / lw groups, so a task holds lg * depth rows; a Q6_K matrix takes
    // `depth` rows per task.  Or one row streamed as C = 2..8 chunks of super-blocks by the same warp (long rows, where even
    // one row does not fit half a ring).  Cost of a candidate = the longest chain of tasks a warp runs, in units of one
    // 64-weight item per lane.  A Q4_K column of 1 / 3 rows costs 4.0 / 4.2: the rows of a column are independent
    // instruction streams that fill each other's latencies (measured per task: 1.3 / 1.35 us).
    // JLLM_B200_GEMV_DEPTH / _WARPS pin either for experiments.
    static const int pin_depth = [] { const char* v = getenv("JLLM_B200_GEMV_DEPTH"); return v ? atoi(v) : 0; }();
    static const int pin_warps = [] { const char* v = getenv("JLLM_B200_GEMV_WARPS"); return v ? atoi(v) : 0; }();
    struct Lane { int lw, lg, rl, rows; };
    auto lane_map = [&](int type, int depth, int blocks) {      // rows per task of a matrix at this depth
        Lane m = { 32, 1, 1, depth };
        if (type == T_Q4K) {
            const int passes = (blocks + 31) / 32;
            m.lw = (blocks + passes - 1) / passes;
            m.lg = 32 / m.lw;
            static const int q4_env = [] { const char* v = getenv("JLLM_B200_GEMV_Q4DEPTH"); return v ? atoi(v) : 0; }();
            m.rl = (q4_env ? q4_env : depth) >= 3 && m.lw >= 3 ? 3 : 1;  // columns are instantiated 1 and 3 rows deep (code size)
            m.rows = m.lg * m.rl;
        }
        return m;
    };
    int best_w = 0, best_R = 0, best_C = 1; double best_cost = 1e30;
    for (int nwarps : warp_choices) {
        if (nwarps > max_warps || (pin_warps && nwarps != pin_warps && pin_warps <= max_warps)) continue;
        const int ring = (budget - (int)off) / nwarps;        // bytes of staging ring per warp
        const int slot_cap = ring / 2;                        // at least two slots per warp
        for (int cand = 4; cand >= -8; --cand) {
            if (cand == 0 || cand == -1) continue;
            const int R = cand > 0 ? cand : 1, C = cand > 0 ? 1 : -cand;
            if (pin_depth && C == 1 && R != pin_depth) continue;
            if (C > 1 && (a.out_mode == 3 || C > nb)) continue;
            const int cb = (nb + C - 1) / C;                  // super-blocks per chunk
            if (C > 1 && (nb + cb - 1) / cb != C) continue;   // this chunk count would leave an empty last chunk
            long long tasks = 0; double work = 0; bool fits = true;
            for (int i = 0; i < (a.out_mode == 3 ? 1 : a.nseg) && fits; ++i) {
                const int type = a.seg[i].type, bbytes = block_bytes(type);
                const Lane m = lane_map(type, C > 1 ? 1 : R, C > 1 ? cb : nb);
                const int rows = C > 1 ? 1 : m.rows;
                const long long task_bytes = (long long)rows * (C > 1 ? cb : nb) * bbytes;
                if (task_bytes + 16 + 127 > slot_cap) { fits = false; break; }
                const long long t = ((long long)a.seg[i].M + rows - 1) / rows;
                const int blocks = C > 1 ? cb : nb;
                static const double column_cost[4] = { 0.0, 4.0, 0.0, 4.2 };
                const double per_task = type == T_Q4K ? ((blocks + m.lw - 1) / m.lw) * column_cost[m.rl] + 0.5
                                                      : (double)((rows * blocks * 4 + 31) / 32) + 0.5;
                tasks += t; work += (double)t * C * per_task;        // the C chunks of a row run one after the other on one warp
            }
            if (!fits || tasks == 0) continue;
            const long long per_cta = (tasks + ncta - 1) / ncta;
            const long long chain = (per_cta + nwarps - 1) / nwarps;
            const double cost = (double)chain * (work / (double)tasks) * (a.out_mode == 3 ? 2 : 1);
            if (cost < best_cost - 1e-9) { best_cost = cost; best_w = nwarps; best_R = R; best_C = C; }
        }
    }
    if (!best_w) return set_error(JB_ERR_LIMIT, "gemv: one row group does not fit the staging ring (K=%d)", K);
    {
        const int nwarps = best_w, R = best_R;
        const int ring = (budget - (int)off) / nwarps;
        p.nchunk = best_C; p.chunk_blocks = (nb + best_C - 1) / best_C;
        int slot = 0;
        p.total_bytes = 0;
        long long groups_total = 0;
        for (int i = 0; i < a.nseg; ++i) {
            GvSegDev& d = p.seg[i];
            d.W = (const uint8_t*)a.seg[i].W; d.y = a.seg[i].y; d.M = a.seg[i].M; d.type = a.seg[i].type;
            d.rb = nb * block_bytes(d.type);
            d.U = U;
            const Lane m = lane_map(d.type, best_C > 1 ? 1 : R, best_C > 1 ? p.chunk_blocks : nb);
            d.lw = (uint8_t)m.lw; d.lg = (uint8_t)(best_C > 1 ? 1 : m.lg); d.rl = (uint8_t)m.rl; d.pad_ = 0;
            d.R = best_C > 1 ? 1 : m.rows;
            const int need = (((best_C > 1 ? p.chunk_blocks * block_bytes(d.type) : d.R * d.rb) + 16 + 127) / 128) * 128;
            slot = need > slot ? need : slot;
            const long long groups = (d.M + d.R - 1) / d.R;
            p.total_bytes += groups * d.R * d.rb;
            groups_total += groups;
        }
        if (ring / slot < 2) return set_error(JB_ERR_LIMIT, "gemv: staging ring too small (K=%d)", K);
        p.slot_bytes = slot;
        p.nslots = ring / slot;
        if (p.nslots > GV_MAXSLOT) p.nslots = GV_MAXSLOT;
        p.nwarps = nwarps;
        static const int early_env = [] { const char* v = getenv("JLLM_B200_GEMV_EARLY"); return v ? atoi(v) : 0; }();
        // two CTAs of this kernel per SM start when the producer is about to finish: half a ring first, the rest behind the
        // activation loads; one CTA per SM starts long before that and fills its whole ring at once
        p.early_slots = early_env > 0 ? (early_env < p.nslots ? early_env : p.nslots) : (two_per_sm && two ? (p.nslots + 1) / 2 : p.nslots);
        smem_bytes = (size_t)p.off_slots + (size_t)nwarps * p.nslots * slot;
        if (p.paired_rows) groups_total /= 2;
        grid = ncta;                                           // every SM streams its share, however few groups that is
        if (grid > groups_total) grid = (int)groups_total;
        if (grid < 1) grid = 1;
        gv_set_split(p, grid);
        static const bool verbose = getenv("JLLM_B200_GEMV_DEBUG") != nullptr;
        if (verbose)
            fprintf(stderr, "[gemv] K=%d nseg=%d M0=%d type0=%d xmode=%d out=%d: grid %d x %d warps, depth %d (rows/task %d, lanes %d x %d), chunks=%d x %d blocks, %d slots of %d B, smem %zu\n",
                    K, a.nseg, a.seg[0].M, a.seg[0].type, a.xmode, a.out_mode, grid, nwarps, R, p.seg[0].R, p.seg[0].lg, p.seg[0].lw, p.nchunk, p.chunk_blocks, p.nslots, p.slot_bytes, smem_bytes);
        return JB_OK;
    }
}

int launch_gemv(const GemvArgs& a0, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    GemvArgs a = a0;
    if (g_tp_wait_set && !a.tp_wait) a.tp_wait = &g_tp_wait;
    if (g_tp_push_set && !a.tp_push) a.tp_push = &g_tp_push;
    g_tp_wait_set = g_tp_push_set = false;
    GvParams p;
    size_t smem_bytes = 0; int grid = 0; bool empty = false;
    const int cap = GV_MAXWARPS;
    const int rc = gv_configure(a, p, cap, cx->gemv_smem_budget, true, smem_bytes, grid, empty);
    if (rc || empty) return rc;
    p.trace = g_trace; g_trace = nullptr;
    static const bool nocompute = getenv("JLLM_B200_GEMV_NOCOMPUTE") != nullptr;
    p.trace_nocompute = (p.trace && nocompute) ? 1 : 0;
    const bool dbg = a.dbg_dots || p.trace;
    const bool tp = a.tp_wait || a.tp_push || a.residual_pk;
    if (dbg && tp) return set_error(JB_ERR_ARG, "gemv: no debug output on a tensor-parallel launch");
    // ONE kernel function serves every single-GPU GEMV of a decode step (both activation formats, both weight types): the
    // launches of a layer alternate between as few functions as possible, and their code stays in the instruction cache.
    void (*kern)(GvParams) = dbg ? gemv_stream_kernel<true, false> : (tp ? gemv_stream_kernel<false, true> : gemv_stream_kernel<false, false>);
    const int ki = dbg ? 1 : (tp ? 2 : 0);
    if (!cx->gemv_attr[ki]) {
        JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cx->gemv_smem_budget));
        JB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
        cx->gemv_attr[ki] = true;
    }
    // warps beyond p.nwarps only help to stage the activation vector (eight elements per thread and round) and leave
    int block_warps = (a.K / 8 + 31) / 32;
    block_warps = block_warps > cap ? cap : block_warps;
    block_warps = block_warps < p.nwarps ? p.nwarps : block_warps;
    JB_CUDA(launch_k(kern, dim3(grid), dim3(block_warps * 32), smem_bytes, st, pdl_enabled(), p));
    count_launch();
    return JB_OK;
}

// Up to four GEMVs, each reading what the one before wrote, in one launch (gemv_chain_kernel).  `bar` = two zeroed
// device words owned by the caller and used by one chain at a time.
int launch_gemv_chain(const GemvArgs* args, int n, unsigned int* bar, cudaStream_t st) {
    DeviceCtx* cx = ctx();
    if (!cx) return JB_ERR_CUDA;
    if (n < 1 || n > 4) return set_error(JB_ERR_ARG, "gemv chain: %d phases", n);
    for (int i = 1; i < n && !bar; ++i)
        if (!args[i].tp_wait || (args[i].out_mode == 2 && !args[i].residual_pk))
            return set_error(JB_ERR_ARG, "gemv chain: without a grid barrier every input of a later phase must arrive as packets");
    GvChain c;
    c.n = n; c.bar = bar;
    size_t smem_max = 0;
    for (int i = 0; i < n; ++i) {
        if (args[i].dbg_dots) return set_error(JB_ERR_ARG, "gemv chain: no debug output");
        size_t smem_bytes = 0; int grid = 0; bool empty = false;
        const int rc = gv_configure(args[i], c.ph[i], GV_CHAINWARPS, cx->max_smem_optin - 2048, false, smem_bytes, grid, empty);
        if (rc) return rc;
        if (empty) return set_error(JB_ERR_ARG, "gemv chain: empty phase");
        c.ph[i].chained = 1; c.ph[i].early_slots = c.ph[i].nslots;
        gv_set_split(c.ph[i], cx->sm_count);   // the chain's grid
        smem_max = smem_bytes > smem_max ? smem_bytes : smem_max;
    }
    if (!cx->gemv_chain_attr) {
        JB_CUDA(cudaFuncSetAttribute(gemv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cx->max_smem_optin - 2048));
        cx->gemv_chain_attr = true;
    }
    // every phase splits its rows over the same grid: one CTA per SM, all resident together
    JB_CUDA(launch_k(gemv_chain_kernel, dim3(cx->sm_count), dim3(GV_CHAINTHREADS), smem_max, st, pdl_enabled(), c));
    count_launch();
    return JB_OK;
}

}  // namespace jb
