// common.cuh — shared device/host helpers of the B200 kernel library.
//
// Block formats follow GGUF as the reference re-declares them
// (src/kernels/gemv_q4.cu:141-164): Q4_K 144 B, Q5_K 176 B, Q6_K 210 B per 256 weights.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>

namespace jb {

constexpr int QK_K      = 256;
constexpr int Q4K_BYTES = 144;
constexpr int Q5K_BYTES = 176;
constexpr int Q6K_BYTES = 210;
constexpr int T_Q4K = 12, T_Q5K = 13, T_Q6K = 14;

__host__ __device__ inline int block_bytes(int t) {
    return t == T_Q4K ? Q4K_BYTES : t == T_Q5K ? Q5K_BYTES : t == T_Q6K ? Q6K_BYTES : 0;
}

// ── error channel (host) ────────────────────────────────────────────────
// The reference logs and falls back to a CPU path; this library has no CPU path, so
// every entry point records a retrievable error instead (and zero-fills its output
// where the reference does).
enum : int {
    JB_OK = 0, JB_ERR_ARG = 1, JB_ERR_TYPE = 2, JB_ERR_PTR = 3, JB_ERR_CUDA = 4,
    JB_ERR_NOMEM = 5, JB_ERR_LIMIT = 6, JB_ERR_TIMEOUT = 7, JB_ERR_STATE = 8,
};
int  set_error(int code, const char* fmt, ...);
int  cuda_error(cudaError_t e, const char* what);
#define JB_CUDA(call)                                                     \
    do { cudaError_t e__ = (call); if (e__ != cudaSuccess) return ::jb::cuda_error(e__, #call); } while (0)

// ── per-device context ──────────────────────────────────────────────────
// Library-owned scratch is per device (the reference keeps process-global statics,
// src/kernels/gemv_q4.cu:1309-1321, attention.cu:975-988, rope.cu:29-40).
struct RopeTable { float theta; int half_dim; int max_seq; float* cos; float* sin; };
struct DeviceCtx {
    int   device = -1;
    int   sm_count = 0;
    int   max_smem_optin = 0;
    int*  d_status = nullptr;           // device status word written by bounded waits
    float* splitk = nullptr; size_t splitk_floats = 0;
    void*  mmq_act = nullptr; size_t mmq_act_bytes = 0;
    RopeTable rope[8]; int n_rope = 0;
    bool gemv_attr[12] = {};
    bool mms_attr[8] = {};
    // the activation operand the few-token GEMM quantised last (see launch_mmq_stream: reuse_operand)
    const void* mms_op_x = nullptr; void* mms_op_scratch = nullptr; void* mms_op_stream = nullptr; int mms_op_n = 0, mms_op_k = 0, mms_op_ds4 = -1;
    const void* tc_op_x = nullptr; void* tc_op_xq = nullptr; void* tc_op_stream = nullptr; int tc_op_n = 0, tc_op_k = 0, tc_op_ds4 = -1;   // the same for the tensor-core GEMM's operand
    bool gemv_chain_attr = false;
    bool attn_tma_attr[6] = { false, false, false, false, false, false };
    bool attn_prefill_attr[3] = { false, false, false };
    unsigned int* attn_tickets = nullptr;   // ATTN_TICKET_WORDS zeroed words: slice counters of the TMA attention kernel
    int  gemv_smem_budget = 0;          // dynamic shared memory of a GEMV CTA that shares its SM with one other CTA
};
constexpr int ATTN_TICKET_WORDS = 65536;
DeviceCtx* ctx();                        // context of the current device (created on first use)

// ── device helpers ──────────────────────────────────────────────────────
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself block for a
// hardware-defined short interval) and reports false; callers set the status word
// and return instead of spinning forever.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}
// Bounded in polls AND in time (2 s): a poll may itself block for a hardware-defined interval, so a poll count alone
// does not bound the wait.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    unsigned long long t0 = 0;
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 4) __nanosleep(40);          // back off: waiting warps must not crowd the issue slots of working ones
        if ((i & 63) == 63) {
            const unsigned long long t = global_ns();
            if (!t0) t0 = t; else if (t - t0 > 2000000000ull) return false;
        }
    }
    return false;
}
// Guard of a polling loop on memory that another rank (or CTA) writes.  The wait is given up — and JB_ERR_TIMEOUT
// recorded in the status word — after `max_polls` polls or `max_ns` nanoseconds, whichever comes first.  A wait that
// starts when the status word already holds a timeout gives up at its first miss: once one wait of a step has run
// out, the later waits of that step (every element, kernel and layer behind it) must not each spin their full bound
// again, so a dead peer costs one bound per step, not one per wait.
struct PollGuard {
    unsigned long long t0 = 0;
    uint32_t polls = 0;
    bool dead;
    __device__ __forceinline__ explicit PollGuard(const int* status) {
        dead = *reinterpret_cast<const volatile int*>(status) == JB_ERR_TIMEOUT;
    }
    // call after a miss; false = stop waiting and use whatever is there
    __device__ __forceinline__ bool again(int* status, uint32_t sleep_ns = 20, uint32_t max_polls = (1u << 21), unsigned long long max_ns = 500000000ull) {
        if (dead) return false;
        if ((++polls & 63u) == 0u) {
            const unsigned long long t = global_ns();
            if (!t0) t0 = t;
            else if (t - t0 > max_ns) polls = max_polls;
        }
        if (polls >= max_polls) { atomicExch(status, JB_ERR_TIMEOUT); dead = true; return false; }
        __nanosleep(sleep_ns);
        return true;
    }
};
// 1-D bulk copy global -> shared through the TMA unit; both addresses 16-byte aligned,
// size a multiple of 16 bytes; completion is signalled on `bar` by byte count.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Programmatic dependent launch: wait for the producer grid's memory / let dependents start.
__device__ __forceinline__ void pdl_wait()   { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d; asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    int d; asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ float warp_sum(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float h2f_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// 6-bit scale / min j (0..7) of a Q4_K/Q5_K block from its three packed scale words
// (bytes 0-3, 4-7, 8-11 of scales[12]; layout per src/kernels/gemv_q4.cu:185-195).
__device__ __forceinline__ void scale_min_k4(int j, uint32_t s0, uint32_t s1, uint32_t s2, int& sc, int& mn) {
    const int sh = 8 * (j & 3);
    if (j < 4) { sc = (s0 >> sh) & 63; mn = (s1 >> sh) & 63; }
    else {
        sc = ((s2 >> sh) & 0xF) | (((s0 >> (sh + 6)) & 3) << 4);
        mn = ((s2 >> (sh + 4)) & 0xF) | (((s1 >> (sh + 6)) & 3) << 4);
    }
}
#endif  // __CUDACC__

// Launch with the programmatic-dependent-launch attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

bool pdl_enabled();          // process-wide switch (default on)
void count_launch(int n = 1);  // launch counter for the benchmark's gpu_launches claim

}  // namespace jb
