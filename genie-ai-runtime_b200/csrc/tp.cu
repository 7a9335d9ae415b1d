// tp.cu — the exchange step of tensor-parallel decode: one process per GPU, every rank owns a contiguous slice of
// the output rows of each weight matrix and the KV heads that go with them, and after each sharded product the
// slices are gathered into a full vector on every GPU.
//
// The reference is single-GPU; the sharding follows its data layout (a row slice of a GGUF matrix is a contiguous
// byte range; KV heads are independent in flash_attention_decode, src/kernels/attention.cu:626-760).
//
// Mechanism: every rank holds one exchange region (plain cudaMalloc memory, opened by the peers through CUDA
// IPC) with one packet vector per exchange point.  A packet is 8 bytes, {fp16 value, epoch}, written with one 64-bit
// store; a rank PUSHES each element it produces into the same slot of every rank's region over NVLink (from the
// epilogue of the GEMV that computes it, or from tp_push_kernel for the attention output) and never waits.  A
// consumer polls the packets of its OWN region while it stages its activation vector: an element is there exactly
// when its epoch word matches.  No fence, no flag and no round trip are on the path, remote data always lands in
// local HBM before it is read, and no TMA touches peer memory.  Only the sharded greedy argmax still uses flag words.
//
// Epochs come from a device-side step counter (epoch = step * layers + layer + 1), so the same captured graph
// serves every step.  A vector is rewritten one layer later, and a rank can only get there after every peer has
// pushed a later exchange, i.e. after the peer's reader of the previous contents has finished.
//
// Every wait is bounded: when it runs out the kernel records JB_ERR_TIMEOUT in the status word and returns.
#include "tp.cuh"

namespace jb {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// waits (bounded) until flags[0..world) of exchange point `point` in this rank's own region have reached `epoch`
__device__ __forceinline__ bool tp_wait_flags(const TpDev& tp, int point, uint32_t epoch, int tid) {
    bool ok = true;
    if (tid < tp.world) {
        const uint32_t* f = reinterpret_cast<const uint32_t*>(tp.peer[tp.rank] + tp.flags_off) + point * TP_MAX_WORLD + tid;
        PollGuard guard(tp.status);
        while (ld_acquire_sys(f) < epoch)
            if (!guard.again(tp.status, 64, TP_WAIT_POLLS)) { ok = false; break; }
    }
    return ok;
}

// fp16 slice -> packets in every rank's region (elements [elem_off, elem_off + n) of the vector at buf_off)
__global__ void __launch_bounds__(256) tp_push_kernel(TpDev tp, const __half* src, int n, int buf_off, int elem_off, int layer) {
    pdl_wait();
    const uint32_t epoch = tp.seq[0] * (uint32_t)tp.epochs_per_step + (uint32_t)layer + 1u;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const uint2 pkt = make_uint2((uint32_t)__half_as_ushort(src[i]), epoch);
        for (int r = 0; r < tp.world; ++r) reinterpret_cast<uint2*>(tp.peer[r] + buf_off)[elem_off + i] = pkt;
    }
}
// packets of this rank's own region -> plain fp16 vector (bounded poll per element)
__global__ void __launch_bounds__(256) tp_unpack_kernel(TpDev tp, __half* dst, int n, int buf_off, int layer) {
    pdl_wait();
    const uint32_t epoch = tp.seq[0] * (uint32_t)tp.epochs_per_step + (uint32_t)layer + 1u;
    const uint2* src = reinterpret_cast<const uint2*>(tp.peer[tp.rank] + buf_off);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint2 q;
        PollGuard guard(tp.status);
        for (;;) {
            q = __ldcv(src + i);
            if (q.y == epoch || !guard.again(tp.status, 32, TP_WAIT_POLLS)) break;
        }
        dst[i] = __ushort_as_half((unsigned short)(q.x & 0xFFFFu));
    }
}

// Greedy sampling over sharded logits: local argmax (lowest index among equal maxima, non-finite skipped, as the
// single-GPU kernel), exchange of (value, global index), the same reduction on every rank, then the step state
// advances exactly as in argmax_advance_kernel.
__global__ void __launch_bounds__(1024) tp_argmax_advance_kernel(TpDev tp, const float* logits, int n_local, int* state, int* out, int out_cap) {
    pdl_wait();
    __shared__ float sv[32]; __shared__ int si[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float best = -INFINITY; int bi = 0x7FFFFFFF;
    for (int i = tid; i < n_local; i += blockDim.x) {
        const float v = logits[i];
        if (isfinite(v) && (v > best || (v == best && i < bi))) { best = v; bi = i; }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o); const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    const uint32_t epoch = tp.seq[0] + 1u;
    if (tid == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
        const int gi = bi == 0x7FFFFFFF ? 0x7FFFFFFF : bi + tp.rank * n_local;
        for (int r = 0; r < tp.world; ++r) {
            float* pv = reinterpret_cast<float*>(tp.peer[r] + tp.argmax_off) + tp.rank;
            int* pi = reinterpret_cast<int*>(tp.peer[r] + tp.argmax_off + TP_MAX_WORLD * 4) + tp.rank;
            *pv = best; *pi = gi;
        }
        __threadfence_system();
        for (int r = 0; r < tp.world; ++r)
            st_release_sys(reinterpret_cast<uint32_t*>(tp.peer[r] + tp.flags_off) + TP_POINT_ARGMAX * TP_MAX_WORLD + tp.rank, epoch);
    }
    __syncthreads();
    const bool ok = tp_wait_flags(tp, TP_POINT_ARGMAX, epoch, tid);
    if (!ok) atomicExch(tp.status, JB_ERR_TIMEOUT);
    __syncthreads();
    if (tid == 0) {
        const volatile float* pv = reinterpret_cast<const volatile float*>(tp.peer[tp.rank] + tp.argmax_off);
        const volatile int* pi = reinterpret_cast<const volatile int*>(tp.peer[tp.rank] + tp.argmax_off + TP_MAX_WORLD * 4);
        float gb = -INFINITY; int gidx = 0x7FFFFFFF;
        for (int r = 0; r < tp.world; ++r) {
            const float v = pv[r]; const int i = pi[r];
            if (i != 0x7FFFFFFF && (v > gb || (v == gb && i < gidx))) { gb = v; gidx = i; }
        }
        if (gidx == 0x7FFFFFFF) gidx = 0;
        const int k = state[2];
        if (out && k < out_cap) out[k] = gidx;
        state[2] = k + 1;
        state[1] = gidx;
        state[0] = state[0] + 1;
        tp.seq[0] = tp.seq[0] + 1u;          // last use of the epoch of this step
    }
}

int launch_tp_push(const TpDev& tp, const void* src, int n, int buf_off, int elem_off, int layer, cudaStream_t st) {
    if (n <= 0) return JB_OK;
    JB_CUDA(launch_k(tp_push_kernel, dim3((n + 255) / 256 > 8 ? 8 : (n + 255) / 256), dim3(256), 0, st, pdl_enabled(), tp, (const __half*)src, n, buf_off, elem_off, layer));
    count_launch();
    return JB_OK;
}
int launch_tp_unpack(const TpDev& tp, void* dst, int n, int buf_off, int layer, cudaStream_t st) {
    JB_CUDA(launch_k(tp_unpack_kernel, dim3((n + 255) / 256 > 8 ? 8 : (n + 255) / 256), dim3(256), 0, st, pdl_enabled(), tp, (__half*)dst, n, buf_off, layer));
    count_launch();
    return JB_OK;
}

int launch_tp_argmax(const TpDev& tp, const float* logits, int n_local, int* state, int* out, int out_cap, cudaStream_t st) {
    JB_CUDA(launch_k(tp_argmax_advance_kernel, dim3(1), dim3(1024), 0, st, pdl_enabled(), tp, logits, n_local, state, out, out_cap));
    count_launch();
    return JB_OK;
}

}  // namespace jb

using namespace jb;

extern "C" {

void* jllm_b200_tp_alloc(size_t bytes) {
    if (!ctx()) return nullptr;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaMalloc(exchange region)"); return nullptr; }
    cudaMemset(p, 0, bytes);
    cudaDeviceSynchronize();
    return p;
}
int jllm_b200_tp_free(void* p) { JB_CUDA(cudaFree(p)); return JB_OK; }
int jllm_b200_tp_export(void* p, void* handle64) {
    cudaIpcMemHandle_t h;
    JB_CUDA(cudaIpcGetMemHandle(&h, p));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    return JB_OK;
}
void* jllm_b200_tp_open(const void* handle64) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaIpcOpenMemHandle"); return nullptr; }
    return p;
}
int jllm_b200_tp_close(void* p) { JB_CUDA(cudaIpcCloseMemHandle(p)); return JB_OK; }
size_t jllm_b200_tp_region_bytes(int hidden_dim, int q_dim, int intermediate_dim) {
    return tp_region_layout(hidden_dim, q_dim, intermediate_dim, nullptr);
}

}  // extern "C"
