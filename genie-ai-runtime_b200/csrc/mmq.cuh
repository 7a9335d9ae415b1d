// mmq.cuh — prefill / batched K-quant GEMM launchers.
#pragma once
#include "common.cuh"

namespace jb {

// y[N x M] half (token-major) = x[N x K] half . W^T, W in Q4_K / Q6_K blocks, with the
// arithmetic of the reference's default prefill path (gemm_quant_batched,
// src/kernels/gemv_q4.cu:2478-2495 -> mmq_q4k_llama.cu / mmq_q6k_llama.cu).
// dbg_dots (optional): integer accumulators [N][M][K/32] (Q4_K) or [N][M][K/16] (Q6_K).
int launch_mmq(__half* y, const void* W, int type, const __half* x, int M, int N, int K, int32_t* dbg_dots, cudaStream_t st);
// the same with a residual added on the way out (y = half(float(residual) + float(half(product))), residual [N][M] or null)
// and, for a second matrix multiplied by the SAME activations right after the first on this stream, `same_x_as_last`
int launch_mmq_ex(__half* y, const void* W, int type, const __half* x, int M, int N, int K, const __half* residual, bool same_x_as_last,
                  cudaStream_t st);
int launch_mmq_pair(__half* y1, __half* y2, const void* W1, int type1, const void* W2, int type2, const __half* x, int M1, int M2, int N, int K,
                    cudaStream_t st);
size_t mmq_scratch_bytes(int N, int K);
// tensor-core path (mmq_tc.cu): tcgen05.mma over fp16 operands built from the same quantised values
bool   mmq_tc_applies(const void* W, int type, int M, int N, int K);
size_t mmq_tc_scratch_bytes(int type, int M, int N, int K);
int    launch_mmq_tc(__half* y, const void* W, int type, const __half* x, __half* xq, int M, int N, int K, bool same_x_as_last, cudaStream_t st);
int    launch_mmq_tc_pair(__half* y, __half* y2, const void* W, const void* W2, int type, const __half* x, __half* xq, int M, int M2, int N, int K,
                          bool same_x_as_last, cudaStream_t st);
size_t mmq_tc_scratch_bytes_pair(int type, int M, int M2, int N, int K);
void*  mmq_scratch(size_t bytes, bool may_alloc);
// few tokens (2..64): weights streamed once, mma.sync on fp16 operands with the tensor-core path's arithmetic (mmq_stream.cu)
bool   mmq_stream_applies(const void* W, int type, int M, int N, int K);
size_t mmq_stream_scratch_bytes(int type, int M, int N, int K);
int    launch_mmq_stream(__half* y, const void* W, int type, const __half* x, void* scratch, int M, int N, int K, const __half* residual,
                         bool reuse_operand, cudaStream_t st);

}  // namespace jb
