// gemv.cuh — host-side argument block of the streaming K-quant GEMV.
#pragma once
#include "common.cuh"

namespace jb {

struct GemvSeg { const void* W; void* y; int M; int type; };

// One launch computes up to three projections that share one activation vector
// (the reference's gemv_quant / _pair / _triple / _add / _f32 family,
// src/kernels/gemv_q4.cu:2633-2775).
struct GemvArgs {
    GemvSeg seg[3];
    int nseg = 1;
    const __half* x = nullptr;
    int K = 0;
    // 0: activations quantised to q8_1 codes, integer dots (reference dp4a path);
    // 1: activations kept as 16-bit fixed point, integer dots (stands in for the
    //    reference's fp16-x float path: same mathematics, no 8-bit activation rounding).
    int xmode = 0;
    int out_mode = 0;                 // 0 half, 1 float, 2 half(half(acc)+residual), 3 silu(seg0)*seg1 -> seg0.y
    const __half* residual = nullptr; // out_mode 2
    // optional fused input RMSNorm: x := half((x [+ norm_res]) * rrms * w) before quantising
    int do_norm = 0;
    const void* norm_w = nullptr; int norm_w_fp32 = 1; float eps = 0.f;
    int32_t* dbg_dots = nullptr;      // optional: integer accumulators of seg 0
};

// Tensor-parallel hooks of one launch (csrc/tp.cu describes the exchange).  `wait`: before the activation vector is
// read, flags[0..world) of this rank's own region must have reached the epoch seq[0]*epochs_per_step + layer + 1.
// `push`: seg.y must point at rows [row_off, row_off + rows) of the fp16 vector at buf_off in this rank's OWN region;
// the last CTA to finish copies that slice to the same place in every other region and raises this rank's flag in
// every region.  rows and row_off must be multiples of 8 (16-byte copies).
struct GemvTpWait { const uint32_t* flags; int world; const uint32_t* seq; int epochs_per_step; int layer; };
struct GemvTpPush {
    unsigned char* peer[8]; int world, rank; int buf_off; int row_off, rows; int flag_off;      // flag_off: byte offset of this rank's flag word
    const uint32_t* seq; int epochs_per_step; int layer; unsigned int* counter;     // counter: zeroed device word, one per exchange point
};
// The next launch_gemv on this thread takes the hooks (either may be null) and forgets them.
void gemv_set_tp_hooks(const GemvTpWait* wait, const GemvTpPush* push);

int launch_gemv(const GemvArgs& a, cudaStream_t st);
int launch_gemv_q5k(__half* y, float* y32, const void* W, const __half* x, const __half* residual,
                    int M, int K, cudaStream_t st);

}  // namespace jb
