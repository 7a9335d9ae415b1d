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
    const void* residual_pk = nullptr; // out_mode 2, tensor-parallel chain: the residual rows as packets in this rank's own region
    // optional fused input RMSNorm: x := half((x [+ norm_res]) * rrms * w) before quantising
    int do_norm = 0;
    const void* norm_w = nullptr; int norm_w_fp32 = 1; float eps = 0.f;
    int32_t* dbg_dots = nullptr;      // optional: integer accumulators of seg 0
    const struct GemvTpWait* tp_wait = nullptr;   // tensor-parallel hooks (see below); null on one GPU
    const struct GemvTpPush* tp_push = nullptr;
};

// Tensor-parallel hooks of one launch (csrc/tp.cu describes the exchange).  Exchanged vectors travel as 8-byte
// packets {fp16 value in the low half of word 0, epoch in word 1}, one packet per element, written with single
// 64-bit stores: a packet is valid exactly when its epoch word equals the epoch of this exchange
// (seq[0]*epochs_per_step + layer + 1), so neither a fence nor a flag is needed and the transfer costs one
// one-way trip over NVLink.
// `wait`: GemvArgs.x points at a packet vector in this rank's own region; the staging pass polls every packet
// (bounded) instead of waiting for the previous kernel only.
// `push`: besides seg.y (this rank's plain fp16 slice, kept for the residual of a later kernel) every finished row
// is sent as a packet to element row_off + row of the vector at buf_off in EVERY rank's region.
struct GemvTpWait { const uint32_t* seq; int epochs_per_step; int layer; };
struct GemvTpPush { unsigned char* peer[8]; int world; int buf_off; int row_off; const uint32_t* seq; int epochs_per_step; int layer; };
// The next launch_gemv on this thread takes the hooks (either may be null) and forgets them.
void gemv_set_tp_hooks(const GemvTpWait* wait, const GemvTpPush* push);

// dispatch helpers shared with the decoder's chained launches (csrc/api.cu)
const void* resolve_weight(const void* W);          // device pointer of a weight tensor (registered host ranges are mapped)
bool triple_dp4a(int t0, int t1, int t2);            // type mixes the reference runs on its q8_1 + dp4a path

int launch_gemv(const GemvArgs& a, cudaStream_t st);
// Diagnostic: the next launch_gemv on this thread records GV_NTRACE (16) %globaltimer stamps per CTA into t[cta * 16 + k]:
// 0 kernel entry, 1 first bulk copies issued, 2 producer kernel complete (griddepcontrol.wait returned), 3 activation
// vector staged, 4 first row group landed, 5 warp 0 done, 6 last warp done, 8 + 2u / 9 + 2u: task u (< 4) of warp 0 has
// landed / has been multiplied.
void gemv_set_trace(unsigned long long* t);
// n <= 4 GEMVs that feed one another, in one launch with grid-wide barriers between them; bar: two zeroed device words,
// or null when every later phase takes all its inputs as packets (tensor-parallel): packets carry their own arrival mark
int launch_gemv_chain(const GemvArgs* args, int n, unsigned int* bar, cudaStream_t st);
int launch_gemv_q5k(__half* y, float* y32, const void* W, const __half* x, const __half* residual,
                    int M, int K, cudaStream_t st);

}  // namespace jb
