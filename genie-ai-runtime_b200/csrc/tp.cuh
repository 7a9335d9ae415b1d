// tp.cuh — tensor-parallel exchange: device-visible description of the rank group and the launchers.
#pragma once
#include "common.cuh"
#include <cstring>

namespace jb {

constexpr int TP_MAX_WORLD = 8;
constexpr int TP_POINTS = 5;                 // attention out, x after Wo, SwiGLU out, x after W_down, argmax
constexpr int TP_POINT_ATT = 0, TP_POINT_X2 = 1, TP_POINT_SW = 2, TP_POINT_X = 3, TP_POINT_ARGMAX = 4;
constexpr uint32_t TP_WAIT_POLLS = 1u << 22;  // x 64 ns sleep: a quarter of a second at least before a wait gives up

struct TpDev {
    unsigned char* peer[TP_MAX_WORLD];       // exchange regions of all ranks, mapped into this process (own at [rank])
    int rank, world;
    int flags_off, argmax_off;               // byte offsets inside a region
    int epochs_per_step;                     // = number of layers: each exchange point is used once per layer
    uint32_t* seq;                           // device step counter (never reset)
    int* status;                             // device status word
};

// Region layout (all ranks identical): full-size packet vectors (8 bytes per element) att [q_dim], x2 [hidden],
// sw [intermediate], x [hidden], each 256-byte aligned, then TP_POINTS x TP_MAX_WORLD flag words, then the argmax slots (values, indices).
// Returns the region size; offs (optional) receives {att, x2, sw, x, flags, argmax}.
inline size_t tp_region_layout(int hidden, int q_dim, int inter, int* offs) {
    auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
    size_t o = 0;
    const size_t a = o; o += al((size_t)q_dim * 8);
    const size_t b = o; o += al((size_t)hidden * 8);
    const size_t c = o; o += al((size_t)inter * 8);
    const size_t d = o; o += al((size_t)hidden * 8);
    const size_t f = o; o += al((size_t)TP_POINTS * TP_MAX_WORLD * 4);
    const size_t g = o; o += al((size_t)TP_MAX_WORLD * 8);
    if (offs) { offs[0] = (int)a; offs[1] = (int)b; offs[2] = (int)c; offs[3] = (int)d; offs[4] = (int)f; offs[5] = (int)g; }
    return o;
}

int launch_tp_push(const TpDev& tp, const void* src, int n, int buf_off, int elem_off, int layer, cudaStream_t st);
int launch_tp_unpack(const TpDev& tp, void* dst, int n, int buf_off, int layer, cudaStream_t st);
int launch_tp_argmax(const TpDev& tp, const float* logits, int n_local, int* state, int* out, int out_cap, cudaStream_t st);

}  // namespace jb
