// api.cu — library state, dispatch, and the two faces of the boundary:
//   * C++ symbols in namespace jllm (identical mangling to the reference's include/jllm_kernels.h)
//   * extern "C" mirrors with status returns (include/jllm_b200.h)
// Dispatch rules (which arithmetic an entry point uses) follow the reference's dispatchers:
// src/kernels/gemv_q4.cu:1245-1616 and :2478-2517.
#include "../../include/jllm_b200_api.hpp"
#include "../../include/jllm_b200.h"
#include "common.cuh"
#include "gemv.cuh"
#include "elementwise.cuh"
#include "attention.cuh"
#include "mmq.cuh"
#include <atomic>
#include <new>
#include <vector>
#include <cstdarg>
#include <cstring>
#include <mutex>

namespace jb {

// ── error channel ─────────────────────────────────────────────────────────
static thread_local char g_err[512] = "";
static thread_local int  g_err_code = 0;
int set_error(int code, const char* fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    g_err_code = code;
    return code;
}
int cuda_error(cudaError_t e, const char* what) {
    cudaGetLastError();
    return set_error(JB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// ── contexts ──────────────────────────────────────────────────────────────
static DeviceCtx g_ctx[16];
static std::mutex g_ctx_mu;
DeviceCtx* ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaGetDevice"); return nullptr; }
    if (dev < 0 || dev >= 16) { set_error(JB_ERR_LIMIT, "device ordinal %d out of range", dev); return nullptr; }
    DeviceCtx* c = &g_ctx[dev];
    if (c->device == dev) return c;
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (c->device == dev) return c;
    cudaDeviceProp pr;
    if (cudaGetDeviceProperties(&pr, dev) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaGetDeviceProperties"); return nullptr; }
    if (pr.major != 10) { set_error(JB_ERR_STATE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, pr.major, pr.minor); return nullptr; }
    c->sm_count = pr.multiProcessorCount;
    c->max_smem_optin = (int)pr.sharedMemPerBlockOptin;
    // two CTAs per SM: half the SM's shared memory each, minus the per-CTA system reservation and 2 KB of static arrays
    c->gemv_smem_budget = (int)(pr.sharedMemPerMultiprocessor / 2 - pr.reservedSharedMemPerBlock) - 2048;
    c->gemv_smem_budget &= ~127;
    if (cudaMalloc(&c->d_status, 256) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaMalloc(status)"); return nullptr; }
    cudaMemset(c->d_status, 0, 256);
    if (cudaMalloc(&c->attn_tickets, ATTN_TICKET_WORDS * sizeof(unsigned int)) != cudaSuccess) { cuda_error(cudaGetLastError(), "cudaMalloc(tickets)"); return nullptr; }
    cudaMemset(c->attn_tickets, 0, ATTN_TICKET_WORDS * sizeof(unsigned int));
    c->device = dev;
    return c;
}

static std::atomic<long long> g_launches{0};
static std::atomic<int> g_pdl{1};
void count_launch(int n) { g_launches += n; }
bool pdl_enabled() { return g_pdl.load() != 0; }

// ── weight pointer resolution (gemv_q4.cu:105-128, model.cpp:39-66) ─────────
struct MappedRegion { const char* host; const char* dev; int64_t bytes; };
static MappedRegion g_region = { nullptr, nullptr, 0 };
static const void* g_ok_cache[64];

const void* resolve_weight(const void* W) {
    if (!W) return nullptr;
    if (g_region.host && g_region.dev) {
        const char* p = (const char*)W;
        if (p >= g_region.host && p < g_region.host + g_region.bytes) return g_region.dev + (p - g_region.host);
    }
    const size_t slot = ((uintptr_t)W >> 8) & 63;
    if (g_ok_cache[slot] == W) return W;
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, W) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) { g_ok_cache[slot] = W; return W; }
    return nullptr;
}

static int zero_fill(void* y, size_t bytes, cudaStream_t st) { if (y && bytes) cudaMemsetAsync(y, 0, bytes, st); return 0; }

// ── GEMV family ─────────────────────────────────────────────────────────
static bool is_k(int t) { return t == T_Q4K || t == T_Q5K || t == T_Q6K; }

// one projection; mode: 0 = half out (gemv_quant), 1 = fp32 out, 2 = + residual
static int gemv_one(void* y, const void* W, int type, const __half* x, const __half* residual, int M, int K, int mode,
                    int32_t* dbg, cudaStream_t st) {
    const size_t ybytes = (size_t)(M > 0 ? M : 0) * (mode == 1 ? 4 : 2);
    if (M <= 0) return JB_OK;
    if (!is_k(type)) { zero_fill(y, ybytes, st); return set_error(JB_ERR_TYPE, "unsupported ggml type %d (M=%d K=%d)", type, M, K); }
    const void* Wd = resolve_weight(W);
    if (!Wd) { zero_fill(y, ybytes, st); return set_error(JB_ERR_PTR, "weight pointer %p is not device-visible", W); }
    if (type == T_Q5K) {
        if (K <= 0 || K % QK_K) return set_error(JB_ERR_ARG, "gemv: K=%d", K);
        return launch_gemv_q5k(mode == 1 ? nullptr : (__half*)y, mode == 1 ? (float*)y : nullptr, Wd, x, mode == 2 ? residual : nullptr, M, K, st);
    }
    GemvArgs a;
    a.nseg = 1; a.seg[0] = GemvSeg{ Wd, y, M, type };
    a.x = x; a.K = K; a.dbg_dots = dbg;
    if (mode == 0)      { a.xmode = 0; a.out_mode = 0; }                                // Q4_K / Q6_K: q8_1 + integer dots
    else if (mode == 1) { a.xmode = type == T_Q4K ? 0 : 1; a.out_mode = 1; }           // logits: Q4_K dp4a, Q6_K fp16-x arithmetic
    else                { a.xmode = 1; a.out_mode = 2; a.residual = residual; }         // residual exits: fp16-x arithmetic
    const int rc = launch_gemv(a, st);
    if (rc) zero_fill(y, ybytes, st);
    return rc;
}

bool triple_dp4a(int a, int b, int c) {          // gemv_q4.cu:1474-1489
    return (a == 12 && b == 12 && c == 14) || (a == 12 && b == 12 && c == 12) || (a == 14 && b == 14 && c == 14) || (a == 14 && b == 12 && c == 12);
}

struct NormSpec { const void* w; int fp32; float eps; };

static int gemv_multi(int n, void* const* y, const void* const* W, const int* type, const int* M, const __half* x, int K,
                      const NormSpec* norm, int swiglu, cudaStream_t st) {
    bool all_k = true, any_q5 = false;
    for (int i = 0; i < n; ++i) { all_k = all_k && is_k(type[i]); any_q5 = any_q5 || type[i] == T_Q5K; }
    const void* Wd[3];
    bool ptr_ok = true;
    for (int i = 0; i < n; ++i) { Wd[i] = resolve_weight(W[i]); ptr_ok = ptr_ok && Wd[i]; }
    if (!all_k || !ptr_ok || any_q5) {
        if (norm || swiglu) return set_error(all_k ? JB_ERR_PTR : JB_ERR_TYPE, "fused norm/SwiGLU GEMV needs device-resident Q4_K/Q6_K matrices");
        // the reference falls back to one gemv_quant per matrix (gemv_q4.cu:2732-2733, :2750-2752)
        int rc = 0;
        for (int i = 0; i < n; ++i) { const int r = gemv_one(y[i], W[i], type[i], x, nullptr, M[i], K, 0, nullptr, st); rc = rc ? rc : r; }
        return rc;
    }
    const bool dp4a = n == 2 ? (type[0] == 12 && type[1] == 12) : triple_dp4a(type[0], type[1], type[2]);
    GemvArgs a;
    a.nseg = n;
    for (int i = 0; i < n; ++i) a.seg[i] = GemvSeg{ Wd[i], y[i], M[i], type[i] };
    a.x = x; a.K = K; a.xmode = dp4a ? 0 : 1; a.out_mode = swiglu ? 3 : 0;
    if (norm) { a.do_norm = 1; a.norm_w = norm->w; a.norm_w_fp32 = norm->fp32; a.eps = norm->eps; }
    const int rc = launch_gemv(a, st);
    if (rc) for (int i = 0; i < n; ++i) zero_fill(y[i], (size_t)(M[i] > 0 ? M[i] : 0) * 2, st);
    return rc;
}

static int gemm_batched(__half* y, const void* W, int type, const __half* x, int M, int N, int K, int32_t* dbg, cudaStream_t st) {
    if (N <= 0 || M <= 0 || K <= 0) return JB_OK;                         // gemv_q4.cu:2482
    if (N == 1 && !dbg) return gemv_one(y, W, type, x, nullptr, M, K, 0, nullptr, st);
    const size_t ybytes = (size_t)M * N * 2;
    if (!is_k(type)) { zero_fill(y, ybytes, st); return set_error(JB_ERR_TYPE, "unsupported ggml type %d", type); }
    const void* Wd = resolve_weight(W);
    if (!Wd) { zero_fill(y, ybytes, st); return set_error(JB_ERR_PTR, "weight pointer %p is not device-visible", W); }
    if (type == T_Q5K) {                                                   // scalar batched kernel in the reference: fp16-x float math per token
        int rc = 0;
        for (int t = 0; t < N && !rc; ++t) rc = launch_gemv_q5k(y + (size_t)t * M, nullptr, Wd, x + (size_t)t * K, nullptr, M, K, st);
        return rc;
    }
    const int rc = launch_mmq(y, Wd, type, x, M, N, K, dbg, st);
    if (rc) zero_fill(y, ybytes, st);
    return rc;
}

static int attention_decode(__half* out, const __half* q, const void* k, const void* v, int n_heads, int n_kv, int hd, int chd,
                            int seq_len, const int* d_pos, float scale, bool kv_int8, const float* ks, const float* vs, int window,
                            int n_splits, cudaStream_t st) {
    AttnCall c;
    c.out = out; c.q = q; c.k = k; c.v = v; c.ks = ks; c.vs = vs; c.n_heads = n_heads; c.n_kv = n_kv; c.hd = hd; c.chd = chd;
    c.seq_len = seq_len; c.d_pos = d_pos; c.scale = scale; c.kv_int8 = kv_int8; c.window = window; c.n_splits = n_splits;
    return launch_attention(c, st);
}

}  // namespace jb

using namespace jb;
#define ST(s) ((cudaStream_t)(s))
#define H(p)  ((__half*)(p))
#define CH(p) ((const __half*)(p))

// ══ extern "C" face ═══════════════════════════════════════════════════════
extern "C" {

int jllm_b200_init(int device) {
    if (device >= 0) JB_CUDA(cudaSetDevice(device));
    return ctx() ? JB_OK : g_err_code;
}
const char* jllm_b200_last_error(void) { return g_err; }
int  jllm_b200_last_error_code(void) { return g_err_code; }
void jllm_b200_clear_error(void) { g_err[0] = 0; g_err_code = 0; }
int jllm_b200_device_status(void* stream) {
    DeviceCtx* c = ctx();
    if (!c) return g_err_code;
    int h = 0;
    JB_CUDA(cudaMemcpyAsync(&h, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, ST(stream)));
    JB_CUDA(cudaStreamSynchronize(ST(stream)));
    if (h) { cudaMemsetAsync(c->d_status, 0, sizeof(int), ST(stream)); set_error(h, "a bounded device-side wait ran out"); }
    return h;
}
long long jllm_b200_launch_count(void) { return g_launches.load(); }
void jllm_b200_set_pdl(int on) { g_pdl.store(on ? 1 : 0); }
void jllm_b200_debug_gemv_trace(unsigned long long* device_buf) { gemv_set_trace(device_buf); }

const void* jllm_b200_resolve_mapped_weight_device_ptr(const void* p) {
    if (!p || !g_region.host || !g_region.dev) return nullptr;
    const char* c = (const char*)p;
    return (c >= g_region.host && c < g_region.host + g_region.bytes) ? g_region.dev + (c - g_region.host) : nullptr;
}
void jllm_b200_register_mapped_weight_region(const void* hb, const void* db, int64_t bytes) { g_region = { (const char*)hb, (const char*)db, bytes }; }
void jllm_b200_clear_mapped_weight_region(const void* hb) { if (g_region.host == hb) g_region = { nullptr, nullptr, 0 }; }

int jllm_b200_gemv_quant(void* y, const void* W, int t, const void* x, int M, int K, void* s) { return gemv_one(y, W, t, CH(x), nullptr, M, K, 0, nullptr, ST(s)); }
int jllm_b200_gemv_q4(void* y, const void* W, const void*, const void* x, int M, int K, int, void* s) { return gemv_one(y, W, 12, CH(x), nullptr, M, K, 0, nullptr, ST(s)); }
int jllm_b200_gemv_quant_add(void* y, const void* W, int t, const void* x, const void* r, int M, int K, void* s) {
    if (!r) return set_error(JB_ERR_PTR, "gemv_quant_add: null residual");
    return gemv_one(y, W, t, CH(x), CH(r), M, K, 2, nullptr, ST(s));
}
int jllm_b200_gemv_quant_pair(void* y0, const void* W0, int t0, int M0, void* y1, const void* W1, int t1, int M1, const void* x, int K, void* s) {
    void* y[2] = { y0, y1 }; const void* W[2] = { W0, W1 }; int t[2] = { t0, t1 }, M[2] = { M0, M1 };
    return gemv_multi(2, y, W, t, M, CH(x), K, nullptr, 0, ST(s));
}
int jllm_b200_gemv_quant_triple(void* y0, const void* W0, int t0, int M0, void* y1, const void* W1, int t1, int M1,
                                void* y2, const void* W2, int t2, int M2, const void* x, int K, void* s) {
    void* y[3] = { y0, y1, y2 }; const void* W[3] = { W0, W1, W2 }; int t[3] = { t0, t1, t2 }, M[3] = { M0, M1, M2 };
    return gemv_multi(3, y, W, t, M, CH(x), K, nullptr, 0, ST(s));
}
int jllm_b200_gemv_quant_f32(float* y, const void* W, int t, const void* x, int M, int K, void* s) { return gemv_one(y, W, t, CH(x), nullptr, M, K, 1, nullptr, ST(s)); }
int jllm_b200_gemm_quant_batched(void* y, const void* W, int t, const void* x, int M, int N, int K, void* s) { return gemm_batched(H(y), W, t, CH(x), M, N, K, nullptr, ST(s)); }
int jllm_b200_dequant_embedding_row(void* dst, const void* W, int t, int token, int hidden, void* s) {
    if (hidden <= 0 || hidden % QK_K) return set_error(JB_ERR_ARG, "embedding row: hidden=%d", hidden);
    const void* Wd = resolve_weight(W);
    if (!Wd) return set_error(JB_ERR_PTR, "embedding table %p is not device-visible", W);
    return launch_embed_row(H(dst), Wd, t, token, nullptr, hidden, ST(s));
}
int jllm_b200_gemv_dense(void* out, const void* W, int wt, const void* x, int M, int K, void* s) {
    const void* Wd = resolve_weight(W);
    if (!Wd) return set_error(JB_ERR_PTR, "dense weight %p is not device-visible", W);
    return launch_dense(H(out), Wd, wt, CH(x), M, 1, K, ST(s));
}
int jllm_b200_gemm_dense_batched(void* out, const void* W, int wt, const void* x, int M, int N, int K, void* s) {
    const void* Wd = resolve_weight(W);
    if (!Wd) return set_error(JB_ERR_PTR, "dense weight %p is not device-visible", W);
    return launch_dense(H(out), Wd, wt, CH(x), M, N, K, ST(s));
}

int jllm_b200_fused_rmsnorm_residual(void* o, const void* x, const void* r, const void* w, int rows, int dim, float eps, int wf32, void* s) {
    return launch_rmsnorm(H(o), CH(x), CH(r), w, wf32 != 0, rows, dim, eps, ST(s));
}
int jllm_b200_fused_swiglu(void* o, const void* g, const void* u, int rows, int dim, void* s) { return launch_glu(H(o), CH(g), CH(u), rows, dim, false, ST(s)); }
int jllm_b200_fused_geglu(void* o, const void* g, const void* u, int rows, int dim, void* s) { return launch_glu(H(o), CH(g), CH(u), rows, dim, true, ST(s)); }
int jllm_b200_vec_scale(void* x, int n, float sc, void* s) { return launch_vec_scale(H(x), n, sc, ST(s)); }
int jllm_b200_logit_softcap(float* x, int n, float cap, void* s) { return launch_softcap(x, n, cap, ST(s)); }
int jllm_b200_softmax_inplace(float* x, int n, void* s) { return launch_softmax(x, n, ST(s)); }
int jllm_b200_fp16_to_int8(int8_t* dst, float* sc, const void* src, int rows, int cols, void* s) { return launch_fp16_to_int8(dst, sc, CH(src), rows, cols, ST(s)); }

int jllm_b200_rope_precompute_table(int max_seq, int hd, float theta) { return rope_build_table(max_seq, hd, theta); }
int jllm_b200_rope_clear_tables(void) { rope_free_tables(); return JB_OK; }
int jllm_b200_rope_inplace(void* q, void* k, int nh, int nkv, int hd, int pos, float th, int neox, void* s) {
    return launch_rope(H(q), H(k), nullptr, nullptr, nullptr, nh, nkv, hd, hd, pos, nullptr, th, neox != 0, 1, 0, 0, 0, false, ST(s));
}
int jllm_b200_rope_inplace_store_kv_fp16(void* q, void* k, const void* v, void* kd, void* vd, int nh, int nkv, int hd, int pos, float th, int neox, void* s) {
    return launch_rope(H(q), H(k), CH(v), H(kd), H(vd), nh, nkv, hd, hd, pos, nullptr, th, neox != 0, 1, 0, 0, 0, false, ST(s));
}
int jllm_b200_rope_inplace_batched(void* q, void* k, int nh, int nkv, int hd, int start, int N, int qs, int ks, float th, int neox, void* s) {
    if (N <= 0) return JB_OK;
    return launch_rope(H(q), H(k), nullptr, nullptr, nullptr, nh, nkv, hd, hd, start, nullptr, th, neox != 0, N, qs, ks, 0, false, ST(s));
}
int jllm_b200_rope_inplace_store_kv_fp16_batched(void* q, void* k, const void* v, void* kb, void* vb, int kv_slot, int nh, int nkv, int hd,
                                                 int start, int N, int qs, int kvs, float th, int neox, void* s) {
    if (N <= 0) return JB_OK;
    return launch_rope(H(q), H(k), CH(v), H(kb), H(vb), nh, nkv, hd, hd, start, nullptr, th, neox != 0, N, qs, kvs, kv_slot, false, ST(s));
}
int jllm_b200_rope_inplace_store_kv_fp16_dyn(void* q, void* k, const void* v, void* kb, void* vb, int nh, int nkv, int hd, int chd,
                                             const int* d_pos, float th, int neox, void* s) {
    if (!d_pos) return set_error(JB_ERR_PTR, "rope dyn: null position pointer");
    return launch_rope(H(q), H(k), CH(v), H(kb), H(vb), nh, nkv, hd, chd, 0, d_pos, th, neox != 0, 1, 0, 0, 0, true, ST(s));
}
int jllm_b200_rope_inplace_dyn(void* q, void* k, int nh, int nkv, int hd, const int* d_pos, float th, int neox, void* s) {
    if (!d_pos) return set_error(JB_ERR_PTR, "rope dyn: null position pointer");
    return launch_rope(H(q), H(k), nullptr, nullptr, nullptr, nh, nkv, hd, hd, 0, d_pos, th, neox != 0, 1, 0, 0, 0, false, ST(s));
}

int jllm_b200_flash_attention_decode(void* o, const void* q, const void* k, const void* v, int nh, int nkv, int hd, int chd, int seq,
                                     float scale, int i8, const float* ks, const float* vs, int window, void* s) {
    return attention_decode(H(o), CH(q), k, v, nh, nkv, hd, chd, seq, nullptr, scale, i8 != 0, ks, vs, window, 0, ST(s));
}
int jllm_b200_flash_attention_prefill_batched(void* o, const void* q, const void* k, const void* v, int nh, int nkv, int hd, int chd,
                                              int N, int start, float scale, int i8, const float* ks, const float* vs, int window, void* s) {
    if (N <= 0) return JB_OK;
    AttnCall c;
    c.out = H(o); c.q = CH(q); c.k = k; c.v = v; c.ks = ks; c.vs = vs; c.n_heads = nh; c.n_kv = nkv; c.hd = hd; c.chd = chd;
    c.scale = scale; c.kv_int8 = i8; c.window = window; c.causal_start = start; c.batch = N; c.n_splits = 1;
    if (start < 0) return set_error(JB_ERR_ARG, "prefill attention: start_pos=%d", start);
    if (!c.out || !c.q || !k || !v) return set_error(JB_ERR_PTR, "prefill attention: null pointer");
    // INT8 cache with 128-wide heads: query-tiled tensor-core kernel; everything else: the general slice, one CTA per (head, token)
    return attention_prefill_fast_applies(c) ? launch_attention_prefill_fast(c, ST(s)) : launch_attention_general(c, ST(s));
}
int jllm_b200_flash_attention_decode_dyn(void* o, const void* q, const void* k, const void* v, int nh, int nkv, int hd, int chd,
                                         const int* d_pos, float scale, int i8, const float* kvs, int window, int n_splits, void* s) {
    if (!d_pos) return set_error(JB_ERR_PTR, "attention dyn: null position pointer");
    return attention_decode(H(o), CH(q), k, v, nh, nkv, hd, chd, 0, d_pos, scale, i8 != 0, kvs, kvs, window, n_splits > 0 ? n_splits : 1, ST(s));
}
int jllm_b200_decode_attn_splits(int seq_len) { return attn_splits_for(seq_len); }
float* jllm_b200_get_splitk_partials(int nh, int ns, int hd) { return splitk_buffer((size_t)nh * ns * (hd + 2), true); }

int jllm_b200_gemv_quant_int_dots(void* y, int32_t* dots, const void* W, int t, const void* x, int M, int K, void* s) {
    if (t != T_Q4K && t != T_Q6K) return set_error(JB_ERR_TYPE, "int dots: ggml type %d has no integer path", t);
    return gemv_one(y, W, t, CH(x), nullptr, M, K, 0, dots, ST(s));
}
int jllm_b200_gemm_quant_batched_pair(void* y0, const void* W0, int t0, int M0, void* y1, const void* W1, int t1, int M1, const void* x, int N, int K,
                                      void* s) {
    if (N < 2 || M0 <= 0 || M1 <= 0 || K <= 0 || K % QK_K) return set_error(JB_ERR_ARG, "gemm_quant_batched_pair: M0=%d M1=%d N=%d K=%d", M0, M1, N, K);
    if (!y0 || !y1 || !x) return set_error(JB_ERR_PTR, "gemm_quant_batched_pair: null pointer");
    if ((t0 != T_Q4K && t0 != T_Q6K) || (t1 != T_Q4K && t1 != T_Q6K)) return set_error(JB_ERR_TYPE, "gemm_quant_batched_pair: ggml types %d, %d", t0, t1);
    const void* Wd0 = resolve_weight(W0); const void* Wd1 = resolve_weight(W1);
    if (!Wd0 || !Wd1) return set_error(JB_ERR_PTR, "gemm_quant_batched_pair: weight pointer is not device-visible");
    return launch_mmq_pair(H(y0), H(y1), Wd0, t0, Wd1, t1, CH(x), M0, M1, N, K, ST(s));
}
int jllm_b200_gemm_quant_batched_int_dots(void* y, int32_t* dots, const void* W, int t, const void* x, int M, int N, int K, void* s) {
    if (t != T_Q4K && t != T_Q6K) return set_error(JB_ERR_TYPE, "int dots: ggml type %d has no integer path", t);
    return gemm_batched(H(y), W, t, CH(x), M, N, K, dots, ST(s));
}
int jllm_b200_norm_gemv_quant_pair(void* y0, const void* W0, int t0, int M0, void* y1, const void* W1, int t1, int M1, const void* x,
                                   const void* nw, int wf32, float eps, int K, void* s) {
    void* y[2] = { y0, y1 }; const void* W[2] = { W0, W1 }; int t[2] = { t0, t1 }, M[2] = { M0, M1 };
    NormSpec n = { nw, wf32, eps };
    return gemv_multi(2, y, W, t, M, CH(x), K, &n, 0, ST(s));
}
int jllm_b200_norm_gemv_quant_triple(void* y0, const void* W0, int t0, int M0, void* y1, const void* W1, int t1, int M1,
                                     void* y2, const void* W2, int t2, int M2, const void* x, const void* nw, int wf32, float eps, int K, void* s) {
    void* y[3] = { y0, y1, y2 }; const void* W[3] = { W0, W1, W2 }; int t[3] = { t0, t1, t2 }, M[3] = { M0, M1, M2 };
    NormSpec n = { nw, wf32, eps };
    return gemv_multi(3, y, W, t, M, CH(x), K, &n, 0, ST(s));
}
int jllm_b200_norm_gemv_pair_swiglu(void* out, const void* Wg, const void* Wu, int t, int M, const void* x, const void* nw, int wf32,
                                    float eps, int K, void* s) {
    void* y[2] = { out, out }; const void* W[2] = { Wg, Wu }; int tt[2] = { t, t }, MM[2] = { M, M };
    NormSpec n = { nw, wf32, eps };
    return gemv_multi(2, y, W, tt, MM, CH(x), K, nw ? &n : nullptr, 1, ST(s));
}
int jllm_b200_qkv_prep_int8(void* q, const void* k, const void* v, const float* qn, const float* kn, float eps, int8_t* kc, int8_t* vc,
                            float* ksc, float* vsc, int nh, int nkv, int hd, int pos, const int* d_pos, float th, int neox, void* s) {
    return launch_qkv_prep(H(q), CH(k), CH(v), qn, kn, eps, kc, vc, ksc, vsc, nh, nkv, hd, pos, d_pos, th, neox != 0, true, ST(s));
}
int jllm_b200_flash_attention_decode_batched(void* o, const void* q, const void* const* kl, const void* const* vl, const float* const* ksl,
                                             const float* const* vsl, const int* seq_lens, int batch, int max_seq, int nh, int nkv, int hd,
                                             float scale, int i8, void* s) {
    if (batch <= 0) return JB_OK;
    if (!kl || !vl || !seq_lens) return set_error(JB_ERR_PTR, "batched attention: null list pointer");
    AttnCall c;
    c.out = H(o); c.q = CH(q); c.k_list = kl; c.v_list = vl; c.ks_list = ksl; c.vs_list = vsl; c.seq_lens = seq_lens; c.batch = batch;
    c.max_seq = max_seq; c.n_heads = nh; c.n_kv = nkv; c.hd = hd; c.chd = hd; c.scale = scale; c.kv_int8 = i8;
    return launch_attention(c, ST(s));
}

/* ── attention plan: tensor maps of a fixed set of INT8 caches, built once on the host ── */
struct jllm_b200_attn_plan { std::vector<unsigned char> maps; const float** ks = nullptr; const float** vs = nullptr; int batch = 0, max_seq = 0, n_kv = 0, hd = 0; };

jllm_b200_attn_plan* jllm_b200_attn_plan_create(const void* const* k_list, const void* const* v_list, const float* const* ks_list,
                                                const float* const* vs_list, int batch, int max_seq_len, int n_kv_heads, int head_dim) {
    if (!k_list || !v_list || !ks_list || !vs_list || batch <= 0 || max_seq_len <= 0 || n_kv_heads <= 0) { set_error(JB_ERR_ARG, "attention plan: bad arguments"); return nullptr; }
    if (head_dim != 128) { set_error(JB_ERR_LIMIT, "attention plan: head_dim %d (the tensor-map path handles 128)", head_dim); return nullptr; }
    if (!ctx()) return nullptr;
    std::vector<unsigned char> maps((size_t)batch * 2 * 128);
    for (int b = 0; b < batch; ++b)
        if (!attn_tma_encode(&maps[((size_t)b * 2 + 0) * 128], k_list[b], max_seq_len, n_kv_heads) ||
            !attn_tma_encode(&maps[((size_t)b * 2 + 1) * 128], v_list[b], max_seq_len, n_kv_heads)) {
            set_error(JB_ERR_PTR, "attention plan: tensor map of cache %d refused (caches must be 16-byte aligned device memory)", b);
            return nullptr;
        }
    jllm_b200_attn_plan* p = new (std::nothrow) jllm_b200_attn_plan();
    if (!p) return nullptr;
    p->batch = batch; p->max_seq = max_seq_len; p->n_kv = n_kv_heads; p->hd = head_dim;
    p->maps.swap(maps);                  // the maps stay on the host: they travel to the kernel as launch parameters
    if (cudaMalloc((void**)&p->ks, (size_t)batch * sizeof(void*)) != cudaSuccess || cudaMalloc((void**)&p->vs, (size_t)batch * sizeof(void*)) != cudaSuccess) {
        cuda_error(cudaGetLastError(), "cudaMalloc(attention plan)"); jllm_b200_attn_plan_destroy(p); return nullptr;
    }
    cudaMemcpy((void*)p->ks, ks_list, (size_t)batch * sizeof(void*), cudaMemcpyHostToDevice);
    cudaMemcpy((void*)p->vs, vs_list, (size_t)batch * sizeof(void*), cudaMemcpyHostToDevice);
    return p;
}
void jllm_b200_attn_plan_destroy(jllm_b200_attn_plan* p) {
    if (!p) return;
    if (p->ks) cudaFree((void*)p->ks);
    if (p->vs) cudaFree((void*)p->vs);
    delete p;
}
int jllm_b200_flash_attention_decode_planned(const jllm_b200_attn_plan* p, void* o, const void* q, const int* seq_lens, int nh, float scale, void* s) {
    if (!p || !o || !q || !seq_lens) return set_error(JB_ERR_PTR, "planned attention: null pointer");
    AttnCall c;
    c.out = H(o); c.q = CH(q); c.tma_maps = p->maps.data(); c.ks_list = p->ks; c.vs_list = p->vs; c.seq_lens = seq_lens; c.batch = p->batch;
    c.max_seq = p->max_seq; c.n_heads = nh; c.n_kv = p->n_kv; c.hd = p->hd; c.chd = p->hd; c.scale = scale; c.kv_int8 = 1;
    if (!attention_tma_applies(c)) return set_error(JB_ERR_ARG, "planned attention: %d query heads over %d KV heads is not a supported group", nh, p->n_kv);
    return launch_attention_tma(c, ST(s));
}

}  // extern "C"

// ══ C++ face: the reference's own symbols ═══════════════════════════════════
namespace jllm {

const void* resolve_mapped_weight_device_ptr(const void* p) { return jllm_b200_resolve_mapped_weight_device_ptr(p); }
void register_mapped_weight_region(const void* hb, const void* db, int64_t bytes) { jllm_b200_register_mapped_weight_region(hb, db, bytes); }
void clear_mapped_weight_region(const void* hb) { jllm_b200_clear_mapped_weight_region(hb); }

static void report(int rc, const char* fn) {
    if (rc) fprintf(stderr, "[jllm-b200] %s failed (%d): %s\n", fn, rc, jllm_b200_last_error());
}
#define RUN(fn, call) report((call), fn)

void gemv_q4(half* y, const void* W, const half* sc, const half* x, int M, int K, int gs, cudaStream_t s) { RUN("gemv_q4", jllm_b200_gemv_q4(y, W, sc, x, M, K, gs, s)); }
void gemv_quant(half* y, const void* W, int t, const half* x, int M, int K, cudaStream_t s) { RUN("gemv_quant", jllm_b200_gemv_quant(y, W, t, x, M, K, s)); }
void gemv_quant_add(half* y, const void* W, int t, const half* x, const half* r, int M, int K, cudaStream_t s) { RUN("gemv_quant_add", jllm_b200_gemv_quant_add(y, W, t, x, r, M, K, s)); }
void gemv_quant_pair(half* y0, const void* W0, int t0, int M0, half* y1, const void* W1, int t1, int M1, const half* x, int K, cudaStream_t s) {
    RUN("gemv_quant_pair", jllm_b200_gemv_quant_pair(y0, W0, t0, M0, y1, W1, t1, M1, x, K, s));
}
void gemv_quant_triple(half* y0, const void* W0, int t0, int M0, half* y1, const void* W1, int t1, int M1, half* y2, const void* W2, int t2, int M2,
                       const half* x, int K, cudaStream_t s) {
    RUN("gemv_quant_triple", jllm_b200_gemv_quant_triple(y0, W0, t0, M0, y1, W1, t1, M1, y2, W2, t2, M2, x, K, s));
}
void gemm_quant_batched(half* y, const void* W, int t, const half* x, int M, int N, int K, cudaStream_t s) { RUN("gemm_quant_batched", jllm_b200_gemm_quant_batched(y, W, t, x, M, N, K, s)); }
void gemv_quant_f32(float* y, const void* W, int t, const half* x, int M, int K, cudaStream_t s) { RUN("gemv_quant_f32", jllm_b200_gemv_quant_f32(y, W, t, x, M, K, s)); }
bool dequant_embedding_row(half* dst, const void* W, int t, int token, int hidden, cudaStream_t s) { return jllm_b200_dequant_embedding_row(dst, W, t, token, hidden, s) == 0; }

void fused_rmsnorm_residual(half* o, const half* x, const half* r, const void* w, int rows, int dim, float eps, bool wf32, cudaStream_t s) {
    RUN("fused_rmsnorm_residual", jllm_b200_fused_rmsnorm_residual(o, x, r, w, rows, dim, eps, wf32, s));
}
void fused_swiglu(half* o, const half* g, const half* u, int rows, int dim, cudaStream_t s) { RUN("fused_swiglu", jllm_b200_fused_swiglu(o, g, u, rows, dim, s)); }
void fused_geglu(half* o, const half* g, const half* u, int rows, int dim, cudaStream_t s) { RUN("fused_geglu", jllm_b200_fused_geglu(o, g, u, rows, dim, s)); }
void vec_scale(half* x, int n, float sc, cudaStream_t s) { RUN("vec_scale", jllm_b200_vec_scale(x, n, sc, s)); }
void logit_softcap(float* x, int n, float cap, cudaStream_t s) { RUN("logit_softcap", jllm_b200_logit_softcap(x, n, cap, s)); }
void gemv_dense(half* o, const void* W, int wt, const half* x, int M, int K, cudaStream_t s) { RUN("gemv_dense", jllm_b200_gemv_dense(o, W, wt, x, M, K, s)); }
void gemm_dense_batched(half* o, const void* W, int wt, const half* x, int M, int N, int K, cudaStream_t s) { RUN("gemm_dense_batched", jllm_b200_gemm_dense_batched(o, W, wt, x, M, N, K, s)); }

void rope_precompute_table(int max_seq, int hd, float th) { RUN("rope_precompute_table", jllm_b200_rope_precompute_table(max_seq, hd, th)); }
void rope_clear_tables() { jllm_b200_rope_clear_tables(); }
void rope_inplace(half* q, half* k, int nh, int nkv, int hd, int pos, float th, bool neox, cudaStream_t s) { RUN("rope_inplace", jllm_b200_rope_inplace(q, k, nh, nkv, hd, pos, th, neox, s)); }
void rope_inplace_store_kv_fp16(half* q, half* k, const half* v, half* kd, half* vd, int nh, int nkv, int hd, int pos, float th, bool neox, cudaStream_t s) {
    RUN("rope_inplace_store_kv_fp16", jllm_b200_rope_inplace_store_kv_fp16(q, k, v, kd, vd, nh, nkv, hd, pos, th, neox, s));
}
void rope_inplace_batched(half* q, half* k, int nh, int nkv, int hd, int start, int N, int qs, int ks, float th, bool neox, cudaStream_t s) {
    RUN("rope_inplace_batched", jllm_b200_rope_inplace_batched(q, k, nh, nkv, hd, start, N, qs, ks, th, neox, s));
}
void rope_inplace_store_kv_fp16_batched(half* q, half* k, const half* v, half* kb, half* vb, int kv_slot, int nh, int nkv, int hd, int start, int N,
                                        int qs, int kvs, float th, bool neox, cudaStream_t s) {
    RUN("rope_inplace_store_kv_fp16_batched", jllm_b200_rope_inplace_store_kv_fp16_batched(q, k, v, kb, vb, kv_slot, nh, nkv, hd, start, N, qs, kvs, th, neox, s));
}
void rope_inplace_store_kv_fp16_dyn(half* q, half* k, const half* v, half* kb, half* vb, int nh, int nkv, int hd, int chd, const int* d_pos, float th,
                                    bool neox, cudaStream_t s) {
    RUN("rope_inplace_store_kv_fp16_dyn", jllm_b200_rope_inplace_store_kv_fp16_dyn(q, k, v, kb, vb, nh, nkv, hd, chd, d_pos, th, neox, s));
}
void rope_inplace_dyn(half* q, half* k, int nh, int nkv, int hd, const int* d_pos, float th, bool neox, cudaStream_t s) {
    RUN("rope_inplace_dyn", jllm_b200_rope_inplace_dyn(q, k, nh, nkv, hd, d_pos, th, neox, s));
}

void flash_attention_decode(half* o, const half* q, const void* k, const void* v, int nh, int nkv, int hd, int chd, int seq, float scale, bool i8,
                            const float* ks, const float* vs, int window, cudaStream_t s) {
    const int rc = jllm_b200_flash_attention_decode(o, q, k, v, nh, nkv, hd, chd, seq, scale, i8, ks, vs, window, s);
    if (rc) { cudaMemsetAsync(o, 0, (size_t)nh * hd * sizeof(half), s); report(rc, "flash_attention_decode"); }   // reference zero-fills, attention.cu:1078-1082
}
void flash_attention_prefill_batched(half* o, const half* q, const void* k, const void* v, int nh, int nkv, int hd, int chd, int N, int start,
                                     float scale, bool i8, const float* ks, const float* vs, int window, cudaStream_t s) {
    RUN("flash_attention_prefill_batched", jllm_b200_flash_attention_prefill_batched(o, q, k, v, nh, nkv, hd, chd, N, start, scale, i8, ks, vs, window, s));
}
void flash_attention_decode_dyn(half* o, const half* q, const void* k, const void* v, int nh, int nkv, int hd, int chd, const int* d_pos, float scale,
                                bool i8, const float* kvs, int window, int n_splits, cudaStream_t s) {
    RUN("flash_attention_decode_dyn", jllm_b200_flash_attention_decode_dyn(o, q, k, v, nh, nkv, hd, chd, d_pos, scale, i8, kvs, window, n_splits, s));
}
int decode_attn_splits(int seq_len) { return jllm_b200_decode_attn_splits(seq_len); }
float* get_splitk_partials(int nh, int ns, int hd) { return jllm_b200_get_splitk_partials(nh, ns, hd); }

void softmax_inplace(float* x, int n, cudaStream_t s) { RUN("softmax_inplace", jllm_b200_softmax_inplace(x, n, s)); }
void fp16_to_int8(int8_t* dst, float* sc, const half* src, int rows, int cols, cudaStream_t s) { RUN("fp16_to_int8", jllm_b200_fp16_to_int8(dst, sc, src, rows, cols, s)); }

}  // namespace jllm
