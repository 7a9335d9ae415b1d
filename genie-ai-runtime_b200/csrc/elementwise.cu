// elementwise.cu — RMSNorm, RoPE, SwiGLU/GeGLU, KV int8 quantiser, embedding-row
// dequantiser and the small helpers of the kernel API, for sm_100a.
// Reference: src/kernels/fused_norm.cu, rope.cu, convert.cu, softmax.cu,
// gemv_q4.cu:793-864 (embedding), :2811-2885 (dense GEMV).
#include "elementwise.cuh"
#include <cmath>
#include <cfloat>

namespace jb {

// ── RMSNorm (+ optional residual): out = half((x[+res]) * rrms * w) ─────────
// fused_norm.cu:33-101.  One CTA per row for wide rows, one warp per row for
// per-head rows (Qwen3 QK-norm: rows = heads, dim = head_dim).
template <int THREADS>
__global__ void rmsnorm_kernel(__half* out, const __half* x, const __half* res, const void* w, int w_fp32,
                               int rows, int dim, float eps) {
    pdl_wait();
    constexpr int WARPS = THREADS / 32;
    const int row = THREADS == 32 ? blockIdx.x * blockDim.y + threadIdx.y : blockIdx.x;
    if (row >= rows) return;
    const int tid = threadIdx.x, lane = tid & 31;
    const size_t off = (size_t)row * dim;
    float ss = 0.f;
    for (int i = tid * 2; i < dim; i += THREADS * 2) {
        float2 v = __half22float2(*reinterpret_cast<const __half2*>(x + off + i));
        if (res) { const float2 r = __half22float2(*reinterpret_cast<const __half2*>(res + off + i)); v.x += r.x; v.y += r.y; }
        ss += v.x * v.x + v.y * v.y;
    }
    ss = warp_sum(ss);
    if (WARPS > 1) {
        __shared__ float part[WARPS];
        if (lane == 0) part[tid >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        #pragma unroll
        for (int i = 0; i < WARPS; ++i) ss += part[i];
    }
    const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    for (int i = tid * 2; i < dim; i += THREADS * 2) {
        float2 v = __half22float2(*reinterpret_cast<const __half2*>(x + off + i));
        if (res) { const float2 r = __half22float2(*reinterpret_cast<const __half2*>(res + off + i)); v.x += r.x; v.y += r.y; }
        float w0, w1;
        if (w_fp32) { w0 = reinterpret_cast<const float*>(w)[i]; w1 = reinterpret_cast<const float*>(w)[i + 1]; }
        else { const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(w) + i)); w0 = wf.x; w1 = wf.y; }
        *reinterpret_cast<__half2*>(out + off + i) =
            __floats2half2_rn(__fmul_rn(__fmul_rn(v.x, rrms), w0), __fmul_rn(__fmul_rn(v.y, rrms), w1));
    }
}

int launch_rmsnorm(__half* out, const __half* x, const __half* res, const void* w, bool w_fp32,
                   int rows, int dim, float eps, cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return JB_OK;
    if (!out || !x || !w) return set_error(JB_ERR_PTR, "rmsnorm: null pointer");
    if (dim & 1) return set_error(JB_ERR_ARG, "rmsnorm: dim=%d must be even", dim);
    if (dim >= 1024) {
        JB_CUDA(launch_k(rmsnorm_kernel<256>, dim3(rows), dim3(256), 0, st, pdl_enabled(), out, x, res, w, (int)w_fp32, rows, dim, eps));
    } else {
        JB_CUDA(launch_k(rmsnorm_kernel<32>, dim3((rows + 3) / 4), dim3(32, 4), 0, st, pdl_enabled(), out, x, res, w, (int)w_fp32, rows, dim, eps));
    }
    count_launch();
    return JB_OK;
}

// ── RoPE ─────────────────────────────────────────────────────────────────
// rope.cu:322-367: freq = 1/powf(theta, 2i/hd), angle = pos*freq, rotate (i, i+hd/2)
// (NeoX) or (2i, 2i+1).  The per-pair frequencies are computed on the host with the
// same fp32 formula and passed by value, so no device powf rounding enters the angle.
RopeFreq make_rope_freq(int head_dim, float theta) {
    RopeFreq f = {};
    for (int i = 0; i < head_dim / 2 && i < 256; ++i) f.f[i] = 1.0f / powf(theta, (2.0f * i) / head_dim);
    return f;
}

__device__ __forceinline__ void rope_pair(__half* ptr, int pair, int h2, float c, float s, bool neox, __half& r0, __half& r1, int& i0, int& i1) {
    i0 = neox ? pair : 2 * pair; i1 = neox ? pair + h2 : 2 * pair + 1;
    const float v0 = __half2float(ptr[i0]), v1 = __half2float(ptr[i1]);
    r0 = __float2half_rn(__fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s)));
    r1 = __float2half_rn(__fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c)));
}

// One kernel covers rope_inplace / _store_kv_fp16 / _dyn / _batched: position from an int or a
// device int, optional K/V fp16 cache store (cache row stride cache_hd per head), optional table.
struct RopeArgs {
    __half* q; __half* k; const __half* v; __half* k_dst; __half* v_dst;
    int n_heads, n_kv, hd, cache_hd, pos; const int* d_pos; int neox;
    const float* cos_tbl; const float* sin_tbl;
    int N, q_stride, k_stride, kv_slot;      // batched: token t at q + t*q_stride; cache row (pos+t)*kv_slot
    int dyn_cache;                            // cache destination = base + pos*n_kv*cache_hd
};
__global__ void rope_kernel(const RopeArgs a, const __grid_constant__ RopeFreq fr) {
    pdl_wait();
    const int t = blockIdx.y;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int h2 = a.hd / 2, q_pairs = a.n_heads * h2, total = (a.n_heads + a.n_kv) * h2;
    const int pos = (a.d_pos ? *a.d_pos : a.pos) + t;
    __half* q = a.q + (size_t)t * a.q_stride;
    __half* k = a.k ? a.k + (size_t)t * a.k_stride : nullptr;
    __half* kd = a.k_dst; __half* vd = a.v_dst;
    if (kd) {
        const size_t row = a.dyn_cache ? (size_t)pos * a.n_kv * a.cache_hd : (size_t)t * a.kv_slot;
        kd += row; vd += row;
    }
    if (tid < total) {
        const bool is_q = tid < q_pairs;
        const int kt = is_q ? tid : tid - q_pairs, head = kt / h2, pair = kt % h2;
        __half* ptr = (is_q ? q : k) + (size_t)head * a.hd;
        float c, s;
        if (a.cos_tbl) { c = a.cos_tbl[(size_t)pos * h2 + pair]; s = a.sin_tbl[(size_t)pos * h2 + pair]; }
        else { const float ang = __fmul_rn((float)pos, fr.f[pair]); c = cosf(ang); s = sinf(ang); }
        __half r0, r1; int i0, i1;
        rope_pair(ptr, pair, h2, c, s, a.neox, r0, r1, i0, i1);
        ptr[i0] = r0; ptr[i1] = r1;
        if (!is_q && kd) { kd[(size_t)head * a.cache_hd + i0] = r0; kd[(size_t)head * a.cache_hd + i1] = r1; }
    }
    if (vd && a.v && tid < a.n_kv * a.hd) {
        const int head = tid / a.hd, d = tid % a.hd;
        vd[(size_t)head * a.cache_hd + d] = a.v[(size_t)t * a.k_stride + tid];
    }
}

__global__ void rope_table_kernel(float* cos_tbl, float* sin_tbl, int h2, int max_seq, const __grid_constant__ RopeFreq fr) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= max_seq * h2) return;
    const float ang = __fmul_rn((float)(idx / h2), fr.f[idx % h2]);
    cos_tbl[idx] = cosf(ang); sin_tbl[idx] = sinf(ang);
}

static const RopeTable* find_table(float theta, int h2) {
    DeviceCtx* c = ctx();
    if (!c) return nullptr;
    for (int i = 0; i < c->n_rope; ++i) if (c->rope[i].theta == theta && c->rope[i].half_dim == h2) return &c->rope[i];
    return nullptr;
}

int rope_build_table(int max_seq, int head_dim, float theta) {
    DeviceCtx* c = ctx();
    if (!c) return JB_ERR_CUDA;
    const int h2 = head_dim / 2;
    if (h2 <= 0 || h2 > 256 || max_seq <= 0) return set_error(JB_ERR_ARG, "rope table: head_dim=%d max_seq=%d", head_dim, max_seq);
    if (find_table(theta, h2)) return JB_OK;
    if (c->n_rope >= 8) return set_error(JB_ERR_LIMIT, "rope table: all 8 slots in use");
    const size_t n = (size_t)max_seq * h2;
    float *dc = nullptr, *ds = nullptr;
    if (cudaMalloc(&dc, n * 4) != cudaSuccess || cudaMalloc(&ds, n * 4) != cudaSuccess) {
        cudaFree(dc); cudaGetLastError();
        return set_error(JB_ERR_NOMEM, "rope table: allocation of %zu floats failed", 2 * n);
    }
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256>>>(dc, ds, h2, max_seq, make_rope_freq(head_dim, theta));
    JB_CUDA(cudaGetLastError());
    JB_CUDA(cudaDeviceSynchronize());
    c->rope[c->n_rope++] = RopeTable{ theta, h2, max_seq, dc, ds };
    return JB_OK;
}
void rope_free_tables() {
    DeviceCtx* c = ctx();
    if (!c) return;
    for (int i = 0; i < c->n_rope; ++i) { cudaFree(c->rope[i].cos); cudaFree(c->rope[i].sin); }
    c->n_rope = 0;
}

int launch_rope(__half* q, __half* k, const __half* v, __half* k_dst, __half* v_dst, int n_heads, int n_kv, int hd, int cache_hd,
                int pos, const int* d_pos, float theta, bool neox, int N, int q_stride, int k_stride, int kv_slot, bool dyn_cache,
                cudaStream_t st) {
    if (!q || hd <= 0 || (hd & 1) || hd > 512) return set_error(JB_ERR_ARG, "rope: q=%p head_dim=%d", (void*)q, hd);
    if (!k) n_kv = 0;
    RopeArgs a = {};
    a.q = q; a.k = k; a.v = v; a.k_dst = k_dst; a.v_dst = v_dst; a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.cache_hd = cache_hd;
    a.pos = pos; a.d_pos = d_pos; a.neox = neox; a.N = N; a.q_stride = q_stride; a.k_stride = k_stride; a.kv_slot = kv_slot; a.dyn_cache = dyn_cache;
    const RopeTable* tb = find_table(theta, hd / 2);
    // the table is only used for positions it covers; device positions are checked by the caller's context length
    if (tb && !d_pos && pos + N <= tb->max_seq) { a.cos_tbl = tb->cos; a.sin_tbl = tb->sin; }
    if (tb && d_pos) { a.cos_tbl = tb->cos; a.sin_tbl = tb->sin; }
    const int work = max((n_heads + n_kv) * (hd / 2), v_dst ? n_kv * hd : 0);
    JB_CUDA(launch_k(rope_kernel, dim3((work + 127) / 128, N), dim3(128), 0, st, pdl_enabled(), a, make_rope_freq(hd, theta)));
    count_launch();
    return JB_OK;
}

// ── SwiGLU / GeGLU / scale / softcap (convert.cu:85-181) ───────────────────
__global__ void glu_kernel(__half* out, const __half* gate, const __half* up, long long total, int gelu) {
    pdl_wait();
    const long long i2 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i2 >= total) return;
    float g[2], u[2], r[2];
    g[0] = __half2float(gate[i2]); u[0] = __half2float(up[i2]);
    const bool two = i2 + 1 < total;
    g[1] = two ? __half2float(gate[i2 + 1]) : 0.f; u[1] = two ? __half2float(up[i2 + 1]) : 0.f;
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (gelu) {
            const float x = g[i];
            const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(x, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x)));
            r[i] = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner))), u[i]);
        } else {
            r[i] = __fmul_rn(__fdiv_rn(g[i], __fadd_rn(1.0f, expf(-g[i]))), u[i]);
        }
    }
    out[i2] = __float2half_rn(r[0]);
    if (two) out[i2 + 1] = __float2half_rn(r[1]);
}
// the same arithmetic, eight elements per thread with 16-byte accesses (batched layers: millions of elements)
__global__ void glu8_kernel(__half* out, const __half* gate, const __half* up, long long total8, int gelu) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const uint4 gv = reinterpret_cast<const uint4*>(gate)[i], uv = reinterpret_cast<const uint4*>(up)[i];
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t ow[4];
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&gw[k])), u = __half22float2(*reinterpret_cast<const __half2*>(&uw[k]));
        const float gs[2] = {g.x, g.y}, us[2] = {u.x, u.y};
        float r[2];
        #pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (gelu) {
                const float x = gs[e];
                const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(x, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, x), x), x)));
                r[e] = __fmul_rn(__fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, tanhf(inner))), us[e]);
            } else {
                r[e] = __fmul_rn(__fdiv_rn(gs[e], __fadd_rn(1.0f, expf(-gs[e]))), us[e]);
            }
        }
        const __half2 h = __halves2half2(__float2half_rn(r[0]), __float2half_rn(r[1]));
        ow[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}
int launch_glu(__half* out, const __half* gate, const __half* up, int rows, int dim, bool gelu, cudaStream_t st) {
    const long long total = (long long)rows * dim;
    if (total <= 0) return JB_OK;
    if (!out || !gate || !up) return set_error(JB_ERR_PTR, "glu: null pointer");
    if (total >= 4096 && total % 8 == 0 && (((uintptr_t)out | (uintptr_t)gate | (uintptr_t)up) & 15) == 0) {
        JB_CUDA(launch_k(glu8_kernel, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0, st, pdl_enabled(), out, gate, up, total / 8, (int)gelu));
        count_launch();
        return JB_OK;
    }
    const long long t2 = (total + 1) / 2;
    JB_CUDA(launch_k(glu_kernel, dim3((unsigned)((t2 + 255) / 256)), dim3(256), 0, st, pdl_enabled(), out, gate, up, total, (int)gelu));
    count_launch();
    return JB_OK;
}

__global__ void vec_scale_kernel(__half* x, int n, float s) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {   // convert.cu:152-161: full pairs use a half multiply by half(s), an odd last element a float multiply
        if ((i & ~1) + 1 < n) x[i] = __hmul(x[i], __float2half_rn(s));
        else x[i] = __float2half_rn(__half2float(x[i]) * s);
    }
}
int launch_vec_scale(__half* x, int n, float s, cudaStream_t st) {
    if (n <= 0) return JB_OK;
    JB_CUDA(launch_k(vec_scale_kernel, dim3((n + 255) / 256), dim3(256), 0, st, pdl_enabled(), x, n, s));
    count_launch();
    return JB_OK;
}
__global__ void softcap_kernel(float* x, int n, float cap) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}
int launch_softcap(float* x, int n, float cap, cudaStream_t st) {
    if (n <= 0) return JB_OK;
    JB_CUDA(launch_k(softcap_kernel, dim3((n + 255) / 256), dim3(256), 0, st, pdl_enabled(), x, n, cap));
    count_launch();
    return JB_OK;
}

// ── softmax over a logits vector (softmax.cu:15-74), one CTA ───────────────
__global__ void softmax_kernel(float* x, int n) {
    pdl_wait();
    __shared__ float red[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = -FLT_MAX;
    for (int i = tid; i < n; i += blockDim.x) m = fmaxf(m, x[i]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float s = 0.f;
    for (int i = tid; i < n; i += blockDim.x) { const float e = expf(x[i] - m); x[i] = e; s += e; }
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    for (int i = tid; i < n; i += blockDim.x) x[i] = __fdiv_rn(x[i], s);
}
int launch_softmax(float* x, int n, cudaStream_t st) {
    if (n <= 0) return JB_OK;
    JB_CUDA(launch_k(softmax_kernel, dim3(1), dim3(1024), 0, st, pdl_enabled(), x, n));
    count_launch();
    return JB_OK;
}

// ── fp16 -> int8 with one absmax scale per row (convert.cu:26-69) ──────────
// scale = max/127, q = clamp(rn(x * (127/max)), ±127).  One warp per row.
__global__ void fp16_to_int8_kernel(int8_t* dst, float* scale_out, const __half* src, int rows, int cols) {
    pdl_wait();
    const int row = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    if (row >= rows) return;
    const size_t off = (size_t)row * cols;
    float mx = 0.f;
    for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, fabsf(__half2float(src[off + c])));
    mx = warp_max(mx);
    const float scale = __fdiv_rn(mx, 127.0f);
    const float inv = scale > 0.f ? __fdiv_rn(127.0f, mx) : 0.f;
    if (lane == 0 && scale_out) scale_out[row] = scale;
    for (int c = lane; c < cols; c += 32)
        dst[off + c] = (int8_t)max(-127, min(127, __float2int_rn(__fmul_rn(__half2float(src[off + c]), inv))));
}
int launch_fp16_to_int8(int8_t* dst, float* scale_out, const __half* src, int rows, int cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return JB_OK;
    if (!dst || !src) return set_error(JB_ERR_PTR, "fp16_to_int8: null pointer");
    JB_CUDA(launch_k(fp16_to_int8_kernel, dim3((rows + 3) / 4), dim3(32, 4), 0, st, pdl_enabled(), dst, scale_out, src, rows, cols));
    count_launch();
    return JB_OK;
}

// ── one embedding row -> fp16 (gemv_q4.cu:793-864) ─────────────────────────
// blockIdx.y = row of a batch: token d_token[y], destination dst + y * hidden
__global__ void embed_row_kernel(__half* dst, const uint8_t* W, int type, const int* d_token, int token, int hidden) {
    pdl_wait();
    const int b = blockIdx.x, i = threadIdx.x, nb = hidden / QK_K;
    const int tok = d_token ? d_token[blockIdx.y] : token;
    dst += (size_t)blockIdx.y * hidden;
    float val;
    if (type == T_Q4K) {
        const uint8_t* blk = W + ((size_t)tok * nb + b) * Q4K_BYTES;
        const uint32_t* s = reinterpret_cast<const uint32_t*>(blk + 4);
        int sc, mn; scale_min_k4(i >> 5, s[0], s[1], s[2], sc, mn);
        const uint8_t qb = blk[16 + 32 * (i >> 6) + (i & 31)];
        const int q = (i & 32) ? (qb >> 4) : (qb & 0xF);
        const float dall = h2f_bits(*reinterpret_cast<const unsigned short*>(blk)), dmin = h2f_bits(*reinterpret_cast<const unsigned short*>(blk + 2));
        val = __fsub_rn(__fmul_rn(__fmul_rn(dall, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
    } else {
        const uint8_t* blk = W + ((size_t)tok * nb + b) * Q6K_BYTES;
        const int n = i >> 7, r = i & 127, quarter = r >> 5, l = r & 31;
        int lo = (quarter & 1) ? blk[64 * n + 32 + l] : blk[64 * n + l];
        lo = (quarter & 2) ? (lo >> 4) : (lo & 0xF);
        const int q = lo | (((blk[128 + 32 * n + l] >> (2 * quarter)) & 3) << 4);
        const float d = h2f_bits(blk[208] | (blk[209] << 8));
        val = __fmul_rn(__fmul_rn(d, (float)(int8_t)blk[192 + (i >> 4)]), (float)(q - 32));
    }
    dst[b * QK_K + i] = __float2half_rn(val);
}
int launch_embed_rows(__half* dst, const void* W, int type, const int* d_tokens, int rows, int hidden, cudaStream_t st) {
    if (rows <= 0) return JB_OK;
    if (hidden <= 0 || hidden % QK_K) return set_error(JB_ERR_ARG, "embedding rows: hidden=%d is not a multiple of 256", hidden);
    if (type != T_Q4K && type != T_Q6K) return set_error(JB_ERR_TYPE, "embedding rows: ggml type %d", type);
    if (!dst || !W || !d_tokens) return set_error(JB_ERR_PTR, "embedding rows: null pointer");
    JB_CUDA(launch_k(embed_row_kernel, dim3(hidden / QK_K, rows), dim3(QK_K), 0, st, pdl_enabled(), dst, (const uint8_t*)W, type, d_tokens, 0, hidden));
    count_launch();
    return JB_OK;
}
int launch_embed_row(__half* dst, const void* W, int type, int token, const int* d_token, int hidden, cudaStream_t st) {
    if (hidden <= 0 || hidden % QK_K) return set_error(JB_ERR_ARG, "embedding row: hidden=%d is not a multiple of 256", hidden);
    if (type != T_Q4K && type != T_Q6K) return set_error(JB_ERR_TYPE, "embedding row: ggml type %d", type);
    if (!dst || !W) return set_error(JB_ERR_PTR, "embedding row: null pointer");
    if (type == T_Q4K && ((uintptr_t)W & 3)) return set_error(JB_ERR_PTR, "embedding row: Q4_K table must be 4-byte aligned");
    JB_CUDA(launch_k(embed_row_kernel, dim3(hidden / QK_K), dim3(QK_K), 0, st, pdl_enabled(), dst, (const uint8_t*)W, type, d_token, token, hidden));
    count_launch();
    return JB_OK;
}

// ── dense GEMV / batched GEMV for F32/F16/BF16 weights (gemv_q4.cu:2811-2885) ─
__device__ __forceinline__ float dense_w(const void* W, int wtype, size_t i) {
    if (wtype == 0) return reinterpret_cast<const float*>(W)[i];
    if (wtype == 1) return __half2float(reinterpret_cast<const __half*>(W)[i]);
    return __uint_as_float((uint32_t)reinterpret_cast<const unsigned short*>(W)[i] << 16);
}
__global__ void dense_kernel(__half* out, const void* W, int wtype, const __half* x, int M, int N, int K) {
    pdl_wait();
    const int m = blockIdx.x * 4 + (threadIdx.x >> 5), n = blockIdx.y, lane = threadIdx.x & 31;
    if (m >= M || n >= N) return;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc += dense_w(W, wtype, (size_t)m * K + k) * __half2float(x[(size_t)n * K + k]);
    acc = warp_sum(acc);
    if (lane == 0) out[(size_t)n * M + m] = __float2half_rn(acc);
}
int launch_dense(__half* out, const void* W, int wtype, const __half* x, int M, int N, int K, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return JB_OK;
    if (wtype != 0 && wtype != 1 && wtype != 30) return set_error(JB_ERR_TYPE, "dense: weight type %d", wtype);
    if (!out || !W || !x) return set_error(JB_ERR_PTR, "dense: null pointer");
    JB_CUDA(launch_k(dense_kernel, dim3((M + 3) / 4, N), dim3(128), 0, st, pdl_enabled(), out, W, wtype, x, M, N, K));
    count_launch();
    return JB_OK;
}

// ── decode glue (extension): per-head RMSNorm of q and k, RoPE, int8 quantise K and V of
// the new position straight into the cache — the sequence Engine::transformer_layer_attn_compute
// runs as five launches (src/engine/decode.cu:1443-1478).  One warp per head.
struct QkvPrepArgs {
    __half* q; const __half* k; const __half* v;
    const float* q_norm; const float* k_norm; float eps;
    int8_t* k_cache; int8_t* v_cache; float* k_scales; float* v_scales;   // layer bases, position 0
    int n_heads, n_kv, hd, pos; const int* d_pos; int neox; int do_rope;
    // batch of independent streams at the same position (blockIdx.y = stream): activations q/k/v + y * stride, caches from lists
    int q_stride, kv_stride;
    int8_t* const* k_list; int8_t* const* v_list; float* const* ks_list; float* const* vs_list;
    int pos_step;       // prompt prefill: row y is the token at position pos + y * pos_step of ONE cache (lists null)
};
__global__ void qkv_prep_kernel(const QkvPrepArgs a, const __grid_constant__ RopeFreq fr) {
    pdl_wait();
    const int w = blockIdx.x * blockDim.y + threadIdx.y, lane = threadIdx.x;
    const int hd = a.hd, h2 = hd / 2;
    const int sq = blockIdx.y;
    const int pos = (a.d_pos ? *a.d_pos : a.pos) + sq * a.pos_step;
    if (w >= a.n_heads + 2 * a.n_kv) return;
    __half* qb = a.q + (size_t)sq * a.q_stride;
    const __half* kb = a.k + (size_t)sq * a.kv_stride; const __half* vb = a.v + (size_t)sq * a.kv_stride;
    int8_t* kcache = a.k_list ? a.k_list[sq] : a.k_cache; int8_t* vcache = a.k_list ? a.v_list[sq] : a.v_cache;
    float* kscales = a.k_list ? a.ks_list[sq] : a.k_scales; float* vscales = a.k_list ? a.vs_list[sq] : a.v_scales;
    extern __shared__ float sh[];
    float* buf = sh + (size_t)threadIdx.y * hd;
    const bool is_q = w < a.n_heads, is_k = !is_q && w < a.n_heads + a.n_kv;
    const int head = is_q ? w : (is_k ? w - a.n_heads : w - a.n_heads - a.n_kv);
    const __half* src = is_q ? qb + (size_t)head * hd : (is_k ? kb : vb) + (size_t)head * hd;
    if (is_q || is_k) {
        const float* nw = is_q ? a.q_norm : a.k_norm;
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) { const float v = __half2float(src[i]); ss += v * v; }
        if (nw) {
            ss = warp_sum(ss);
            const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hd), a.eps)));
            for (int i = lane; i < hd; i += 32)
                buf[i] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(__half2float(src[i]), rrms), nw[i])));
        } else {
            for (int i = lane; i < hd; i += 32) buf[i] = __half2float(src[i]);
        }
        __syncwarp();
        for (int pr = lane; a.do_rope && pr < h2; pr += 32) {
            const float ang = __fmul_rn((float)pos, fr.f[pr]);
            float c, s;
            sincosf(ang, &s, &c);          // one range reduction for both (and half the code of cosf + sinf)
            const int i0 = a.neox ? pr : 2 * pr, i1 = a.neox ? pr + h2 : 2 * pr + 1;
            const float v0 = buf[i0], v1 = buf[i1];
            const float r0 = __half2float(__float2half_rn(__fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s))));
            const float r1 = __half2float(__float2half_rn(__fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c))));
            buf[i0] = r0; buf[i1] = r1;
        }
        __syncwarp();
        if (is_q) { for (int i = lane; i < hd; i += 32) qb[(size_t)head * hd + i] = __float2half_rn(buf[i]); return; }
    } else {
        for (int i = lane; i < hd; i += 32) buf[i] = __half2float(src[i]);
        __syncwarp();
    }
    // K or V head: absmax quantise into the cache row of this position
    float mx = 0.f;
    for (int i = lane; i < hd; i += 32) mx = fmaxf(mx, fabsf(buf[i]));
    mx = warp_max(mx);
    const float scale = __fdiv_rn(mx, 127.0f), inv = scale > 0.f ? __fdiv_rn(127.0f, mx) : 0.f;
    int8_t* dst = (is_k ? kcache : vcache) + ((size_t)pos * a.n_kv + head) * hd;
    float* sc = (is_k ? kscales : vscales) + (size_t)pos * a.n_kv + head;
    if (lane == 0) *sc = scale;
    for (int i = lane; i < hd; i += 32) dst[i] = (int8_t)max(-127, min(127, __float2int_rn(__fmul_rn(buf[i], inv))));
}
int launch_qkv_prep(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                    int8_t* k_cache, int8_t* v_cache, float* k_scales, float* v_scales, int n_heads, int n_kv, int hd,
                    int pos, const int* d_pos, float theta, bool neox, bool do_rope, cudaStream_t st) {
    if (!q || !k || !v || !k_cache || !v_cache || !k_scales || !v_scales) return set_error(JB_ERR_PTR, "qkv_prep: null pointer");
    if (hd <= 0 || (hd & 1) || hd > 512) return set_error(JB_ERR_ARG, "qkv_prep: head_dim=%d", hd);
    QkvPrepArgs a = { q, k, v, q_norm, k_norm, eps, k_cache, v_cache, k_scales, v_scales, n_heads, n_kv, hd, pos, d_pos, (int)neox, (int)do_rope,
                      0, 0, nullptr, nullptr, nullptr, nullptr, 0 };
    const int warps = n_heads + 2 * n_kv;
    JB_CUDA(launch_k(qkv_prep_kernel, dim3((warps + 3) / 4), dim3(32, 4), (size_t)4 * hd * sizeof(float), st, pdl_enabled(), a, make_rope_freq(hd, theta)));
    count_launch();
    return JB_OK;
}

// the same for `batch` independent streams at one position: q [batch][n_heads*hd], k/v [batch][n_kv*hd], caches by list
int launch_qkv_prep_batched(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                            int8_t* const* k_list, int8_t* const* v_list, float* const* ks_list, float* const* vs_list, int batch,
                            int n_heads, int n_kv, int hd, const int* d_pos, float theta, bool neox, cudaStream_t st) {
    if (batch <= 0) return JB_OK;
    if (!q || !k || !v || !k_list || !v_list || !ks_list || !vs_list || !d_pos) return set_error(JB_ERR_PTR, "qkv_prep: null pointer");
    if (hd <= 0 || (hd & 1) || hd > 512) return set_error(JB_ERR_ARG, "qkv_prep: head_dim=%d", hd);
    QkvPrepArgs a = { q, k, v, q_norm, k_norm, eps, nullptr, nullptr, nullptr, nullptr, n_heads, n_kv, hd, 0, d_pos, (int)neox, 1,
                      n_heads * hd, n_kv * hd, k_list, v_list, ks_list, vs_list, 0 };
    const int warps = n_heads + 2 * n_kv;
    JB_CUDA(launch_k(qkv_prep_kernel, dim3((warps + 3) / 4, batch), dim3(32, 4), (size_t)4 * hd * sizeof(float), st, pdl_enabled(), a, make_rope_freq(hd, theta)));
    count_launch();
    return JB_OK;
}

// the same for the N tokens of a prompt chunk at positions start .. start+N-1 of one cache: q [N][n_heads*hd], k/v [N][n_kv*hd]
// (Engine::transformer_prefill's per-token RoPE + KV store loop, src/engine/decode.cu:1812-1846, in one launch)
int launch_qkv_prep_tokens(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                           int8_t* k_cache, int8_t* v_cache, float* k_scales, float* v_scales, int N, int n_heads, int n_kv, int hd,
                           int start_pos, float theta, bool neox, cudaStream_t st) {
    if (N <= 0) return JB_OK;
    if (!q || !k || !v || !k_cache || !v_cache || !k_scales || !v_scales) return set_error(JB_ERR_PTR, "qkv_prep: null pointer");
    if (hd <= 0 || (hd & 1) || hd > 512) return set_error(JB_ERR_ARG, "qkv_prep: head_dim=%d", hd);
    QkvPrepArgs a = { q, k, v, q_norm, k_norm, eps, k_cache, v_cache, k_scales, v_scales, n_heads, n_kv, hd, start_pos, nullptr, (int)neox, 1,
                      n_heads * hd, n_kv * hd, nullptr, nullptr, nullptr, nullptr, 1 };
    const int warps = n_heads + 2 * n_kv;
    JB_CUDA(launch_k(qkv_prep_kernel, dim3((warps + 3) / 4, N), dim3(32, 4), (size_t)4 * hd * sizeof(float), st, pdl_enabled(), a, make_rope_freq(hd, theta)));
    count_launch();
    return JB_OK;
}

// out = half(float(a) + float(b)), element-wise (the residual exit of a batched layer)
__global__ void add_half_kernel(__half* out, const __half* a, const __half* b, long long n) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(__fadd_rn(__half2float(a[i]), __half2float(b[i])));
}
__global__ void add_half8_kernel(__half* out, const __half* a, const __half* b, long long n8) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 av = reinterpret_cast<const uint4*>(a)[i], bv = reinterpret_cast<const uint4*>(b)[i];
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
    uint32_t ow[4];
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __half22float2(*reinterpret_cast<const __half2*>(&aw[k])), y = __half22float2(*reinterpret_cast<const __half2*>(&bw[k]));
        const __half2 h = __halves2half2(__float2half_rn(__fadd_rn(x.x, y.x)), __float2half_rn(__fadd_rn(x.y, y.y)));
        ow[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}
int launch_add_half(__half* out, const __half* a, const __half* b, long long n, cudaStream_t st) {
    if (n <= 0) return JB_OK;
    if (n >= 4096 && n % 8 == 0 && (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15) == 0) {
        JB_CUDA(launch_k(add_half8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, pdl_enabled(), out, a, b, n / 8));
        count_launch();
        return JB_OK;
    }
    JB_CUDA(launch_k(add_half_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, pdl_enabled(), out, a, b, n));
    count_launch();
    return JB_OK;
}

}  // namespace jb
