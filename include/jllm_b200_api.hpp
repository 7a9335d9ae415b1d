// jllm_b200_api.hpp — the C++ face of the library: functions and classes in namespace
// `jllm` with the same names, parameter types and therefore the same mangled symbols as
// the reference's include/jllm_kernels.h and include/jllm_memory.h.  The reference engine
// is compiled against ITS OWN headers; this header exists so that this library defines
// those symbols and so that C++ callers without the reference tree can use them.
//
// Each declaration cites the reference declaration it stands in for
// (K = include/jllm_kernels.h, M = include/jllm_memory.h).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace jllm {

// K:40-43 — host-mmap -> device alias registry (pass-through for device pointers)
const void* resolve_mapped_weight_device_ptr(const void* host_ptr);
void register_mapped_weight_region(const void* host_base, const void* device_base, int64_t bytes);
void clear_mapped_weight_region(const void* host_base);

// K:51-60, K:64-72, K:78-87, K:92-104, K:106-122, K:135-144, K:148-156, K:160-167
void gemv_q4(half* y, const void* W_q4, const half* scales, const half* x, int M, int K, int group_size, cudaStream_t stream);
void gemv_quant(half* y, const void* W, int ggml_type, const half* x, int M, int K, cudaStream_t stream);
void gemv_quant_add(half* y, const void* W, int ggml_type, const half* x, const half* residual, int M, int K, cudaStream_t stream);
void gemv_quant_pair(half* y0, const void* W0, int ggml_type0, int M0, half* y1, const void* W1, int ggml_type1, int M1,
                     const half* x, int K, cudaStream_t stream);
void gemv_quant_triple(half* y0, const void* W0, int ggml_type0, int M0, half* y1, const void* W1, int ggml_type1, int M1,
                       half* y2, const void* W2, int ggml_type2, int M2, const half* x, int K, cudaStream_t stream);
void gemm_quant_batched(half* y, const void* W, int ggml_type, const half* x, int M, int N, int K, cudaStream_t stream);
void gemv_quant_f32(float* y, const void* W, int ggml_type, const half* x, int M, int K, cudaStream_t stream);
bool dequant_embedding_row(half* dst, const void* W, int ggml_type, int token_id, int hidden_dim, cudaStream_t stream);

// K:174-184, K:191-216, K:220-227
void fused_rmsnorm_residual(half* output, const half* x, const half* residual, const void* weight, int rows, int hidden_dim,
                            float eps, bool weight_fp32, cudaStream_t stream);
void fused_swiglu(half* output, const half* gate, const half* up, int rows, int intermediate_dim, cudaStream_t stream);
void fused_geglu(half* output, const half* gate, const half* up, int rows, int intermediate_dim, cudaStream_t stream);
void vec_scale(half* x, int n, float s, cudaStream_t stream);
void logit_softcap(float* x, int n, float cap, cudaStream_t stream);
void gemv_dense(half* out, const void* W, int wtype, const half* x, int M, int K, cudaStream_t stream);
void gemm_dense_batched(half* out, const void* W, int wtype, const half* x, int M, int N, int K, cudaStream_t stream);

// K:238-316
void rope_precompute_table(int max_seq, int head_dim, float theta_base);
void rope_clear_tables();
void rope_inplace(half* q, half* k, int n_heads, int n_kv_heads, int head_dim, int position, float theta_base, bool neox,
                  cudaStream_t stream);
void rope_inplace_store_kv_fp16(half* q, half* k, const half* v, half* k_cache_dst, half* v_cache_dst, int n_heads,
                                int n_kv_heads, int head_dim, int position, float theta_base, bool neox, cudaStream_t stream);
void rope_inplace_batched(half* q, half* k, int n_heads, int n_kv_heads, int head_dim, int start_pos, int N, int q_stride,
                          int k_stride, float theta_base, bool neox, cudaStream_t stream);
void rope_inplace_store_kv_fp16_batched(half* q, half* k, const half* v, half* k_cache_base, half* v_cache_base, int kv_slot,
                                        int n_heads, int n_kv_heads, int head_dim, int start_pos, int N, int q_stride,
                                        int kv_stride, float theta_base, bool neox, cudaStream_t stream);
void rope_inplace_store_kv_fp16_dyn(half* q, half* k, const half* v, half* k_cache_layer_base, half* v_cache_layer_base,
                                    int n_heads, int n_kv_heads, int head_dim, int cache_head_dim, const int* d_pos,
                                    float theta_base, bool neox, cudaStream_t stream);
void rope_inplace_dyn(half* q, half* k, int n_heads, int n_kv_heads, int head_dim, const int* d_pos, float theta_base, bool neox,
                      cudaStream_t stream);

// K:323-342, K:354-373, K:380-396, K:402-403
void flash_attention_decode(half* output, const half* q, const void* k_cache, const void* v_cache, int n_heads, int n_kv_heads,
                            int head_dim, int cache_head_dim, int seq_len, float scale, bool kv_int8, const float* k_scales,
                            const float* v_scales, int window, cudaStream_t stream);
void flash_attention_prefill_batched(half* output, const half* q, const void* k_cache, const void* v_cache, int n_heads,
                                     int n_kv_heads, int head_dim, int cache_head_dim, int N, int start_pos, float scale,
                                     bool kv_int8, const float* k_scales, const float* v_scales, int window, cudaStream_t stream);
void flash_attention_decode_dyn(half* output, const half* q, const void* k_cache, const void* v_cache, int n_heads, int n_kv_heads,
                                int head_dim, int cache_head_dim, const int* d_pos, float scale, bool kv_int8,
                                const float* kv_scales, int window, int n_splits, cudaStream_t stream);
int    decode_attn_splits(int seq_len);
float* get_splitk_partials(int n_heads, int n_splits, int head_dim);

// K:406-420
void softmax_inplace(float* x, int n, cudaStream_t stream);
void fp16_to_int8(int8_t* dst, float* scale_out, const half* src, int rows, int cols, cudaStream_t stream);

// M:104-197 — KV cache: per layer [K: ctx x (n_kv*hd*bytes)][V: same]; INT8 mode adds an fp32
// scale slab, per layer [K: ctx x n_kv][V: same].  Member order and types match the reference
// object (the engine embeds the pool by value, include/jllm_engine.h:306-307).
class KVCachePool {
public:
    struct Config {
        int n_layers;
        int n_kv_heads;
        int head_dim;
        int max_context;
        int overflow_context;
        int kv_type_bytes;      // 1 = INT8, 2 = FP16
    };
    bool  init(const Config& cfg);
    void  destroy();
    void* key_ptr(int layer, int pos);
    void* val_ptr(int layer, int pos);
    int64_t used_bytes() const;
    int64_t capacity_bytes() const;
    int  used_tokens() const { return used_tokens_; }
    int  max_tokens() const { return cfg_.max_context + cfg_.overflow_context; }
    bool is_fast_position(int pos) const { return pos < cfg_.max_context; }
    void evict(int n_tokens);
    void clear();
    const Config& config() const { return cfg_; }
    void*   gpu_pool_ptr() const { return gpu_pool_; }
    int64_t gpu_pool_bytes() const { return (int64_t)cfg_.n_layers * cfg_.max_context * entry_bytes(); }
    int64_t packed_used_bytes(int used_tokens) const {
        return used_tokens <= 0 ? 0 : (int64_t)cfg_.n_layers * used_tokens * entry_bytes();
    }
    bool gather_used_to_host(void* dst, int used_tokens) const;
    bool scatter_from_host(const void* src, int used_tokens, bool zero_remaining);
    float*  kv_scale_ptr(int layer, int pos, bool is_value);
    int64_t kv_scales_bytes() const;

private:
    Config cfg_ = {};
    void*  gpu_pool_ = nullptr;
    void*  cpu_pool_ = nullptr;
    float* kv_scales_ = nullptr;
    int    used_tokens_ = 0;
    int    gpu_tokens_ = 0;
    int64_t entry_bytes() const { return 2LL * cfg_.n_kv_heads * cfg_.head_dim * cfg_.kv_type_bytes; }
    int64_t layer_stride() const { return entry_bytes() * (cfg_.max_context + cfg_.overflow_context); }
};

// M:201-222 — 256-byte aligned bump allocator over one device allocation.
class ScratchPool {
public:
    bool  init(int64_t size_bytes);
    void  destroy();
    void* get(int64_t size);
    void  reset();
    int64_t mark() const { return offset_; }
    void    rewind_to(int64_t saved_offset);
    int64_t used() const { return offset_; }
    int64_t capacity() const { return capacity_; }

private:
    void*   base_ = nullptr;
    int64_t capacity_ = 0;
    int64_t offset_ = 0;
};

}  // namespace jllm
