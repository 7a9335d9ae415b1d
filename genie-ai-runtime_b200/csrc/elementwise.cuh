// elementwise.cuh — launchers of the small kernels (see elementwise.cu).
#pragma once
#include "common.cuh"

namespace jb {

struct RopeFreq { float f[256]; };      // 1/theta^(2i/hd) per rotation pair, computed on the host
RopeFreq make_rope_freq(int head_dim, float theta);

int launch_rmsnorm(__half* out, const __half* x, const __half* res, const void* w, bool w_fp32,
                   int rows, int dim, float eps, cudaStream_t st);
int launch_rope(__half* q, __half* k, const __half* v, __half* k_dst, __half* v_dst, int n_heads, int n_kv, int hd, int cache_hd,
                int pos, const int* d_pos, float theta, bool neox, int N, int q_stride, int k_stride, int kv_slot, bool dyn_cache,
                cudaStream_t st);
int rope_build_table(int max_seq, int head_dim, float theta);
void rope_free_tables();
int launch_glu(__half* out, const __half* gate, const __half* up, int rows, int dim, bool gelu, cudaStream_t st);
int launch_vec_scale(__half* x, int n, float s, cudaStream_t st);
int launch_softcap(float* x, int n, float cap, cudaStream_t st);
int launch_softmax(float* x, int n, cudaStream_t st);
int launch_fp16_to_int8(int8_t* dst, float* scale_out, const __half* src, int rows, int cols, cudaStream_t st);
int launch_embed_row(__half* dst, const void* W, int type, int token, const int* d_token, int hidden, cudaStream_t st);
int launch_dense(__half* out, const void* W, int wtype, const __half* x, int M, int N, int K, cudaStream_t st);
int launch_qkv_prep(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                    int8_t* k_cache, int8_t* v_cache, float* k_scales, float* v_scales, int n_heads, int n_kv, int hd,
                    int pos, const int* d_pos, float theta, bool neox, bool do_rope, cudaStream_t st);

int launch_embed_rows(__half* dst, const void* W, int type, const int* d_tokens, int rows, int hidden, cudaStream_t st);
int launch_qkv_prep_batched(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                            int8_t* const* k_list, int8_t* const* v_list, float* const* ks_list, float* const* vs_list, int batch,
                            int n_heads, int n_kv, int hd, const int* d_pos, float theta, bool neox, cudaStream_t st);
int launch_qkv_prep_tokens(__half* q, const __half* k, const __half* v, const float* q_norm, const float* k_norm, float eps,
                           int8_t* k_cache, int8_t* v_cache, float* k_scales, float* v_scales, int N, int n_heads, int n_kv, int hd,
                           int start_pos, float theta, bool neox, cudaStream_t st);
int launch_add_half(__half* out, const __half* a, const __half* b, long long n, cudaStream_t st);

}  // namespace jb
