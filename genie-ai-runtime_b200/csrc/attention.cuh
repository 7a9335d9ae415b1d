// attention.cuh — host-side call block of the attention kernels.
#pragma once
#include "common.cuh"

namespace jb {

struct AttnCall {
    __half* out = nullptr; const __half* q = nullptr;
    const void* k = nullptr; const void* v = nullptr; const float* ks = nullptr; const float* vs = nullptr;
    // ragged batch: device arrays of per-sequence pointers / lengths (batch entries)
    const void* const* k_list = nullptr; const void* const* v_list = nullptr;
    const float* const* ks_list = nullptr; const float* const* vs_list = nullptr; const int* seq_lens = nullptr;
    // ragged batch on the TMA path: HOST array of [batch][K, V] tensor maps (built from the caches' addresses, see
    // jllm_b200_attn_plan_create; they travel to the kernel as parameters); the K/V pointer lists are then not needed
    const void* tma_maps = nullptr;
    int batch = 1, max_seq = 0;      // max_seq: rows every cache holds (bounds the slices of a ragged batch and the tensor maps)
    int n_heads = 0, n_kv = 0, hd = 0, chd = 0, seq_len = 0;
    const int* d_pos = nullptr;       // device position: seq_len = *d_pos + 1
    float scale = 1.f; int kv_int8 = 0, window = 0, n_splits = 0;
    int causal_start = -1;            // >= 0: prefill, `batch` = number of query tokens
};

int    attn_splits_for(int seq_len);
float* splitk_buffer(size_t floats, bool may_alloc);
int    launch_attention_general(const AttnCall& c, cudaStream_t st);
int    launch_attention(const AttnCall& c, cudaStream_t st);      // picks the fast path when it applies
int    launch_attn_reduce(__half* out, const float* part, int n_heads, int hd, int n_splits, int batch, cudaStream_t st);
unsigned int* attn_tickets();                                     // 65536 zeroed words per device (slice counters of the TMA kernel)
bool   attention_tma_applies(const AttnCall& c);                  // INT8 KV, head_dim 128, GQA 1/2/4, no window, cache extent known
int    launch_attention_tma(const AttnCall& c, cudaStream_t st);
bool   attn_tma_encode(void* map_out128, const void* cache_base, int rows, int n_kv);
bool   attention_prefill_fast_applies(const AttnCall& c);          // causal prefill (causal_start >= 0), INT8 KV, head_dim 128, GQA 1/2/4
int    launch_attention_prefill_fast(const AttnCall& c, cudaStream_t st);

}  // namespace jb
