// pools.cpp — jllm::KVCachePool and jllm::ScratchPool for a discrete-memory GPU.
//
// Behaviour follows the reference pools (src/memory/kv_cache.cpp:20-281, src/memory/pool.cpp:9-59):
// same slab layout, same pointer arithmetic, same return values; the classes keep the reference's
// object layout (see include/jllm_b200_api.hpp).  Gather / scatter move all layers with one
// strided copy each for keys and values instead of two copies per layer.
#include "../../include/jllm_b200_api.hpp"
#include "../../include/jllm_b200.h"
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

namespace jllm {

bool KVCachePool::init(const Config& cfg) {
    cfg_ = cfg;
    gpu_pool_ = nullptr; cpu_pool_ = nullptr; kv_scales_ = nullptr;
    used_tokens_ = gpu_tokens_ = 0;
    const int64_t fast = (int64_t)cfg.n_layers * entry_bytes() * cfg.max_context;
    const int64_t over = (int64_t)cfg.n_layers * entry_bytes() * cfg.overflow_context;
    if (fast <= 0) { fprintf(stderr, "[kv_cache] invalid configuration\n"); return false; }
    if (cudaMalloc(&gpu_pool_, (size_t)fast) != cudaSuccess) {
        fprintf(stderr, "[kv_cache] cudaMalloc(%lld B) failed: %s\n", (long long)fast, cudaGetErrorString(cudaGetLastError()));
        gpu_pool_ = nullptr;
        return false;
    }
    if (cudaMemset(gpu_pool_, 0, (size_t)fast) != cudaSuccess) { cudaFree(gpu_pool_); gpu_pool_ = nullptr; return false; }
    if (cfg.overflow_context > 0 && over > 0) {
        cpu_pool_ = calloc(1, (size_t)over);
        if (!cpu_pool_) { fprintf(stderr, "[kv_cache] overflow pool unavailable, disabled\n"); cfg_.overflow_context = 0; }
    }
    if (cfg.kv_type_bytes == 1) {
        const int64_t sb = kv_scales_bytes();
        if (cudaMalloc(&kv_scales_, (size_t)sb) != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "[kv_cache] scale slab (%lld B) unavailable; INT8 KV cannot be used\n", (long long)sb);
            kv_scales_ = nullptr;          // like the reference: init still succeeds, kv_scale_ptr() returns null
        } else {
            cudaMemset(kv_scales_, 0, (size_t)sb);
        }
    }
    return true;
}

void KVCachePool::destroy() {
    if (gpu_pool_) cudaFree(gpu_pool_);
    if (cpu_pool_) free(cpu_pool_);
    if (kv_scales_) cudaFree(kv_scales_);
    gpu_pool_ = cpu_pool_ = nullptr; kv_scales_ = nullptr;
    used_tokens_ = gpu_tokens_ = 0;
}

// Per layer: keys for every position, then values for every position (kv_cache.cpp:96-120).
static inline char* slab_ptr(void* pool, int layer, int pos, int ctx, int64_t entry, bool value) {
    const int64_t half = entry / 2;
    return (char*)pool + (int64_t)layer * ctx * entry + (value ? (int64_t)ctx * half : 0) + (int64_t)pos * half;
}
void* KVCachePool::key_ptr(int layer, int pos) {
    return pos < cfg_.max_context ? slab_ptr(gpu_pool_, layer, pos, cfg_.max_context, entry_bytes(), false)
                                  : slab_ptr(cpu_pool_, layer, pos - cfg_.max_context, cfg_.overflow_context, entry_bytes(), false);
}
void* KVCachePool::val_ptr(int layer, int pos) {
    return pos < cfg_.max_context ? slab_ptr(gpu_pool_, layer, pos, cfg_.max_context, entry_bytes(), true)
                                  : slab_ptr(cpu_pool_, layer, pos - cfg_.max_context, cfg_.overflow_context, entry_bytes(), true);
}

int64_t KVCachePool::used_bytes() const { return (int64_t)used_tokens_ * entry_bytes() * cfg_.n_layers; }
int64_t KVCachePool::capacity_bytes() const { return (int64_t)(cfg_.max_context + cfg_.overflow_context) * entry_bytes() * cfg_.n_layers; }

// Oldest n tokens of the fast pool go to the host pool, the rest shifts down (kv_cache.cpp:130-152).
void KVCachePool::evict(int n_tokens) {
    if (!cpu_pool_ || n_tokens <= 0) return;
    const int64_t eb = entry_bytes();
    for (int l = 0; l < cfg_.n_layers; ++l) {
        char* src = (char*)gpu_pool_ + (int64_t)l * cfg_.max_context * eb;
        char* dst = (char*)cpu_pool_ + (int64_t)l * cfg_.overflow_context * eb;
        cudaMemcpy(dst, src, (size_t)n_tokens * eb, cudaMemcpyDeviceToHost);
        const int rest = gpu_tokens_ - n_tokens;
        if (rest > 0) cudaMemcpy(src, src + (int64_t)n_tokens * eb, (size_t)rest * eb, cudaMemcpyDeviceToDevice);
    }
    gpu_tokens_ -= n_tokens;
}

void KVCachePool::clear() { used_tokens_ = gpu_tokens_ = 0; }

// Packed host image: per layer [used keys][used values] (kv_cache.cpp:169-253).
bool KVCachePool::gather_used_to_host(void* dst, int used) const {
    if (!gpu_pool_ || used <= 0 || used > cfg_.max_context) return false;
    const int64_t eb = entry_bytes(), half = eb / 2;
    const size_t width = (size_t)used * half;
    const char* keys = (const char*)gpu_pool_;
    const char* vals = keys + (int64_t)cfg_.max_context * half;
    char* d = (char*)dst;
    if (cudaMemcpy2D(d, (size_t)used * eb, keys, (size_t)cfg_.max_context * eb, width, cfg_.n_layers, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    if (cudaMemcpy2D(d + width, (size_t)used * eb, vals, (size_t)cfg_.max_context * eb, width, cfg_.n_layers, cudaMemcpyDeviceToHost) != cudaSuccess) return false;
    return true;
}
bool KVCachePool::scatter_from_host(const void* src, int used, bool zero_remaining) {
    if (!gpu_pool_ || used <= 0 || used > cfg_.max_context) return false;
    const int64_t eb = entry_bytes(), half = eb / 2;
    const size_t width = (size_t)used * half, rest = (size_t)(cfg_.max_context - used) * half;
    char* keys = (char*)gpu_pool_;
    char* vals = keys + (int64_t)cfg_.max_context * half;
    const char* s = (const char*)src;
    if (cudaMemcpy2D(keys, (size_t)cfg_.max_context * eb, s, (size_t)used * eb, width, cfg_.n_layers, cudaMemcpyHostToDevice) != cudaSuccess) return false;
    if (cudaMemcpy2D(vals, (size_t)cfg_.max_context * eb, s + width, (size_t)used * eb, width, cfg_.n_layers, cudaMemcpyHostToDevice) != cudaSuccess) return false;
    if (zero_remaining && rest > 0) {
        if (cudaMemset2D(keys + width, (size_t)cfg_.max_context * eb, 0, rest, cfg_.n_layers) != cudaSuccess) return false;
        if (cudaMemset2D(vals + width, (size_t)cfg_.max_context * eb, 0, rest, cfg_.n_layers) != cudaSuccess) return false;
    }
    used_tokens_ = gpu_tokens_ = used;
    return true;
}

int64_t KVCachePool::kv_scales_bytes() const {
    return cfg_.kv_type_bytes != 1 ? 0 : 2LL * cfg_.n_layers * cfg_.max_context * cfg_.n_kv_heads * (int64_t)sizeof(float);
}
// Per layer: [K scales: ctx x n_kv][V scales: ctx x n_kv] (kv_cache.cpp:257-281).
float* KVCachePool::kv_scale_ptr(int layer, int pos, bool is_value) {
    if (!kv_scales_ || cfg_.kv_type_bytes != 1) return nullptr;
    if (layer < 0 || layer >= cfg_.n_layers || pos < 0 || pos >= cfg_.max_context) return nullptr;
    const int64_t region = (int64_t)cfg_.max_context * cfg_.n_kv_heads;
    return kv_scales_ + (int64_t)layer * 2 * region + (is_value ? region : 0) + (int64_t)pos * cfg_.n_kv_heads;
}

bool ScratchPool::init(int64_t size_bytes) {
    base_ = nullptr; capacity_ = offset_ = 0;
    if (size_bytes <= 0 || cudaMalloc(&base_, (size_t)size_bytes) != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "[scratch] cudaMalloc(%lld B) failed\n", (long long)size_bytes);
        base_ = nullptr;
        return false;
    }
    capacity_ = size_bytes;
    return true;
}
void ScratchPool::destroy() { if (base_) cudaFree(base_); base_ = nullptr; capacity_ = offset_ = 0; }
void* ScratchPool::get(int64_t size) {
    const int64_t need = (size + 255) & ~255LL;
    if (offset_ + need > capacity_) {
        fprintf(stderr, "[scratch] pool exhausted (%lld of %lld B)\n", (long long)(offset_ + need), (long long)capacity_);
        return nullptr;
    }
    void* p = (char*)base_ + offset_;
    offset_ += need;
    return p;
}
void ScratchPool::reset() { offset_ = 0; }
void ScratchPool::rewind_to(int64_t saved) { if (saved >= 0 && saved <= capacity_) offset_ = saved; }

}  // namespace jllm

// ── C handles ───────────────────────────────────────────────────────────
struct jllm_b200_kv_pool { jllm::KVCachePool pool; };
struct jllm_b200_scratch { jllm::ScratchPool pool; };

extern "C" {
jllm_b200_kv_pool* jllm_b200_kv_pool_create(int n_layers, int n_kv_heads, int head_dim, int max_context, int overflow_context, int kv_type_bytes) {
    jllm_b200_kv_pool* h = new (std::nothrow) jllm_b200_kv_pool();
    if (!h) return nullptr;
    jllm::KVCachePool::Config c = { n_layers, n_kv_heads, head_dim, max_context, overflow_context, kv_type_bytes };
    if (!h->pool.init(c)) { delete h; return nullptr; }
    return h;
}
void    jllm_b200_kv_pool_destroy(jllm_b200_kv_pool* p) { if (p) { p->pool.destroy(); delete p; } }
void*   jllm_b200_kv_pool_key_ptr(jllm_b200_kv_pool* p, int layer, int pos) { return p->pool.key_ptr(layer, pos); }
void*   jllm_b200_kv_pool_val_ptr(jllm_b200_kv_pool* p, int layer, int pos) { return p->pool.val_ptr(layer, pos); }
float*  jllm_b200_kv_pool_scale_ptr(jllm_b200_kv_pool* p, int layer, int pos, int is_value) { return p->pool.kv_scale_ptr(layer, pos, is_value != 0); }
int64_t jllm_b200_kv_pool_scales_bytes(jllm_b200_kv_pool* p) { return p->pool.kv_scales_bytes(); }
int64_t jllm_b200_kv_pool_capacity_bytes(jllm_b200_kv_pool* p) { return p->pool.capacity_bytes(); }
int64_t jllm_b200_kv_pool_used_bytes(jllm_b200_kv_pool* p) { return p->pool.used_bytes(); }
int64_t jllm_b200_kv_pool_packed_used_bytes(jllm_b200_kv_pool* p, int used_tokens) { return p->pool.packed_used_bytes(used_tokens); }
int     jllm_b200_kv_pool_gather_used_to_host(jllm_b200_kv_pool* p, void* dst, int used) { return p->pool.gather_used_to_host(dst, used) ? 0 : JLLM_B200_ERR_ARG; }
int     jllm_b200_kv_pool_scatter_from_host(jllm_b200_kv_pool* p, const void* src, int used, int zero_remaining) { return p->pool.scatter_from_host(src, used, zero_remaining != 0) ? 0 : JLLM_B200_ERR_ARG; }
int     jllm_b200_kv_pool_used_tokens(jllm_b200_kv_pool* p) { return p->pool.used_tokens(); }
void    jllm_b200_kv_pool_clear(jllm_b200_kv_pool* p) { p->pool.clear(); }
jllm_b200_scratch* jllm_b200_scratch_create(int64_t size_bytes) {
    jllm_b200_scratch* h = new (std::nothrow) jllm_b200_scratch();
    if (!h) return nullptr;
    if (!h->pool.init(size_bytes)) { delete h; return nullptr; }
    return h;
}
void    jllm_b200_scratch_destroy(jllm_b200_scratch* s) { if (s) { s->pool.destroy(); delete s; } }
void*   jllm_b200_scratch_get(jllm_b200_scratch* s, int64_t size) { return s->pool.get(size); }
void    jllm_b200_scratch_reset(jllm_b200_scratch* s) { s->pool.reset(); }
int64_t jllm_b200_scratch_mark(jllm_b200_scratch* s) { return s->pool.mark(); }
void    jllm_b200_scratch_rewind_to(jllm_b200_scratch* s, int64_t saved) { s->pool.rewind_to(saved); }
int64_t jllm_b200_scratch_used(jllm_b200_scratch* s) { return s->pool.used(); }
int64_t jllm_b200_scratch_capacity(jllm_b200_scratch* s) { return s->pool.capacity(); }
}
