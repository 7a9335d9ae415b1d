"""Mirror of the reference's memory pools (include/jllm_memory.h:104-222) over the C handles."""
from __future__ import annotations

import ctypes as C

from . import lib


class KVCachePool:
    """Pre-allocated KV slab: per layer [K: ctx x n_kv*hd*bytes][V: same]; INT8 mode adds fp32 scales
    per layer [K: ctx x n_kv][V: same].  Pointers are returned as integer device addresses."""

    def __init__(self):
        self._h = None
        self.cfg = None

    def init(self, n_layers, n_kv_heads, head_dim, max_context, overflow_context=0, kv_type_bytes=1):
        self._h = lib.jllm_b200_kv_pool_create(n_layers, n_kv_heads, head_dim, max_context, overflow_context, kv_type_bytes)
        self.cfg = dict(n_layers=n_layers, n_kv_heads=n_kv_heads, head_dim=head_dim, max_context=max_context,
                        overflow_context=overflow_context, kv_type_bytes=kv_type_bytes)
        return self._h is not None

    def destroy(self):
        if self._h:
            lib.jllm_b200_kv_pool_destroy(C.c_void_p(self._h))
            self._h = None

    def key_ptr(self, layer, pos):
        return lib.jllm_b200_kv_pool_key_ptr(C.c_void_p(self._h), layer, pos)

    def val_ptr(self, layer, pos):
        return lib.jllm_b200_kv_pool_val_ptr(C.c_void_p(self._h), layer, pos)

    def kv_scale_ptr(self, layer, pos, is_value):
        return lib.jllm_b200_kv_pool_scale_ptr(C.c_void_p(self._h), layer, pos, 1 if is_value else 0)

    def kv_scales_bytes(self):
        return int(lib.jllm_b200_kv_pool_scales_bytes(C.c_void_p(self._h)))

    def capacity_bytes(self):
        return int(lib.jllm_b200_kv_pool_capacity_bytes(C.c_void_p(self._h)))

    def used_bytes(self):
        return int(lib.jllm_b200_kv_pool_used_bytes(C.c_void_p(self._h)))

    def packed_used_bytes(self, used_tokens):
        return int(lib.jllm_b200_kv_pool_packed_used_bytes(C.c_void_p(self._h), used_tokens))

    def gather_used_to_host(self, host_array, used_tokens):
        return lib.jllm_b200_kv_pool_gather_used_to_host(C.c_void_p(self._h), host_array.ctypes.data_as(C.c_void_p), used_tokens) == 0

    def scatter_from_host(self, host_array, used_tokens, zero_remaining):
        return lib.jllm_b200_kv_pool_scatter_from_host(C.c_void_p(self._h), host_array.ctypes.data_as(C.c_void_p), used_tokens,
                                                       1 if zero_remaining else 0) == 0

    def used_tokens(self):
        return int(lib.jllm_b200_kv_pool_used_tokens(C.c_void_p(self._h)))

    def clear(self):
        lib.jllm_b200_kv_pool_clear(C.c_void_p(self._h))


class ScratchPool:
    """256-byte aligned bump allocator over one device allocation."""

    def __init__(self):
        self._h = None

    def init(self, size_bytes):
        self._h = lib.jllm_b200_scratch_create(C.c_int64(size_bytes))
        return self._h is not None

    def destroy(self):
        if self._h:
            lib.jllm_b200_scratch_destroy(C.c_void_p(self._h))
            self._h = None

    def get(self, size):
        return lib.jllm_b200_scratch_get(C.c_void_p(self._h), C.c_int64(size))

    def reset(self):
        lib.jllm_b200_scratch_reset(C.c_void_p(self._h))

    def mark(self):
        return int(lib.jllm_b200_scratch_mark(C.c_void_p(self._h)))

    def rewind_to(self, saved):
        lib.jllm_b200_scratch_rewind_to(C.c_void_p(self._h), C.c_int64(saved))

    def used(self):
        return int(lib.jllm_b200_scratch_used(C.c_void_p(self._h)))

    def capacity(self):
        return int(lib.jllm_b200_scratch_capacity(C.c_void_p(self._h)))
