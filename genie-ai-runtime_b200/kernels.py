"""Mirror of the reference's kernel functions (include/jllm_kernels.h), one Python function each.

Tensors must live on the current CUDA device; activations are torch.float16, weights are
uint8 images of GGUF K-quant blocks, logits float32.  `stream` defaults to torch's current stream.
"""
from __future__ import annotations

import ctypes as C

from . import lib, _ptr, _stream, check

i32, f32 = C.c_int, C.c_float


def gemv_quant(y, W, ggml_type, x, M, K, stream=None):
    check(lib.jllm_b200_gemv_quant(_ptr(y), _ptr(W), i32(ggml_type), _ptr(x), i32(M), i32(K), _stream(stream)))


def gemv_q4(y, W_q4, scales, x, M, K, group_size, stream=None):
    check(lib.jllm_b200_gemv_q4(_ptr(y), _ptr(W_q4), _ptr(scales), _ptr(x), i32(M), i32(K), i32(group_size), _stream(stream)))


def gemv_quant_add(y, W, ggml_type, x, residual, M, K, stream=None):
    check(lib.jllm_b200_gemv_quant_add(_ptr(y), _ptr(W), i32(ggml_type), _ptr(x), _ptr(residual), i32(M), i32(K), _stream(stream)))


def gemv_quant_pair(y0, W0, t0, M0, y1, W1, t1, M1, x, K, stream=None):
    check(lib.jllm_b200_gemv_quant_pair(_ptr(y0), _ptr(W0), i32(t0), i32(M0), _ptr(y1), _ptr(W1), i32(t1), i32(M1),
                                        _ptr(x), i32(K), _stream(stream)))


def gemv_quant_triple(y0, W0, t0, M0, y1, W1, t1, M1, y2, W2, t2, M2, x, K, stream=None):
    check(lib.jllm_b200_gemv_quant_triple(_ptr(y0), _ptr(W0), i32(t0), i32(M0), _ptr(y1), _ptr(W1), i32(t1), i32(M1),
                                          _ptr(y2), _ptr(W2), i32(t2), i32(M2), _ptr(x), i32(K), _stream(stream)))


def gemv_quant_f32(y, W, ggml_type, x, M, K, stream=None):
    check(lib.jllm_b200_gemv_quant_f32(_ptr(y), _ptr(W), i32(ggml_type), _ptr(x), i32(M), i32(K), _stream(stream)))


def gemm_quant_batched(y, W, ggml_type, x, M, N, K, stream=None):
    check(lib.jllm_b200_gemm_quant_batched(_ptr(y), _ptr(W), i32(ggml_type), _ptr(x), i32(M), i32(N), i32(K), _stream(stream)))


def dequant_embedding_row(dst, W, ggml_type, token_id, hidden_dim, stream=None):
    """Returns True on success, like the reference."""
    return lib.jllm_b200_dequant_embedding_row(_ptr(dst), _ptr(W), i32(ggml_type), i32(token_id), i32(hidden_dim), _stream(stream)) == 0


def gemv_dense(out, W, wtype, x, M, K, stream=None):
    check(lib.jllm_b200_gemv_dense(_ptr(out), _ptr(W), i32(wtype), _ptr(x), i32(M), i32(K), _stream(stream)))


def gemm_dense_batched(out, W, wtype, x, M, N, K, stream=None):
    check(lib.jllm_b200_gemm_dense_batched(_ptr(out), _ptr(W), i32(wtype), _ptr(x), i32(M), i32(N), i32(K), _stream(stream)))


def fused_rmsnorm_residual(output, x, residual, weight, rows, hidden_dim, eps, weight_fp32, stream=None):
    check(lib.jllm_b200_fused_rmsnorm_residual(_ptr(output), _ptr(x), _ptr(residual), _ptr(weight), i32(rows), i32(hidden_dim),
                                               f32(eps), i32(1 if weight_fp32 else 0), _stream(stream)))


def fused_swiglu(output, gate, up, rows, intermediate_dim, stream=None):
    check(lib.jllm_b200_fused_swiglu(_ptr(output), _ptr(gate), _ptr(up), i32(rows), i32(intermediate_dim), _stream(stream)))


def fused_geglu(output, gate, up, rows, intermediate_dim, stream=None):
    check(lib.jllm_b200_fused_geglu(_ptr(output), _ptr(gate), _ptr(up), i32(rows), i32(intermediate_dim), _stream(stream)))


def vec_scale(x, n, s, stream=None):
    check(lib.jllm_b200_vec_scale(_ptr(x), i32(n), f32(s), _stream(stream)))


def logit_softcap(x, n, cap, stream=None):
    check(lib.jllm_b200_logit_softcap(_ptr(x), i32(n), f32(cap), _stream(stream)))


def softmax_inplace(x, n, stream=None):
    check(lib.jllm_b200_softmax_inplace(_ptr(x), i32(n), _stream(stream)))


def fp16_to_int8(dst, scale_out, src, rows, cols, stream=None):
    check(lib.jllm_b200_fp16_to_int8(_ptr(dst), _ptr(scale_out), _ptr(src), i32(rows), i32(cols), _stream(stream)))


def rope_precompute_table(max_seq, head_dim, theta_base):
    check(lib.jllm_b200_rope_precompute_table(i32(max_seq), i32(head_dim), f32(theta_base)))


def rope_clear_tables():
    check(lib.jllm_b200_rope_clear_tables())


def rope_inplace(q, k, n_heads, n_kv_heads, head_dim, position, theta_base, neox, stream=None):
    check(lib.jllm_b200_rope_inplace(_ptr(q), _ptr(k), i32(n_heads), i32(n_kv_heads), i32(head_dim), i32(position), f32(theta_base),
                                     i32(1 if neox else 0), _stream(stream)))


def rope_inplace_store_kv_fp16(q, k, v, k_cache_dst, v_cache_dst, n_heads, n_kv_heads, head_dim, position, theta_base, neox, stream=None):
    check(lib.jllm_b200_rope_inplace_store_kv_fp16(_ptr(q), _ptr(k), _ptr(v), _ptr(k_cache_dst), _ptr(v_cache_dst), i32(n_heads),
                                                   i32(n_kv_heads), i32(head_dim), i32(position), f32(theta_base), i32(1 if neox else 0),
                                                   _stream(stream)))


def rope_inplace_batched(q, k, n_heads, n_kv_heads, head_dim, start_pos, N, q_stride, k_stride, theta_base, neox, stream=None):
    check(lib.jllm_b200_rope_inplace_batched(_ptr(q), _ptr(k), i32(n_heads), i32(n_kv_heads), i32(head_dim), i32(start_pos), i32(N),
                                             i32(q_stride), i32(k_stride), f32(theta_base), i32(1 if neox else 0), _stream(stream)))


def rope_inplace_dyn(q, k, n_heads, n_kv_heads, head_dim, d_pos, theta_base, neox, stream=None):
    check(lib.jllm_b200_rope_inplace_dyn(_ptr(q), _ptr(k), i32(n_heads), i32(n_kv_heads), i32(head_dim), _ptr(d_pos), f32(theta_base),
                                         i32(1 if neox else 0), _stream(stream)))


def rope_inplace_store_kv_fp16_dyn(q, k, v, k_base, v_base, n_heads, n_kv_heads, head_dim, cache_head_dim, d_pos, theta_base, neox, stream=None):
    check(lib.jllm_b200_rope_inplace_store_kv_fp16_dyn(_ptr(q), _ptr(k), _ptr(v), _ptr(k_base), _ptr(v_base), i32(n_heads), i32(n_kv_heads),
                                                       i32(head_dim), i32(cache_head_dim), _ptr(d_pos), f32(theta_base),
                                                       i32(1 if neox else 0), _stream(stream)))


def flash_attention_decode(output, q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, cache_head_dim, seq_len, scale, kv_int8,
                           k_scales, v_scales, window, stream=None):
    check(lib.jllm_b200_flash_attention_decode(_ptr(output), _ptr(q), _ptr(k_cache), _ptr(v_cache), i32(n_heads), i32(n_kv_heads),
                                               i32(head_dim), i32(cache_head_dim), i32(seq_len), f32(scale), i32(1 if kv_int8 else 0),
                                               _ptr(k_scales), _ptr(v_scales), i32(window), _stream(stream)))


def flash_attention_prefill_batched(output, q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, cache_head_dim, N, start_pos, scale,
                                    kv_int8, k_scales, v_scales, window, stream=None):
    check(lib.jllm_b200_flash_attention_prefill_batched(_ptr(output), _ptr(q), _ptr(k_cache), _ptr(v_cache), i32(n_heads), i32(n_kv_heads),
                                                        i32(head_dim), i32(cache_head_dim), i32(N), i32(start_pos), f32(scale),
                                                        i32(1 if kv_int8 else 0), _ptr(k_scales), _ptr(v_scales), i32(window),
                                                        _stream(stream)))


def flash_attention_decode_dyn(output, q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, cache_head_dim, d_pos, scale, kv_int8,
                               kv_scales, window, n_splits, stream=None):
    check(lib.jllm_b200_flash_attention_decode_dyn(_ptr(output), _ptr(q), _ptr(k_cache), _ptr(v_cache), i32(n_heads), i32(n_kv_heads),
                                                   i32(head_dim), i32(cache_head_dim), _ptr(d_pos), f32(scale), i32(1 if kv_int8 else 0),
                                                   _ptr(kv_scales), i32(window), i32(n_splits), _stream(stream)))


def decode_attn_splits(seq_len):
    return int(lib.jllm_b200_decode_attn_splits(i32(seq_len)))


def get_splitk_partials(n_heads, n_splits, head_dim):
    return lib.jllm_b200_get_splitk_partials(i32(n_heads), i32(n_splits), i32(head_dim))


# ── extension entry points ──────────────────────────────────────────────
def gemv_quant_int_dots(y, dots, W, ggml_type, x, M, K, stream=None):
    check(lib.jllm_b200_gemv_quant_int_dots(_ptr(y), _ptr(dots), _ptr(W), i32(ggml_type), _ptr(x), i32(M), i32(K), _stream(stream)))


def gemm_quant_batched_int_dots(y, dots, W, ggml_type, x, M, N, K, stream=None):
    check(lib.jllm_b200_gemm_quant_batched_int_dots(_ptr(y), _ptr(dots), _ptr(W), i32(ggml_type), _ptr(x), i32(M), i32(N), i32(K),
                                                    _stream(stream)))


def gemm_quant_batched_pair(y0, W0, t0, M0, y1, W1, t1, M1, x, N, K, stream=None):
    check(lib.jllm_b200_gemm_quant_batched_pair(_ptr(y0), _ptr(W0), i32(t0), i32(M0), _ptr(y1), _ptr(W1), i32(t1), i32(M1), _ptr(x), i32(N), i32(K),
                                                _stream(stream)))


def norm_gemv_quant_pair(y0, W0, t0, M0, y1, W1, t1, M1, x, norm_weight, weight_fp32, eps, K, stream=None):
    check(lib.jllm_b200_norm_gemv_quant_pair(_ptr(y0), _ptr(W0), i32(t0), i32(M0), _ptr(y1), _ptr(W1), i32(t1), i32(M1), _ptr(x),
                                             _ptr(norm_weight), i32(1 if weight_fp32 else 0), f32(eps), i32(K), _stream(stream)))


def norm_gemv_quant_triple(y0, W0, t0, M0, y1, W1, t1, M1, y2, W2, t2, M2, x, norm_weight, weight_fp32, eps, K, stream=None):
    check(lib.jllm_b200_norm_gemv_quant_triple(_ptr(y0), _ptr(W0), i32(t0), i32(M0), _ptr(y1), _ptr(W1), i32(t1), i32(M1), _ptr(y2),
                                               _ptr(W2), i32(t2), i32(M2), _ptr(x), _ptr(norm_weight), i32(1 if weight_fp32 else 0),
                                               f32(eps), i32(K), _stream(stream)))


def norm_gemv_pair_swiglu(out, Wgate, Wup, ggml_type, M, x, norm_weight, weight_fp32, eps, K, stream=None):
    check(lib.jllm_b200_norm_gemv_pair_swiglu(_ptr(out), _ptr(Wgate), _ptr(Wup), i32(ggml_type), i32(M), _ptr(x), _ptr(norm_weight),
                                              i32(1 if weight_fp32 else 0), f32(eps), i32(K), _stream(stream)))


def qkv_prep_int8(q, k, v, q_norm, k_norm, eps, k_cache, v_cache, k_scales, v_scales, n_heads, n_kv_heads, head_dim, position, d_pos,
                  theta_base, neox, stream=None):
    check(lib.jllm_b200_qkv_prep_int8(_ptr(q), _ptr(k), _ptr(v), _ptr(q_norm), _ptr(k_norm), f32(eps), _ptr(k_cache), _ptr(v_cache),
                                      _ptr(k_scales), _ptr(v_scales), i32(n_heads), i32(n_kv_heads), i32(head_dim), i32(position),
                                      _ptr(d_pos), f32(theta_base), i32(1 if neox else 0), _stream(stream)))


def flash_attention_decode_batched(output, q, k_list, v_list, ks_list, vs_list, seq_lens, batch, max_seq_len, n_heads, n_kv_heads,
                                   head_dim, scale, kv_int8, stream=None):
    check(lib.jllm_b200_flash_attention_decode_batched(_ptr(output), _ptr(q), _ptr(k_list), _ptr(v_list), _ptr(ks_list), _ptr(vs_list),
                                                       _ptr(seq_lens), i32(batch), i32(max_seq_len), i32(n_heads), i32(n_kv_heads),
                                                       i32(head_dim), f32(scale), i32(1 if kv_int8 else 0), _stream(stream)))


def flash_attention_decode_noalloc(output, q, k_cache, v_cache, n_heads, n_kv_heads, head_dim, cache_head_dim, seq_len, scale, kv_int8,
                                   k_scales, v_scales, window, stream=None):
    """flash_attention_decode for hosts that must not let the library allocate: the split-K partials sit in a fixed
    array inside the library (1 MiB per GPU).  Raises JllmError (code 6) when heads x slices x (head_dim + 2) floats
    do not fit; calls that overlap on one GPU must be ordered by the caller."""
    check(lib.jllm_b200_flash_attention_decode_noalloc(_ptr(output), _ptr(q), _ptr(k_cache), _ptr(v_cache), i32(n_heads), i32(n_kv_heads),
                                                       i32(head_dim), i32(cache_head_dim), i32(seq_len), f32(scale),
                                                       i32(1 if kv_int8 else 0), _ptr(k_scales), _ptr(v_scales), i32(window),
                                                       _stream(stream)))


class AttnPlan:
    """Ragged batched decode attention over a fixed set of INT8 caches (jllm_b200_attn_plan_*): the tensor maps of the
    caches are built once; `k_list` ... `vs_list` are sequences of torch CUDA tensors (one per sequence), every cache
    holding max_seq_len positions of n_kv_heads x 128 int8 values."""

    def __init__(self, k_list, v_list, ks_list, vs_list, max_seq_len, n_kv_heads, head_dim=128):
        import ctypes as C
        from . import JllmError, last_error
        self._keep = (list(k_list), list(v_list), list(ks_list), list(vs_list))
        B = len(self._keep[0])
        arr = lambda ts: (C.c_void_p * B)(*[t.data_ptr() for t in ts])
        lib.jllm_b200_attn_plan_create.restype = C.c_void_p
        self._h = lib.jllm_b200_attn_plan_create(arr(k_list), arr(v_list), arr(ks_list), arr(vs_list), i32(B), i32(max_seq_len),
                                                 i32(n_kv_heads), i32(head_dim))
        if not self._h:
            raise JllmError(-1, last_error())
        self.batch = B

    def decode(self, output, q, seq_lens, n_heads, scale, stream=None):
        import ctypes as C
        check(lib.jllm_b200_flash_attention_decode_planned(C.c_void_p(self._h), _ptr(output), _ptr(q), _ptr(seq_lens), i32(n_heads),
                                                           f32(scale), _stream(stream)))

    def close(self):
        import ctypes as C
        if self._h:
            lib.jllm_b200_attn_plan_destroy(C.c_void_p(self._h))
            self._h = None
