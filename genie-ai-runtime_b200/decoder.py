"""Decoder session over the C ABI (jllm_b200_decoder_*): the reference engine's per-token kernel
sequence (src/engine/decode.cu:1169-1246, :2101-2194) with greedy sampling on the device."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib, _stream, check, JllmError, last_error


class LayerDesc(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")] + \
               [(n, C.c_int) for n in ("type_wq", "type_wk", "type_wv", "type_wo", "type_w_gate", "type_w_up", "type_w_down")] + \
               [(n, C.c_void_p) for n in ("rms_attn", "rms_ffn", "q_norm", "k_norm")]


class ModelDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden_dim", "n_heads", "n_kv_heads", "head_dim", "intermediate_dim", "vocab_size",
                                        "max_context")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float), ("rope_neox", C.c_int),
                ("tok_embd", C.c_void_p), ("embd_type", C.c_int), ("output", C.c_void_p), ("output_type", C.c_int),
                ("output_norm", C.c_void_p), ("layers", C.POINTER(LayerDesc))]


lib.jllm_b200_decoder_create.restype = C.c_void_p
lib.jllm_b200_decoder_logits.restype = C.c_void_p

FUSED, GRAPH, PREFILL = 1, 2, 16          # PREFILL: generate() runs the prompt through the batched prefill path


class Decoder:
    """`weights` is a dict shaped like oracle.gen_model(): per-layer (uint8 block image, ggml type) pairs
    and float32 norm vectors, given as torch CUDA tensors (see `upload`)."""

    def __init__(self, cfg, weights, max_context, flags=FUSED | GRAPH):
        self._keep = weights
        L = cfg["n_layers"]
        self._layers = (LayerDesc * L)()
        names = dict(wq="wq", wk="wk", wv="wv", wo="wo", w_gate="gate", w_up="up", w_down="down")
        for i, lw in enumerate(weights["layers"]):
            for f, k in names.items():
                setattr(self._layers[i], f, lw[k][0].data_ptr())
                setattr(self._layers[i], "type_" + f, lw[k][1])
            for k in ("rms_attn", "rms_ffn", "q_norm", "k_norm"):
                setattr(self._layers[i], k, lw[k].data_ptr() if lw.get(k) is not None else None)
        m = ModelDesc()
        m.n_layers, m.hidden_dim, m.n_heads, m.n_kv_heads = L, cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"]
        m.head_dim, m.intermediate_dim, m.vocab_size, m.max_context = cfg["head_dim"], cfg["ffn"], cfg["vocab"], max_context
        m.rope_theta, m.rms_eps, m.rope_neox = cfg["rope_theta"], cfg["eps"], 1
        m.tok_embd, m.embd_type = weights["tok_embd"][0].data_ptr(), weights["tok_embd"][1]
        m.output, m.output_type = weights["output"][0].data_ptr(), weights["output"][1]
        m.output_norm = weights["out_norm"].data_ptr()
        m.layers = self._layers
        self.cfg, self.max_context = cfg, max_context
        self._h = lib.jllm_b200_decoder_create(C.byref(m), C.c_int(flags))
        if not self._h:
            raise JllmError(-1, last_error())

    def close(self):
        if self._h:
            lib.jllm_b200_decoder_destroy(C.c_void_p(self._h))
            self._h = None

    def step(self, token, position, stream=None):
        check(lib.jllm_b200_decoder_step(C.c_void_p(self._h), int(token), int(position), _stream(stream)))
        return int(lib.jllm_b200_decoder_last_token(C.c_void_p(self._h), _stream(stream)))

    def step_sync(self, host_pos_token, host_next, stream=None):
        """host_pos_token: pinned int32 tensor [position, token]; host_next: pinned int32 tensor of one element."""
        check(lib.jllm_b200_decoder_step_sync(C.c_void_p(self._h), C.c_void_p(host_pos_token.data_ptr()), C.c_void_p(host_next.data_ptr()),
                                              _stream(stream)))

    def step_device(self, stream):
        """Enqueues the next step from the position and token the previous step left on the device (no copy, no wait)."""
        check(lib.jllm_b200_decoder_step_device(C.c_void_p(self._h), _stream(stream)))

    def reset(self):
        check(lib.jllm_b200_decoder_reset(C.c_void_p(self._h)))

    def prefill(self, tokens, start_pos=0, stream=None, chunk=None):
        """Batched prompt prefill (enqueue only); afterwards last_token() / step_device() continue the stream."""
        t = np.ascontiguousarray(tokens, np.int32)
        if chunk:
            check(lib.jllm_b200_decoder_set_prefill_chunk(C.c_void_p(self._h), C.c_int(chunk)))
        check(lib.jllm_b200_decoder_prefill(C.c_void_p(self._h), t.ctypes.data_as(C.c_void_p), C.c_int(t.size), C.c_int(start_pos), _stream(stream)))

    def last_token(self, stream=None):
        return int(lib.jllm_b200_decoder_last_token(C.c_void_p(self._h), _stream(stream)))

    def logits(self):
        import torch
        ptr = lib.jllm_b200_decoder_logits(C.c_void_p(self._h))
        out = torch.empty(self.cfg["vocab"], dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        C.CDLL("libcudart.so").cudaMemcpy(C.c_void_p(out.data_ptr()), C.c_void_p(ptr), C.c_size_t(out.numel() * 4), 3)
        return out

    def generate(self, prompt, n_new, stream=None):
        """Host token ids in, host token ids out (both copies happen inside the call)."""
        p = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(max(n_new, 1), np.int32)
        check(lib.jllm_b200_decoder_generate(C.c_void_p(self._h), p.ctypes.data_as(C.c_void_p), C.c_int(p.size), C.c_int(n_new),
                                             out.ctypes.data_as(C.c_void_p), _stream(stream)))
        return out[:n_new]

    def kernels_per_step(self):
        return int(lib.jllm_b200_decoder_kernels_per_step(C.c_void_p(self._h)))

    def recorded_tokens(self, first=0, n=0, stream=None):
        """(count recorded so far, ids [first, first+n) of the device-side record of every step's greedy token)."""
        out = np.zeros(max(n, 1), np.int32)
        cnt = int(lib.jllm_b200_decoder_recorded_tokens(C.c_void_p(self._h), C.c_int(first), C.c_int(n), out.ctypes.data_as(C.c_void_p), _stream(stream)))
        return cnt, out[:max(0, min(n, cnt - first))]


class BatchDecoder:
    """n_streams requests decoded in lock step through the batched kernels (jllm_b200_batch_decoder_*)."""

    def __init__(self, cfg, weights, max_context, n_streams):
        self._keep = weights
        L = cfg["n_layers"]
        self._layers = (LayerDesc * L)()
        names = dict(wq="wq", wk="wk", wv="wv", wo="wo", w_gate="gate", w_up="up", w_down="down")
        for i, lw in enumerate(weights["layers"]):
            for f, k in names.items():
                setattr(self._layers[i], f, lw[k][0].data_ptr())
                setattr(self._layers[i], "type_" + f, lw[k][1])
            for k in ("rms_attn", "rms_ffn", "q_norm", "k_norm"):
                setattr(self._layers[i], k, lw[k].data_ptr() if lw.get(k) is not None else None)
        m = ModelDesc()
        m.n_layers, m.hidden_dim, m.n_heads, m.n_kv_heads = L, cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"]
        m.head_dim, m.intermediate_dim, m.vocab_size, m.max_context = cfg["head_dim"], cfg["ffn"], cfg["vocab"], max_context
        m.rope_theta, m.rms_eps, m.rope_neox = cfg["rope_theta"], cfg["eps"], 1
        m.tok_embd, m.embd_type = weights["tok_embd"][0].data_ptr(), weights["tok_embd"][1]
        m.output, m.output_type = weights["output"][0].data_ptr(), weights["output"][1]
        m.output_norm = weights["out_norm"].data_ptr()
        m.layers = self._layers
        self.cfg, self.n_streams = cfg, n_streams
        lib.jllm_b200_batch_decoder_create.restype = C.c_void_p
        lib.jllm_b200_batch_decoder_logits.restype = C.c_void_p
        self._h = lib.jllm_b200_batch_decoder_create(C.byref(m), C.c_int(n_streams))
        if not self._h:
            raise JllmError(-1, last_error())

    def close(self):
        if self._h:
            lib.jllm_b200_batch_decoder_destroy(C.c_void_p(self._h))
            self._h = None

    def generate(self, prompts, n_new, stream=None):
        """prompts: int array [n_streams][n_prompt]; returns [n_new][n_streams]."""
        p = np.ascontiguousarray(prompts, np.int32)
        assert p.ndim == 2 and p.shape[0] == self.n_streams
        out = np.zeros((max(n_new, 1), self.n_streams), np.int32)
        check(lib.jllm_b200_batch_decoder_generate(C.c_void_p(self._h), p.ctypes.data_as(C.c_void_p), C.c_int(p.shape[1]), C.c_int(n_new),
                                                   out.ctypes.data_as(C.c_void_p), _stream(stream)))
        return out[:n_new]

    def step_device(self, stream):
        check(lib.jllm_b200_batch_decoder_step_device(C.c_void_p(self._h), _stream(stream)))

    def logits(self):
        import torch
        ptr = lib.jllm_b200_batch_decoder_logits(C.c_void_p(self._h))
        out = torch.empty((self.n_streams, self.cfg["vocab"]), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        C.CDLL("libcudart.so").cudaMemcpy(C.c_void_p(out.data_ptr()), C.c_void_p(ptr), C.c_size_t(out.numel() * 2), 3)
        return out

    def kernels_per_step(self):
        return int(lib.jllm_b200_batch_decoder_kernels_per_step(C.c_void_p(self._h)))


def upload(model):
    """oracle.gen_model()-style numpy weights -> the same structure with torch CUDA tensors."""
    import torch
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = dict(layers=[], tok_embd=(t(model["tok_embd"][0]), model["tok_embd"][1]), output=(t(model["output"][0]), model["output"][1]),
               out_norm=t(model["out_norm"]))
    for lw in model["layers"]:
        d = {}
        for k, v in lw.items():
            d[k] = (t(v[0]), v[1]) if isinstance(v, tuple) else t(v)
        out["layers"].append(d)
    return out
