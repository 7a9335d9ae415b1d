"""Tensor-parallel decode: host side.  One process per GPU (torch.distributed supplies rank, world size and the
exchange of the CUDA IPC handles); the data path itself is the library's own push-style gather over NVLink
(csrc/tp.cu), not a torch collective.

Sharding (the reference is single-GPU; this follows its data layout): rank r of g owns output rows
[r*M/g, (r+1)*M/g) of wq, wk, wv, wo, w_gate, w_up, w_down and output.  Rows of a GGUF K-quant matrix are
contiguous byte ranges, so a slice is a view.  wq/wk/wv rows are head-major, hence a rank owns n_heads/g query heads
and the n_kv_heads/g KV heads they attend to (with GQA the query heads of a rank map onto its own KV heads).  The
embedding table and all norm vectors are replicated.  The contraction dimension is never split: 38 super-blocks
per ffn_down row do not divide by 4 or 8.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

BLOCK_BYTES = {12: 144, 13: 176, 14: 210}
SHARDED = ("wq", "wk", "wv", "wo", "gate", "up", "down")


def check_divisible(cfg, world):
    """Raises ValueError unless every sharded dimension splits evenly (and the slices stay 16-byte granular)."""
    hd = cfg["head_dim"]
    for name, n in (("n_heads", cfg["n_heads"]), ("n_kv_heads", cfg["n_kv_heads"]), ("ffn", cfg["ffn"]), ("hidden", cfg["hidden"]),
                    ("vocab", cfg["vocab"])):
        if n % world:
            raise ValueError(f"{name}={n} does not split over {world} ranks")
    for name, n in (("q slice", cfg["n_heads"] // world * hd), ("hidden slice", cfg["hidden"] // world), ("ffn slice", cfg["ffn"] // world)):
        if (n * 2) % 16:
            raise ValueError(f"{name} of {n} fp16 values is not a multiple of 16 bytes")


def row_ranges(cfg, world, rank):
    """Row range [r0, r1) of every sharded matrix for `rank`."""
    check_divisible(cfg, world)
    qd, kvd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    rows = dict(wq=qd, wk=kvd, wv=kvd, wo=cfg["hidden"], gate=cfg["ffn"], up=cfg["ffn"], down=cfg["hidden"], output=cfg["vocab"])
    return {k: (rank * n // world, (rank + 1) * n // world) for k, n in rows.items()}


def row_bytes(ggml_type, K):
    return (K // 256) * BLOCK_BYTES[ggml_type]


def slice_rows(image, ggml_type, K, r0, r1):
    """Rows [r0, r1) of a flat uint8 block image (numpy array or torch tensor): a view, no copy."""
    rb = row_bytes(ggml_type, K)
    return image.reshape(-1)[r0 * rb:r1 * rb]


def shard_model(model, world, rank):
    """gen_model()-style dict (numpy or torch leaves) -> the same structure holding this rank's slices."""
    cfg = model["cfg"] if "cfg" in model else None
    if cfg is None:
        raise ValueError("model dict needs its cfg")
    rr = row_ranges(cfg, world, rank)
    H, qd, F = cfg["hidden"], cfg["n_heads"] * cfg["head_dim"], cfg["ffn"]
    kdim = dict(wq=H, wk=H, wv=H, wo=qd, gate=H, up=H, down=F)
    out = dict(cfg=cfg, layers=[], tok_embd=model["tok_embd"], out_norm=model["out_norm"],
               output=(slice_rows(model["output"][0], model["output"][1], H, *rr["output"]), model["output"][1]))
    for lw in model["layers"]:
        d = {k: v for k, v in lw.items() if k not in SHARDED}
        for k in SHARDED:
            img, t = lw[k]
            d[k] = (slice_rows(img, t, kdim[k], *rr[k]), t)
        out["layers"].append(d)
    return out


class TPDecoder:
    """Decoder session of one rank.  `local` is shard_model(...) uploaded to this rank's GPU (torch CUDA tensors);
    `group` is a torch.distributed process group (any backend: it only carries the 64-byte IPC handles)."""

    def __init__(self, cfg, local, max_context, rank, world, group=None, flags=3):
        import torch
        import torch.distributed as dist
        from . import lib, JllmError, last_error
        from .decoder import LayerDesc, ModelDesc
        check_divisible(cfg, world)
        self._lib, self.cfg, self.rank, self.world = lib, cfg, rank, world
        lib.jllm_b200_tp_alloc.restype = C.c_void_p
        lib.jllm_b200_tp_open.restype = C.c_void_p
        lib.jllm_b200_tp_region_bytes.restype = C.c_size_t
        lib.jllm_b200_decoder_create_tp.restype = C.c_void_p
        nbytes = lib.jllm_b200_tp_region_bytes(cfg["hidden"], cfg["n_heads"] * cfg["head_dim"], cfg["ffn"])
        self._region = lib.jllm_b200_tp_alloc(C.c_size_t(nbytes))
        if not self._region:
            raise JllmError(-1, last_error())
        handle = (C.c_ubyte * 64)()
        rc = lib.jllm_b200_tp_export(C.c_void_p(self._region), handle)
        if rc:
            raise JllmError(rc, last_error())
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._mapped = []
        regions = (C.c_void_p * world)()
        for r in range(world):
            if r == rank:
                regions[r] = self._region
            else:
                buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                p = lib.jllm_b200_tp_open(buf)
                if not p:
                    raise JllmError(-1, last_error())
                self._mapped.append(p)
                regions[r] = p
        self._keep = local
        L = cfg["n_layers"]
        self._layers = (LayerDesc * L)()
        names = dict(wq="wq", wk="wk", wv="wv", wo="wo", w_gate="gate", w_up="up", w_down="down")
        for i, lw in enumerate(local["layers"]):
            for f, k in names.items():
                setattr(self._layers[i], f, lw[k][0].data_ptr())
                setattr(self._layers[i], "type_" + f, lw[k][1])
            for k in ("rms_attn", "rms_ffn", "q_norm", "k_norm"):
                setattr(self._layers[i], k, lw[k].data_ptr() if lw.get(k) is not None else None)
        m = ModelDesc()
        m.n_layers, m.hidden_dim, m.n_heads, m.n_kv_heads = L, cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"]
        m.head_dim, m.intermediate_dim, m.vocab_size, m.max_context = cfg["head_dim"], cfg["ffn"], cfg["vocab"], max_context
        m.rope_theta, m.rms_eps, m.rope_neox = cfg["rope_theta"], cfg["eps"], 1
        m.tok_embd, m.embd_type = local["tok_embd"][0].data_ptr(), local["tok_embd"][1]
        m.output, m.output_type = local["output"][0].data_ptr(), local["output"][1]
        m.output_norm = local["out_norm"].data_ptr()
        m.layers = self._layers
        # every rank must have mapped every region before anyone pushes into it
        dist.barrier(group=group)
        self._h = lib.jllm_b200_decoder_create_tp(C.byref(m), C.c_int(flags), C.c_int(rank), C.c_int(world), regions)
        if not self._h:
            raise JllmError(-1, last_error())
        self._group = group
        dist.barrier(group=group)

    def close(self):
        import torch
        import torch.distributed as dist
        if self._h:
            torch.cuda.synchronize()
            dist.barrier(group=self._group)          # no rank unmaps while a peer may still push
            self._lib.jllm_b200_decoder_destroy(C.c_void_p(self._h))
            self._h = None
            for p in self._mapped:
                self._lib.jllm_b200_tp_close(C.c_void_p(p))
            dist.barrier(group=self._group)
            self._lib.jllm_b200_tp_free(C.c_void_p(self._region))

    def generate(self, prompt, n_new, stream=None):
        from . import _stream, check
        p = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(max(n_new, 1), np.int32)
        check(self._lib.jllm_b200_decoder_generate(C.c_void_p(self._h), p.ctypes.data_as(C.c_void_p), C.c_int(p.size), C.c_int(n_new),
                                                   out.ctypes.data_as(C.c_void_p), _stream(stream)))
        return out[:n_new]

    def step_sync(self, host_pos_token, host_next, stream=None):
        from . import _stream, check
        check(self._lib.jllm_b200_decoder_step_sync(C.c_void_p(self._h), C.c_void_p(host_pos_token.data_ptr()),
                                                    C.c_void_p(host_next.data_ptr()), _stream(stream)))

    def step_device(self, stream):
        from . import _stream, check
        check(self._lib.jllm_b200_decoder_step_device(C.c_void_p(self._h), _stream(stream)))

    def kernels_per_step(self):
        return int(self._lib.jllm_b200_decoder_kernels_per_step(C.c_void_p(self._h)))

    def reset(self):
        from . import check
        check(self._lib.jllm_b200_decoder_reset(C.c_void_p(self._h)))

    def recorded_tokens(self, first=0, n=0, stream=None):
        from . import _stream
        out = np.zeros(max(n, 1), np.int32)
        cnt = int(self._lib.jllm_b200_decoder_recorded_tokens(C.c_void_p(self._h), C.c_int(first), C.c_int(n), out.ctypes.data_as(C.c_void_p),
                                                              _stream(stream)))
        return cnt, out[:max(0, min(n, cnt - first))]
