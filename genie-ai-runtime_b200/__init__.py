"""genie-ai-runtime_b200 — host-side mirror of the reference kernel API over the B200 library.

The compute lives in ``libjllm_b200.so`` (hand-written CUDA for sm_100a, built by ``build.py``)
and is reached through its C ABI (``include/jllm_b200.h``).  This package only marshals
pointers: every function takes torch CUDA tensors (or raw device pointers), passes their
addresses and the current stream, and raises :class:`JllmError` on a non-zero status.  There
is no CPU path and no fallback: if the shared library is missing the import fails.

Function names, argument order and meaning follow the reference's ``include/jllm_kernels.h``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libjllm_b200.so")

Q4_K, Q5_K, Q6_K = 12, 13, 14


class JllmError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"jllm_b200 status {code}: {text}")
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python genie-ai-runtime_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    lib.jllm_b200_last_error.restype = C.c_char_p
    lib.jllm_b200_launch_count.restype = C.c_longlong
    lib.jllm_b200_get_splitk_partials.restype = C.c_void_p
    lib.jllm_b200_resolve_mapped_weight_device_ptr.restype = C.c_void_p
    for n in ("kv_pool_create", "kv_pool_key_ptr", "kv_pool_val_ptr", "kv_pool_scale_ptr", "scratch_create", "scratch_get"):
        getattr(lib, "jllm_b200_" + n).restype = C.c_void_p
    for n in ("kv_pool_scales_bytes", "kv_pool_capacity_bytes", "kv_pool_used_bytes", "kv_pool_packed_used_bytes",
              "scratch_mark", "scratch_used", "scratch_capacity"):
        getattr(lib, "jllm_b200_" + n).restype = C.c_int64
    return lib


lib = _load()


def _ptr(t):
    """Device address of a torch tensor, an int address, or None."""
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):
        return C.c_void_p(t)
    return C.c_void_p(t.data_ptr())


def _stream(stream=None):
    if stream is not None:
        return C.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc):
    if rc != 0:
        raise JllmError(rc, lib.jllm_b200_last_error().decode())


def last_error():
    return lib.jllm_b200_last_error().decode()


def launch_count():
    return int(lib.jllm_b200_launch_count())


def device_status(stream=None):
    return int(lib.jllm_b200_device_status(_stream(stream)))


from .kernels import *  # noqa: E402,F401,F403
from .pools import KVCachePool, ScratchPool  # noqa: E402,F401
from . import decoder  # noqa: E402,F401
