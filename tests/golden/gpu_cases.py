"""Seeded inputs of the benchmark configurations, shared by make_golden_gpu.py (which records what the reference's
own GPU kernels return for them) and by the parity tests (which regenerate the same inputs and compare the CPU
oracle and the B200 kernels with those records).

Each case draws from numpy.random.Generator(PCG64(seed)), seed = 1000 + configuration index (+ a per-case offset),
with the value distributions the benchmark configurations state.  ref_gpu.npz stores, per case, a SHA-256 prefix of
the input bytes, so a drift of the generators is noticed before any number is compared.
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

H, QD, KVD, FF = 2560, 4096, 1024, 9728
NH, NKV, HD = 32, 8, 128
SCALE = float(1.0 / np.sqrt(HD))
ATTN_LENGTHS = (1024, 4096, 8192, 32768)
GEMM_TOKENS = (512, 2048, 8192)
SAMPLE_ROWS = 8          # token rows of a batched product kept in the record


def rng_for(config, sub=0):
    return np.random.Generator(np.random.PCG64(1000 + config + 100 * sub))


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).view(np.uint8).tobytes())
    return np.frombuffer(h.digest()[:8], np.uint8).copy()


# configuration 0: Q4_K 9728 x 2560 GEMV
def gemv_q4k():
    r = rng_for(0)
    return dict(W=orc.gen_q4k(r, FF, H), x=orc.gen_act(r, H), t=12, M=FF, K=H)


# configuration 1: Q6_K 2560 x 9728 GEMV, batch 1 and batch 8
def gemv_q6k():
    r = rng_for(1)
    W = orc.gen_q6k(r, H, FF)
    x = orc.gen_act(r, FF)
    X8 = orc.gen_act(r, 8 * FF).reshape(8, FF)
    return dict(W=W, x=x, X8=X8, t=14, M=H, K=FF)


# the decoder's other GEMV shapes (shared-activation pair / triple, residual add, fp32 logits slice)
def gemv_pair():
    r = rng_for(0, 1)
    return dict(W0=orc.gen_q4k(r, FF, H), W1=orc.gen_q4k(r, FF, H), x=orc.gen_act(r, H), K=H, Ms=(FF, FF), ts=(12, 12))


def gemv_triple():
    r = rng_for(0, 2)
    return dict(W0=orc.gen_q4k(r, QD, H), W1=orc.gen_q4k(r, KVD, H), W2=orc.gen_q6k(r, KVD, H), x=orc.gen_act(r, H), K=H,
                Ms=(QD, KVD, KVD), ts=(12, 12, 14))


def gemv_add_wo():
    r = rng_for(0, 3)
    return dict(W=orc.gen_q4k(r, H, QD), x=orc.gen_act(r, QD), res=orc.gen_act(r, H), t=12, M=H, K=QD)


def gemv_add_down():
    r = rng_for(1, 3)
    return dict(W=orc.gen_q6k(r, H, FF), x=orc.gen_act(r, FF), res=orc.gen_act(r, H), t=14, M=H, K=FF)


def gemv_f32():
    r = rng_for(1, 4)
    M = 4096          # a slice of the 151936-row output matrix
    return dict(W=orc.gen_q6k(r, M, H), x=orc.gen_act(r, H), t=14, M=M, K=H)


def q8_1():
    r = rng_for(0, 5)
    return dict(x=orc.gen_act(r, FF))


# configuration 2: INT8-KV decode attention
def attention(L):
    r = rng_for(2, L % 97)
    q = orc.gen_act(r, NH * HD)
    k, ks = orc.gen_kv(r, L, NKV, HD)
    v, vs = orc.gen_kv(r, L, NKV, HD)
    return dict(q=q, k=k, v=v, ks=ks, vs=vs, L=L)


def ragged_lengths(batch=64, lo=256, hi=8192):
    return rng_for(2, 7).integers(lo, hi + 1, batch).astype(np.int32)


def attention_prefill(N, start=0):
    r = rng_for(2, 50 + N % 89)
    L = start + N
    q = orc.gen_act(r, N * NH * HD)
    k, ks = orc.gen_kv(r, L, NKV, HD)
    v, vs = orc.gen_kv(r, L, NKV, HD)
    return dict(q=q, k=k, v=v, ks=ks, vs=vs, N=N, start=start)


def prefill_sample(N):
    """Query tokens of a prefill-attention record that are kept (all of them for a short prompt)."""
    if N <= 40:
        return np.arange(N, dtype=np.int32)
    return np.unique(np.concatenate([np.array([0, 1, 31, 32, 63, 64, N // 2, N - 2, N - 1]), rng_for(2, 60).choice(N, 8, replace=False)])).astype(np.int32)


# configuration 3: batched K-quant GEMM (prefill)
def gemm(t, N):
    if t == 12:
        r = rng_for(3, 1)
        W = orc.gen_q4k(r, FF, H); M, K = FF, H
    else:
        r = rng_for(3, 2)
        W = orc.gen_q6k(r, H, FF); M, K = H, FF
    rx = rng_for(3, 10 + N % 83)
    X = rx.standard_normal((N, K), dtype=np.float32).astype(np.float16)
    sel = np.sort(rx.choice(N, min(SAMPLE_ROWS, N), replace=False)).astype(np.int32)
    return dict(W=W, X=X, sel=sel, t=t, M=M, N=N, K=K)


# element-wise kernels at the decoder's shapes
def elementwise():
    r = rng_for(4, 1)
    d = dict(x=orc.gen_act(r, H), res=orc.gen_act(r, H), w=(1.0 + 0.02 * r.standard_normal(H)).astype(np.float32),
             qh=orc.gen_act(r, NH * HD), kh=orc.gen_act(r, NKV * HD), wh=(1.0 + 0.02 * r.standard_normal(HD)).astype(np.float32),
             g=orc.gen_act(r, FF), u=orc.gen_act(r, FF), Wemb=orc.gen_q4k(r, 64, H))
    d["positions"] = np.array([0, 1, 33, 1000, 32767], np.int32)
    return d
