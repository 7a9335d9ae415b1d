"""ctypes front end of the CPU oracle (oracle.c) plus the seeded input generators.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py.  The shipped package never imports this module.

Generators draw with numpy.random.Generator(PCG64(seed)) and pack GGUF K-quant
super-blocks exactly as the reference lays them out
(src/kernels/gemv_q4.cu:141-164 structs, :185-195 scale packing, :378-393 Q6_K).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

Q4_K, Q5_K, Q6_K = 12, 13, 14
BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}


def build(force: bool = False) -> str:
    """Compile oracle.c into liboracle.so (gcc, OpenMP) if it is missing or stale."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_h2f.restype = C.c_float
        _LIB.orc_h2f.argtypes = [C.c_uint16]
        _LIB.orc_f2h.restype = C.c_uint16
        _LIB.orc_f2h.argtypes = [C.c_float]
        _LIB.orc_decode_step.restype = C.c_int
        _LIB.orc_prefill.restype = C.c_int
        _LIB.orc_dequant_embedding_row.restype = C.c_int
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def _h(a):
    """fp16 array -> contiguous uint16 bit view."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return a.view(np.uint16)
    assert a.dtype == np.uint16
    return a


# ── block packers ──────────────────────────────────────────────────────────
def pack_q4k(d, dmin, sc, mn, q):
    """d,dmin: [B] fp16; sc,mn: [B,8] ints 0..63; q: [B,256] ints 0..15 -> [B,144] uint8."""
    B = d.shape[0]
    out = np.zeros((B, 144), np.uint8)
    out[:, 0:2] = np.asarray(d, np.float16).reshape(B, 1).view(np.uint8)
    out[:, 2:4] = np.asarray(dmin, np.float16).reshape(B, 1).view(np.uint8)
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    s = np.zeros((B, 12), np.uint8)
    s[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = mn[:, 0:4] | ((mn[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 0xF) | ((mn[:, 4:8] & 0xF) << 4)
    out[:, 4:16] = s
    q = q.astype(np.uint8).reshape(B, 4, 2, 32)          # [il][lo/hi][l]
    out[:, 16:144] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(B, 128)
    return out


def pack_q6k(d, sc, q):
    """d: [B] fp16; sc: [B,16] int8; q: [B,256] ints 0..63 -> [B,210] uint8."""
    B = d.shape[0]
    out = np.zeros((B, 210), np.uint8)
    q = q.astype(np.uint8).reshape(B, 2, 4, 32)          # [n][quarter][l]
    lo = q & 0xF
    hi = q >> 4
    ql = np.zeros((B, 2, 64), np.uint8)
    ql[:, :, 0:32] = lo[:, :, 0, :] | (lo[:, :, 2, :] << 4)
    ql[:, :, 32:64] = lo[:, :, 1, :] | (lo[:, :, 3, :] << 4)
    qh = hi[:, :, 0, :] | (hi[:, :, 1, :] << 2) | (hi[:, :, 2, :] << 4) | (hi[:, :, 3, :] << 6)
    out[:, 0:128] = ql.reshape(B, 128)
    out[:, 128:192] = qh.reshape(B, 64)
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    out[:, 208:210] = np.asarray(d, np.float16).reshape(B, 1).view(np.uint8)
    return out


def gen_q4k(rng, rows, K, sigma=0.01, min_ratio=1.0):
    """Q4_K matrix with the benchmark's value distributions: d=|N(0,1)|*sigma, dmin=|N(0,1)|*sigma*min_ratio (fp16;
    sigma = 0.01 and min_ratio = 1 in the kernel-level configurations), scales/mins U{0..63}, quants U{0..15}.
    Returns [rows, K/256*144] uint8."""
    B = rows * (K // 256)
    d = (np.abs(rng.standard_normal(B)) * sigma).astype(np.float16)
    dm = (np.abs(rng.standard_normal(B)) * sigma * min_ratio).astype(np.float16)
    sc = rng.integers(0, 64, (B, 8))
    mn = rng.integers(0, 64, (B, 8))
    q = rng.integers(0, 16, (B, 256), dtype=np.uint8)
    return pack_q4k(d, dm, sc, mn, q).reshape(rows, -1)


def gen_q6k(rng, rows, K, sigma=0.01):
    """Q6_K matrix: d=|N(0,1)|*sigma (fp16), int8 scales U{-64..63}, quants U{0..63}."""
    B = rows * (K // 256)
    d = (np.abs(rng.standard_normal(B)) * sigma).astype(np.float16)
    sc = rng.integers(-64, 64, (B, 16))
    q = rng.integers(0, 64, (B, 256), dtype=np.uint8)
    return pack_q6k(d, sc, q).reshape(rows, -1)


def gen_q5k(rng, rows, K):
    """Q5_K matrix with random bytes in scales/qh/qs and small fp16 d/dmin."""
    B = rows * (K // 256)
    out = rng.integers(0, 256, (B, 176), dtype=np.uint8)
    out[:, 0:2] = (np.abs(rng.standard_normal(B)) * 0.01).astype(np.float16).reshape(B, 1).view(np.uint8)
    out[:, 2:4] = (np.abs(rng.standard_normal(B)) * 0.01).astype(np.float16).reshape(B, 1).view(np.uint8)
    return out.reshape(rows, -1)


def gen_weight(rng, ggml_type, rows, K):
    return {Q4_K: gen_q4k, Q5_K: gen_q5k, Q6_K: gen_q6k}[ggml_type](rng, rows, K)


def gen_act(rng, n):
    """fp32 N(0,1) rounded to fp16 (the API takes half activations)."""
    return rng.standard_normal(n).astype(np.float32).astype(np.float16)


def gen_kv(rng, L, n_kv=8, hd=128):
    """INT8 K or V [L, n_kv, hd] U{-127..127} and fp32 scales holding fp16(|N|*0.02) [L, n_kv]."""
    kv = rng.integers(-127, 128, (L, n_kv, hd), dtype=np.int8)
    sc = (np.abs(rng.standard_normal((L, n_kv))) * 0.02).astype(np.float16).astype(np.float32)
    return kv, sc


# ── thin wrappers over oracle.c ────────────────────────────────────────────
def gemv_float(W, t, x, M, K):
    y = np.empty(M, np.float32)
    lib().orc_gemv_float(_p(_u8(W)), C.c_int(t), _p(_h(x)), C.c_int(M), C.c_int(K), _p(y))
    return y


def gemv_q8(W, t, x, M, K):
    y = np.empty(M, np.float32)
    lib().orc_gemv_q8(_p(_u8(W)), C.c_int(t), _p(_h(x)), C.c_int(M), C.c_int(K), _p(y))
    return y


def quantize_q8_1(x):
    K = x.size
    qs = np.empty(K, np.int8)
    d = np.empty(K // 32, np.uint16)
    s = np.empty(K // 32, np.uint16)
    lib().orc_quantize_q8_1(_p(_h(x)), C.c_int(K), _p(qs), _p(d), _p(s))
    return qs, d.view(np.float16), s.view(np.float16)


class q8_override:
    """Context manager: while active, the oracle's q8_1 quantiser returns the given blocks (the 36-byte blocks
    {fp16 d, fp16 s, int8 qs[32]} a run of the reference's GPU quantiser produced) for vectors of that length."""

    def __init__(self, blocks36):
        b = np.ascontiguousarray(blocks36, np.uint8).reshape(-1, 36)
        self.d = np.ascontiguousarray(b[:, 0:2]).view(np.uint16).reshape(-1).copy()
        self.s = np.ascontiguousarray(b[:, 2:4]).view(np.uint16).reshape(-1).copy()
        self.qs = np.ascontiguousarray(b[:, 4:36]).view(np.int8).reshape(-1).copy()

    def __enter__(self):
        lib().orc_set_q8_override(_p(self.qs), _p(self.d), _p(self.s), C.c_int(self.qs.size))
        return self

    def __exit__(self, *a):
        lib().orc_set_q8_override(None, None, None, C.c_int(0))


def q8_int_dots(W, t, M, K, qs):
    G = K // 32 if t == Q4_K else K // 16
    out = np.empty((M, G), np.int32)
    lib().orc_q8_int_dots(_p(_u8(W)), C.c_int(t), C.c_int(M), C.c_int(K), _p(np.ascontiguousarray(qs)), _p(out))
    return out


def entry_gemv_quant(W, t, x, M, K):
    y = np.empty(M, np.uint16)
    lib().orc_entry_gemv_quant(_p(_u8(W)), C.c_int(t), _p(_h(x)), C.c_int(M), C.c_int(K), _p(y))
    return y.view(np.float16)


def entry_gemv_quant_f32(W, t, x, M, K):
    y = np.empty(M, np.float32)
    lib().orc_entry_gemv_quant_f32(_p(_u8(W)), C.c_int(t), _p(_h(x)), C.c_int(M), C.c_int(K), _p(y))
    return y


def entry_gemv_quant_add(W, t, x, res, M, K):
    y = np.empty(M, np.uint16)
    lib().orc_entry_gemv_quant_add(_p(_u8(W)), C.c_int(t), _p(_h(x)), _p(_h(res)), C.c_int(M), C.c_int(K), _p(y))
    return y.view(np.float16)


def entry_gemv_multi(Ws, ts, Ms, x, K):
    n = len(Ws)
    Wb = [_u8(w) for w in Ws]
    ys = [np.empty(m, np.uint16) for m in Ms]
    Wp = (C.c_void_p * n)(*[w.ctypes.data for w in Wb])
    Yp = (C.c_void_p * n)(*[y.ctypes.data for y in ys])
    Tp = (C.c_int * n)(*ts)
    Mp = (C.c_int * n)(*Ms)
    lib().orc_entry_gemv_multi(C.c_int(n), Wp, Tp, Mp, _p(_h(x)), C.c_int(K), Yp)
    return [y.view(np.float16) for y in ys]


def testmodel_float(W, t, X, M, N, K):
    Y = np.empty((N, M), np.uint16)
    lib().orc_testmodel_float(_p(_u8(W)), C.c_int(t), _p(_h(X)), C.c_int(M), C.c_int(N), C.c_int(K), _p(Y))
    return Y.view(np.float16)


def testmodel_int8(W, t, X, M, N, K):
    Y = np.empty((N, M), np.uint16)
    lib().orc_testmodel_int8(_p(_u8(W)), C.c_int(t), _p(_h(X)), C.c_int(M), C.c_int(N), C.c_int(K), _p(Y))
    return Y.view(np.float16)


def mmq(W, t, X, M, N, K):
    Y = np.empty((N, M), np.uint16)
    lib().orc_mmq(_p(_u8(W)), C.c_int(t), _p(_h(X)), C.c_int(M), C.c_int(N), C.c_int(K), _p(Y))
    return Y.view(np.float16)


def mmq_int_dots(W, t, X, M, N, K):
    G = K // 32 if t == Q4_K else K // 16
    out = np.empty((N, M, G), np.int32)
    lib().orc_mmq_int_dots(_p(_u8(W)), C.c_int(t), _p(_h(X)), C.c_int(M), C.c_int(N), C.c_int(K), _p(out))
    return out


def mmq_quantize(x, ds4):
    K = x.size
    q = np.empty(K, np.int8)
    d = np.empty(K // 32, np.float32)
    s = np.empty(K // 32, np.float32)
    lib().orc_mmq_quantize(_p(_h(x)), C.c_int(K), _p(q), _p(d), _p(s), C.c_int(1 if ds4 else 0))
    return q, d, s


def entry_gemm_quant_batched(W, t, X, M, N, K):
    Y = np.empty((N, M), np.uint16)
    lib().orc_entry_gemm_quant_batched(_p(_u8(W)), C.c_int(t), _p(_h(X)), C.c_int(M), C.c_int(N), C.c_int(K), _p(Y))
    return Y.view(np.float16)


def dequant_embedding_row(W, t, token, hidden):
    out = np.empty(hidden, np.uint16)
    ok = lib().orc_dequant_embedding_row(_p(_u8(W)), C.c_int(t), C.c_int(token), C.c_int(hidden), _p(out))
    return out.view(np.float16) if ok else None


def dequant_row(row_bytes, t, n_blocks):
    out = np.empty(n_blocks * 256, np.float32)
    lib().orc_dequant_row(_p(_u8(row_bytes)), C.c_int(t), C.c_int(n_blocks), _p(out))
    return out


def rmsnorm(x, res, w, rows, dim, eps):
    out = np.empty(rows * dim, np.uint16)
    w = np.ascontiguousarray(w)
    fp32 = 1 if w.dtype == np.float32 else 0
    lib().orc_rmsnorm(_p(_h(x)), _p(None if res is None else _h(res)), _p(w if fp32 else _h(w)), C.c_int(fp32),
                      C.c_int(rows), C.c_int(dim), C.c_float(eps), _p(out))
    return out.view(np.float16)


def rope(q, k, n_heads, n_kv, hd, pos, theta, neox=True):
    q = _h(q).copy()
    k = None if k is None else _h(k).copy()
    lib().orc_rope(_p(q), _p(k), C.c_int(n_heads), C.c_int(n_kv if k is not None else 0), C.c_int(hd), C.c_int(pos),
                   C.c_float(theta), C.c_int(1 if neox else 0))
    return q.view(np.float16), (None if k is None else k.view(np.float16))


def swiglu(g, u):
    out = np.empty(g.size, np.uint16)
    lib().orc_swiglu(_p(_h(g)), _p(_h(u)), C.c_int(g.size), _p(out))
    return out.view(np.float16)


def geglu(g, u):
    out = np.empty(g.size, np.uint16)
    lib().orc_geglu(_p(_h(g)), _p(_h(u)), C.c_int(g.size), _p(out))
    return out.view(np.float16)


def fp16_to_int8(src, rows, cols):
    dst = np.empty(rows * cols, np.int8)
    sc = np.empty(rows, np.float32)
    lib().orc_fp16_to_int8(_p(_h(src)), C.c_int(rows), C.c_int(cols), _p(dst), _p(sc))
    return dst.reshape(rows, cols), sc


def softmax(x):
    x = np.ascontiguousarray(x, np.float32).copy()
    lib().orc_softmax(_p(x), C.c_int(x.size))
    return x


def attention_decode(q, k, v, n_heads, n_kv, hd, seq, scale, kv_int8=True, ks=None, vs=None, window=0, chd=None):
    out = np.empty(n_heads * hd, np.uint16)
    chd = hd if chd is None else chd
    k = np.ascontiguousarray(k)
    v = np.ascontiguousarray(v)
    lib().orc_attention_decode(_p(_h(q)), _p(k), _p(v), C.c_int(n_heads), C.c_int(n_kv), C.c_int(hd), C.c_int(chd),
                               C.c_int(seq), C.c_float(scale), C.c_int(1 if kv_int8 else 0),
                               _p(None if ks is None else np.ascontiguousarray(ks, np.float32)),
                               _p(None if vs is None else np.ascontiguousarray(vs, np.float32)),
                               C.c_int(window), _p(out))
    return out.view(np.float16).reshape(n_heads, hd)


def attention_prefill(q, k, v, n_heads, n_kv, hd, N, start, scale, kv_int8=True, ks=None, vs=None, window=0):
    out = np.empty(N * n_heads * hd, np.uint16)
    lib().orc_attention_prefill(_p(_h(q)), _p(np.ascontiguousarray(k)), _p(np.ascontiguousarray(v)), C.c_int(n_heads),
                                C.c_int(n_kv), C.c_int(hd), C.c_int(hd), C.c_int(N), C.c_int(start), C.c_float(scale),
                                C.c_int(1 if kv_int8 else 0),
                                _p(None if ks is None else np.ascontiguousarray(ks, np.float32)),
                                _p(None if vs is None else np.ascontiguousarray(vs, np.float32)),
                                C.c_int(window), _p(out))
    return out.view(np.float16).reshape(N, n_heads, hd)


# ── whole decoder ──────────────────────────────────────────────────────────
class _Cfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "max_ctx")] + \
               [("rope_theta", C.c_float), ("eps", C.c_float)]


class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")] + \
               [(n, C.c_int) for n in ("t_wq", "t_wk", "t_wv", "t_wo", "t_gate", "t_up", "t_down")] + \
               [(n, C.c_void_p) for n in ("rms_attn", "rms_ffn", "q_norm", "k_norm")]


class _Model(C.Structure):
    _fields_ = [("cfg", _Cfg), ("layers", C.POINTER(_Layer)), ("tok_embd", C.c_void_p), ("t_embd", C.c_int),
                ("output", C.c_void_p), ("t_out", C.c_int), ("out_norm", C.c_void_p),
                ("kv", C.c_void_p), ("kv_scales", C.c_void_p)]


# Whole-model weights.  The kernel-level generator (sigma 0.01, dmin ~ d) gives weights of RMS ~3 with a mean of
# +1.6: a stacked decoder overflows fp16 inside its first layer (every logit NaN), and even rescaled its common-mode
# gain makes the network amplify one fp16 ULP into percent-level logit changes.  Model weights therefore use
# dmin = 7.5 d, which centres d*sc*q - dmin*m on zero (E[q] = 7.5, E[sc] = E[m]), and a sigma that gives W.x unit RMS:
# Q4_K  E[w^2] = sigma^2 (E[sc^2]E[q^2] + 7.5^2 E[m^2] - 2*7.5 E|N|^2 E[sc]E[m]E[q]) ~ (327 sigma)^2,
# Q6_K  E[w^2] = sigma^2 * 1365 * 341.5 ~ (683 sigma)^2.
_W_RMS = {Q4_K: 327.0, Q6_K: 683.0}
MODEL_MIN_RATIO = 7.5


def model_sigma(ggml_type, K):
    """sigma that makes W.x of a unit-RMS x come out with RMS ~1."""
    return 1.0 / (_W_RMS[ggml_type] * np.sqrt(K))


def gen_model(seed, n_layers=36, hidden=2560, n_heads=32, n_kv=8, hd=128, ffn=9728, vocab=151936):
    """Random-init Qwen3-shaped weights in the benchmark's quant mix: Q4_K everywhere except
    Q6_K for attn_v, ffn_down and output; F32 norm weights 1+0.02*N(0,1).  Blocks come from the
    kernel-level generators with d (and dmin) scaled by model_sigma() so activations stay O(1).
    Returns a dict of numpy arrays (uint8 block images / float32 norms)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    qd, kvd = n_heads * hd, n_kv * hd
    gen_q4k_u = lambda r, rows, K: gen_q4k(r, rows, K, model_sigma(Q4_K, K), MODEL_MIN_RATIO)
    gen_q6k_u = lambda r, rows, K: gen_q6k(r, rows, K, model_sigma(Q6_K, K))
    m = dict(cfg=dict(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, ffn=ffn,
                      vocab=vocab, rope_theta=1e6, eps=1e-6), layers=[])
    nrm = lambda n: (1.0 + 0.02 * rng.standard_normal(n)).astype(np.float32)
    for _ in range(n_layers):
        m["layers"].append(dict(
            wq=(gen_q4k_u(rng, qd, hidden), Q4_K), wk=(gen_q4k_u(rng, kvd, hidden), Q4_K), wv=(gen_q6k_u(rng, kvd, hidden), Q6_K),
            wo=(gen_q4k_u(rng, hidden, qd), Q4_K), gate=(gen_q4k_u(rng, ffn, hidden), Q4_K), up=(gen_q4k_u(rng, ffn, hidden), Q4_K),
            down=(gen_q6k_u(rng, hidden, ffn), Q6_K),
            rms_attn=nrm(hidden), rms_ffn=nrm(hidden), q_norm=nrm(hd), k_norm=nrm(hd)))
    m["tok_embd"] = (gen_q4k_u(rng, vocab, hidden), Q4_K)
    m["output"] = (gen_q6k_u(rng, vocab, hidden), Q6_K)
    m["out_norm"] = nrm(hidden)
    return m


class Decoder:
    """CPU decoder over a gen_model() dict; greedy decode through orc_decode_step."""

    def __init__(self, model, max_ctx):
        c = model["cfg"]
        self.model, self.max_ctx = model, max_ctx
        L = c["n_layers"]
        self._layers = (_Layer * L)()
        for i, lw in enumerate(model["layers"]):
            for n in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
                setattr(self._layers[i], n, lw[n][0].ctypes.data)
                setattr(self._layers[i], "t_" + n, lw[n][1])
            for n in ("rms_attn", "rms_ffn", "q_norm", "k_norm"):
                setattr(self._layers[i], n, lw[n].ctypes.data)
        self.kv = np.zeros(2 * L * max_ctx * c["n_kv_heads"] * c["head_dim"], np.int8)
        self.kvs = np.zeros(2 * L * max_ctx * c["n_kv_heads"], np.float32)
        self._m = _Model()
        for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab"):
            setattr(self._m.cfg, k, c[k])
        self._m.cfg.max_ctx = max_ctx
        self._m.cfg.rope_theta, self._m.cfg.eps = c["rope_theta"], c["eps"]
        self._m.layers = self._layers
        self._m.tok_embd, self._m.t_embd = model["tok_embd"][0].ctypes.data, model["tok_embd"][1]
        self._m.output, self._m.t_out = model["output"][0].ctypes.data, model["output"][1]
        self._m.out_norm = model["out_norm"].ctypes.data
        self._m.kv, self._m.kv_scales = self.kv.ctypes.data, self.kvs.ctypes.data
        self.logits = np.empty(c["vocab"], np.float32)

    def step(self, token, pos):
        return int(lib().orc_decode_step(C.byref(self._m), C.c_int(int(token)), C.c_int(pos), _p(self.logits)))

    def prefill(self, prompt, start=0):
        """Batched prompt prefill (the reference's transformer_prefill order and prefill arithmetic); returns the greedy
        token after the last prompt token and leaves its logits in self.logits."""
        p = np.ascontiguousarray(prompt, np.int32)
        return int(lib().orc_prefill(C.byref(self._m), _p(p), C.c_int(p.size), C.c_int(start), _p(self.logits)))

    def generate_prefilled(self, prompt, n_new):
        """Batched prefill of the prompt, then n_new greedy tokens by decode steps."""
        tok, out = self.prefill(prompt), []
        pos = len(prompt)
        for i in range(n_new):
            out.append(tok)
            if i + 1 < n_new:
                tok = self.step(tok, pos)
                pos += 1
        return out

    def generate(self, prompt, n_new):
        """Feed the prompt one token per step, then decode n_new tokens greedily."""
        tok, out = None, []
        for pos, t in enumerate(prompt):
            tok = self.step(t, pos)
        pos = len(prompt)
        for i in range(n_new):
            out.append(tok)
            if i + 1 < n_new:
                tok = self.step(tok, pos)
                pos += 1
        return out
