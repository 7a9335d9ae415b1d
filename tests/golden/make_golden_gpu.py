"""Records what the reference's OWN GPU kernels return on the seeded benchmark inputs (tests/golden/gpu_cases.py).

Needs a CUDA device and oracle/_ref/libjllm_ref.so (the reference's kernel sources compiled unmodified for sm_100a by
`make -C oracle ref`, with the C wrappers of oracle/ref_shim_gpu.cu).  Run from the repository root:

    python tests/golden/make_golden_gpu.py [--out DIR] [--time]

Writes ref_gpu.npz (outputs + input digests; inputs are regenerated from their seeds by the tests) into DIR (default:
this folder) and, with --time, ref_gpu_timings.json: mean microseconds per call of the reference's kernels on this GPU,
large operands rotated over enough device copies to exceed the L2 cache.
"""
import argparse
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import gpu_cases as gc  # noqa: E402

P = lambda a: None if a is None else np.ascontiguousarray(a).ctypes.data_as(C.c_void_p)
U16 = lambda a: np.ascontiguousarray(a).view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    lib = C.CDLL(os.path.join(gc.ROOT, "oracle", "_ref", "libjllm_ref.so"))
    rec, times = {}, {}
    fp = C.c_float()
    tp = C.byref(fp) if args.time else None

    def ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: reference call returned {rc}")
        if args.time:
            times[what] = round(fp.value, 3)

    def copies(nbytes):          # enough copies to cover three times a 126 MB L2
        return int(max(1, min(64, (3 * 126e6) // nbytes + 1)))

    def q8_blocks(name, x):
        blocks = np.zeros(x.size // 32 * 36, np.uint8)
        rc = lib.refgpu_quantize_q8_1(P(blocks), P(U16(x)), C.c_int(x.size))
        if rc != 0:
            raise RuntimeError(f"{name}: reference quantiser returned {rc}")
        rec[name + "_q8"] = blocks

    def gemv(name, c, mode, res=None):
        W = np.ascontiguousarray(c["W"])
        y = np.zeros(c["M"], np.float32 if mode == 2 else np.uint16)
        ok(lib.refgpu_gemv(P(y), P(W), C.c_longlong(W.nbytes), C.c_int(c["t"]), P(U16(c["x"])), P(None if res is None else U16(res)),
                           C.c_int(c["M"]), C.c_int(c["K"]), C.c_int(mode), C.c_int(args.iters), C.c_int(copies(W.nbytes)), tp), name)
        rec[name + "_y"] = y
        rec[name + "_in"] = gc.digest(W, c["x"]) if res is None else gc.digest(W, c["x"], res)

    def save():
        os.makedirs(args.out, exist_ok=True)
        np.savez_compressed(os.path.join(args.out, "ref_gpu.npz"), **rec)
        print("wrote", os.path.join(args.out, "ref_gpu.npz"), "with", len(rec), "arrays")
        if args.time:
            with open(os.path.join(args.out, "ref_gpu_timings.json"), "w") as f:
                json.dump({"unit": "us per call", "iters": args.iters, "times": times}, f, indent=1)
            print(json.dumps(times))

    try:
        record(lib, args, rec, times, gemv, ok, copies, tp, q8_blocks)
    finally:
        save()            # a failing call still leaves the records made before it


def record(lib, args, rec, times, gemv, ok, copies, tp, q8_blocks):
    # the dp4a GEMVs quantise their activation vector to q8_1 blocks first: keep the blocks the reference's own
    # quantiser makes of each of those vectors next to the results
    c = gc.gemv_q4k(); gemv("gemv_q4k", c, 0); q8_blocks("gemv_q4k", c["x"])
    c = gc.gemv_q6k(); gemv("gemv_q6k", c, 0); q8_blocks("gemv_q6k", c["x"])
    W = np.ascontiguousarray(c["W"]); y8 = np.zeros((8, c["M"]), np.uint16)
    ok(lib.refgpu_gemm_batched(P(y8), P(W), C.c_longlong(W.nbytes), C.c_int(14), P(U16(c["X8"])), C.c_int(c["M"]), C.c_int(8),
                               C.c_int(c["K"]), C.c_int(args.iters), tp), "gemm_q6k_b8")
    rec["gemm_q6k_b8_y"] = y8; rec["gemm_q6k_b8_in"] = gc.digest(W, c["X8"])
    gemv("gemv_add_wo", (c := gc.gemv_add_wo()), 1, c["res"])
    gemv("gemv_add_down", (c := gc.gemv_add_down()), 1, c["res"])
    gemv("gemv_f32", gc.gemv_f32(), 2)

    for name, c in (("gemv_pair", gc.gemv_pair()), ("gemv_triple", gc.gemv_triple())):
        n = len(c["Ms"])
        Ws = [np.ascontiguousarray(c[f"W{i}"]) for i in range(n)]
        ys = [np.zeros(m, np.uint16) for m in c["Ms"]]
        ok(lib.refgpu_gemv_multi(C.c_int(n), (C.c_void_p * n)(*[y.ctypes.data for y in ys]), (C.c_void_p * n)(*[w.ctypes.data for w in Ws]),
                                 (C.c_longlong * n)(*[w.nbytes for w in Ws]), (C.c_int * n)(*c["ts"]), (C.c_int * n)(*c["Ms"]),
                                 P(U16(c["x"])), C.c_int(c["K"]), C.c_int(args.iters), C.c_int(copies(sum(w.nbytes for w in Ws))), tp), name)
        for i, y in enumerate(ys):
            rec[f"{name}_y{i}"] = y
        rec[name + "_in"] = gc.digest(*Ws, c["x"])
        q8_blocks(name, c["x"])

    c = gc.q8_1()
    blocks = np.zeros(c["x"].size // 32 * 36, np.uint8)
    ok(lib.refgpu_quantize_q8_1(P(blocks), P(U16(c["x"])), C.c_int(c["x"].size)), "q8_1")
    times.pop("q8_1", None)
    rec["q8_1_blocks"] = blocks; rec["q8_1_in"] = gc.digest(c["x"])

    for L in gc.ATTN_LENGTHS:
        c = gc.attention(L)
        out = np.zeros(gc.NH * gc.HD, np.uint16)
        nbytes = 2 * c["k"].nbytes
        ok(lib.refgpu_attention_decode(P(out), P(U16(c["q"])), P(c["k"]), P(c["v"]), P(c["ks"]), P(c["vs"]), C.c_int(gc.NH), C.c_int(gc.NKV),
                                       C.c_int(gc.HD), C.c_int(L), C.c_float(gc.SCALE), C.c_int(args.iters), C.c_int(copies(nbytes)), tp),
           f"attn_L{L}")
        rec[f"attn_L{L}_out"] = out; rec[f"attn_L{L}_in"] = gc.digest(c["q"], c["k"], c["v"], c["ks"], c["vs"])

    for N in (33, 512):
        c = gc.attention_prefill(N)
        out = np.zeros(N * gc.NH * gc.HD, np.uint16)
        ok(lib.refgpu_attention_prefill(P(out), P(U16(c["q"])), P(c["k"]), P(c["v"]), P(c["ks"]), P(c["vs"]), C.c_int(gc.NH), C.c_int(gc.NKV),
                                        C.c_int(gc.HD), C.c_int(N), C.c_int(0), C.c_float(gc.SCALE), C.c_int(max(1, args.iters // 10)), tp),
           f"prefill_attn_N{N}")
        sel = gc.prefill_sample(N)
        rec[f"prefill_attn_N{N}_out"] = out.reshape(N, -1)[sel].copy(); rec[f"prefill_attn_N{N}_sel"] = sel
        rec[f"prefill_attn_N{N}_in"] = gc.digest(c["q"], c["k"], c["v"], c["ks"], c["vs"])

    for t, Ns in ((12, gc.GEMM_TOKENS), (14, (2048,))):
        for N in Ns:
            c = gc.gemm(t, N)
            W = np.ascontiguousarray(c["W"]); y = np.zeros((N, c["M"]), np.uint16)
            name = f"gemm_t{t}_N{N}"
            ok(lib.refgpu_gemm_batched(P(y), P(W), C.c_longlong(W.nbytes), C.c_int(t), P(U16(c["X"])), C.c_int(c["M"]), C.c_int(N),
                                       C.c_int(c["K"]), C.c_int(max(1, args.iters // 10)), tp), name)
            rec[name + "_y"] = y[c["sel"]].copy(); rec[name + "_sel"] = c["sel"]; rec[name + "_in"] = gc.digest(W, c["X"])

    e = gc.elementwise()
    o = np.zeros(gc.H, np.uint16)
    ok(lib.refgpu_rmsnorm(P(o), P(U16(e["x"])), P(U16(e["res"])), P(e["w"]), C.c_int(1), C.c_int(gc.H), C.c_float(1e-6)), "rmsnorm"); rec["rmsnorm_res"] = o.copy()
    ok(lib.refgpu_rmsnorm(P(o), P(U16(e["x"])), None, P(e["w"]), C.c_int(1), C.c_int(gc.H), C.c_float(1e-6)), "rmsnorm"); rec["rmsnorm_plain"] = o.copy()
    oh = np.zeros(gc.NH * gc.HD, np.uint16)
    ok(lib.refgpu_rmsnorm(P(oh), P(U16(e["qh"])), None, P(e["wh"]), C.c_int(gc.NH), C.c_int(gc.HD), C.c_float(1e-6)), "rmsnorm"); rec["rmsnorm_heads"] = oh
    for pos in e["positions"]:
        q = U16(e["qh"]).copy(); k = U16(e["kh"]).copy()
        ok(lib.refgpu_rope(P(q), P(k), C.c_int(gc.NH), C.c_int(gc.NKV), C.c_int(gc.HD), C.c_int(int(pos)), C.c_float(1e6), C.c_int(1)), "rope")
        rec[f"rope_q_{pos}"] = q; rec[f"rope_k_{pos}"] = k
    dst = np.zeros(gc.NKV * gc.HD, np.int8); sc = np.zeros(gc.NKV, np.float32)
    ok(lib.refgpu_fp16_to_int8(P(dst), P(sc), P(U16(e["kh"])), C.c_int(gc.NKV), C.c_int(gc.HD)), "fp16_to_int8")
    rec["kvq_codes"] = dst; rec["kvq_scales"] = sc
    og = np.zeros(gc.FF, np.uint16)
    ok(lib.refgpu_swiglu(P(og), P(U16(e["g"])), P(U16(e["u"])), C.c_int(1), C.c_int(gc.FF)), "swiglu"); rec["swiglu"] = og
    row = np.zeros(gc.H, np.uint16); Wemb = np.ascontiguousarray(e["Wemb"])
    ok(lib.refgpu_embedding_row(P(row), P(Wemb), C.c_longlong(Wemb.nbytes), C.c_int(12), C.c_int(37), C.c_int(gc.H)), "embedding"); rec["embedding_row37"] = row
    rec["elementwise_in"] = gc.digest(e["x"], e["res"], e["w"], e["qh"], e["kh"], e["wh"], e["g"], e["u"], Wemb)
    for k in ("rmsnorm", "rope", "fp16_to_int8", "swiglu", "embedding"):
        times.pop(k, None)



if __name__ == "__main__":
    main()
