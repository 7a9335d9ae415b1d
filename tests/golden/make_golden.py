"""Regenerates the golden fixtures in this folder from the reference's OWN host code.

Run in a container that has the reference tree (default /root/reference):

    make -C oracle ref && python tests/golden/make_golden.py

The reference's test translation units and its GEMV source are compiled unmodified by
oracle/Makefile into oracle/_ref/*.so (see the ref_shim_*.cu files); this script calls
their seeded generators and host references and stores inputs and outputs as .npz so
the checks can run where the reference tree is absent.

  q4k_int8.npz : tests/test_mmq_q4k_int8.cu  fill_random_q4k(0xC0FFEE), fill_random_half(0xFEEDBEEF,-1,1),
                 host_reference, host_int8_reference at M=128 N=16 K=512
  q6k_int8.npz : tests/test_mmq_q6k_int8.cu  fill_q6k(0xABCDEF), fill_half(0x12345), host_ref, host_int8_ref
  gemv_cpu.npz : src/kernels/gemv_q4.cu gemv_quant_cpu on Q4_K/Q5_K/Q6_K matrices drawn by
                 oracle.gen_weight (PCG64 seed 7) at M=40 K=1024
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

REFDIR = os.path.join(ROOT, "oracle", "_ref")
OUT = os.path.dirname(os.path.abspath(__file__))
P = lambda a: a.ctypes.data_as(C.c_void_p)


def main():
    M, N, K = 128, 16, 512
    nb = K // 256
    l4 = C.CDLL(os.path.join(REFDIR, "libref_q4k_int8.so"))
    W = np.zeros(M * nb * 144, np.uint8)
    X = np.zeros(N * K, np.uint16)
    Yf = np.zeros(N * M, np.uint16)
    Yi = np.zeros(N * M, np.uint16)
    l4.ref_q4k_fill(P(W), C.c_int(M * nb), C.c_uint32(0xC0FFEE))
    l4.ref_half_fill(P(X), C.c_int(N * K), C.c_uint32(0xFEEDBEEF), C.c_float(-1.0), C.c_float(1.0))
    l4.ref_q4k_models(P(W), P(X), P(Yf), P(Yi), C.c_int(M), C.c_int(N), C.c_int(K))
    np.savez_compressed(os.path.join(OUT, "q4k_int8.npz"), W=W, X=X, Y_float=Yf, Y_int8=Yi, shape=np.array([M, N, K]))

    l6 = C.CDLL(os.path.join(REFDIR, "libref_q6k_int8.so"))
    W = np.zeros(M * nb * 210, np.uint8)
    l6.ref_q6k_fill(P(W), C.c_int(M * nb), C.c_uint32(0xABCDEF))
    l6.ref_q6k_half_fill(P(X), C.c_int(N * K), C.c_uint32(0x12345))
    l6.ref_q6k_models(P(W), P(X), P(Yf), P(Yi), C.c_int(M), C.c_int(N), C.c_int(K))
    np.savez_compressed(os.path.join(OUT, "q6k_int8.npz"), W=W, X=X, Y_float=Yf, Y_int8=Yi, shape=np.array([M, N, K]))

    lg = C.CDLL(os.path.join(REFDIR, "libjllm_ref.so"))
    lg.ref_gemv_quant_cpu.restype = C.c_int
    rng = np.random.Generator(np.random.PCG64(7))
    Mg, Kg = 40, 1024
    d = {}
    for t in (12, 13, 14):
        Wt = orc.gen_weight(rng, t, Mg, Kg)
        x = orc.gen_act(rng, Kg)
        y = np.zeros(Mg, np.float32)
        assert lg.ref_gemv_quant_cpu(P(y), P(Wt), C.c_int(t), P(x.view(np.uint16)), C.c_int(Mg), C.c_int(Kg)) == 1
        d[f"W{t}"], d[f"x{t}"], d[f"y{t}"] = Wt, x.view(np.uint16), y
    np.savez_compressed(os.path.join(OUT, "gemv_cpu.npz"), shape=np.array([Mg, Kg]), **d)
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    main()
