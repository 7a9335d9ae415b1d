"""GPU parity of the batched K-quant GEMM (prefill) against the oracle and the reference's own
golden vectors (tests/golden/q4k_int8.npz, q6k_int8.npz)."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from gpu_util import pkg, dev, close, close_gemm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,M,N,K", [(12, 128, 16, 512), (12, 130, 7, 1024), (12, 64, 65, 2560), (14, 128, 16, 512), (14, 33, 9, 2560),
                                      (14, 20, 3, 9728), (13, 16, 3, 512),
                                      # several output tiles per persistent CTA, ragged last row / token tile, every token-tile width
                                      (12, 300, 300, 2560), (14, 260, 270, 1024), (12, 1, 2, 256), (14, 129, 33, 256), (12, 257, 129, 768),
                                      (12, 40000, 40, 256), (14, 19000, 70, 512),
                                      # more output tiles than SMs: whole rounds, then the leftover tiles cut into K ranges (ragged edges)
                                      (12, 2500, 2000, 2048), (14, 2500, 1999, 1024)])
def test_gemm_quant_batched_matches_oracle(t, M, N, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1003 + M + N))
    W = orc.gen_weight(rng, t, M, K)
    X = orc.gen_act(rng, N * K)
    y = torch.zeros(N * M, dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched(y, dev(W), t, dev(X), M, N, K)
    want = orc.entry_gemm_quant_batched(W, t, X, M, N, K).astype(np.float32).reshape(-1)
    ok, md = close_gemm(y.float().cpu().numpy(), want, N, M)
    assert ok, md


@pytest.mark.parametrize("t,M,N,K", [(12, 40, 5, 768), (14, 24, 6, 512)])
def test_gemm_integer_accumulators_bit_exact(t, M, N, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1004 + M))
    W = orc.gen_weight(rng, t, M, K)
    X = orc.gen_act(rng, N * K)
    G = K // 32 if t == 12 else K // 16
    dots = torch.zeros((N, M, G), dtype=torch.int32, device="cuda")
    y = torch.zeros(N * M, dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched_int_dots(y, dots, dev(W), t, dev(X), M, N, K)
    assert np.array_equal(dots.cpu().numpy(), orc.mmq_int_dots(W, t, X, M, N, K))


@pytest.mark.parametrize("name,t", [("q4k_int8.npz", 12), ("q6k_int8.npz", 14)])
def test_reference_golden_vectors(golden_dir, name, t):
    """The reference's own acceptance bar for its int8 GEMM: every |Δ| <= 0.5 against its int8 host model
    (tests/test_mmq_q4k_int8.cu:533-541, tests/test_mmq_q6k_int8.cu:298-310)."""
    import torch
    jb = pkg()
    g = np.load(os.path.join(golden_dir, name))
    M, N, K = map(int, g["shape"])
    y = torch.zeros(N * M, dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched(y, dev(g["W"]), t, dev(g["X"].view(np.float16)), M, N, K)
    ref = g["Y_int8"].view(np.float16).astype(np.float32)
    assert np.max(np.abs(y.float().cpu().numpy() - ref)) <= 0.5


@pytest.mark.parametrize("t,M,N,K", [(12, 9728, 48, 2560), (14, 2560, 48, 9728), (12, 9728, 64, 2560), (14, 2560, 64, 9728), (12, 4096, 64, 2560),
                                      (12, 4096, 8, 2560), (14, 1024, 24, 2560), (12, 2560, 2, 4096), (14, 151, 57, 768)])
def test_few_tokens_stream_the_weights_once(t, M, N, K):
    """2..64 tokens go through the weight-streaming kernel (csrc/mmq_stream.cu): the decoder's own shapes at 48 and 64 streams
    (the two largest matrices at 64 streams are handed to the tensor-core kernel, which is faster there), every token-tile
    count, ragged row and token edges, and K ranges split over CTAs (few rows, long K)."""
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1007 + M + N))
    W = orc.gen_weight(rng, t, M, K)
    X = orc.gen_act(rng, N * K)
    y = torch.full((N * M,), float("nan"), dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched(y, dev(W), t, dev(X), M, N, K)
    want = orc.entry_gemm_quant_batched(W, t, X, M, N, K).astype(np.float32).reshape(-1)
    ok, md = close_gemm(y.float().cpu().numpy(), want, N, M)
    assert ok, md
    assert jb.device_status() == 0


@pytest.mark.parametrize("t,M0,M1,N,K", [(12, 300, 200, 100, 1024), (14, 130, 257, 70, 512), (12, 2500, 2300, 1000, 1024), (12, 9728, 9728, 64, 2560),
                                          (12, 96, 64, 8, 512)])
def test_two_products_over_the_same_activations(t, M0, M1, N, K):
    """gemm_quant_batched_pair (the gate and up projections of a batched layer): both outputs against the oracle.  The shapes
    cover the shared launch of the tensor-core kernel with ragged row tiles of both matrices, more tiles than SMs (whole
    rounds plus split tail tiles that belong to either matrix), the decoder's own pair at 64 streams, and the few-token
    path (two launches)."""
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1010 + M0 + N))
    W0 = orc.gen_weight(rng, t, M0, K); W1 = orc.gen_weight(rng, t, M1, K)
    X = orc.gen_act(rng, N * K)
    y0 = torch.full((N * M0,), float("nan"), dtype=torch.float16, device="cuda")
    y1 = torch.full((N * M1,), float("nan"), dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched_pair(y0, dev(W0), t, M0, y1, dev(W1), t, M1, dev(X), N, K)
    for y, W, M in ((y0, W0, M0), (y1, W1, M1)):
        want = orc.entry_gemm_quant_batched(W, t, X, M, N, K).astype(np.float32).reshape(-1)
        ok, md = close_gemm(y.float().cpu().numpy(), want, N, M)
        assert ok, md
    assert jb.device_status() == 0


@pytest.mark.parametrize("t", [12, 14])
def test_tensor_core_and_cuda_core_paths_agree(t):
    """The tcgen05 kernel and the CUDA-core kernel (the one that exports the integer accumulators) compute the same
    quantised product; they differ by the fp16 rounding of the operand products only."""
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1006 + t))
    M, N, K = 200, 48, 1536
    W = dev(orc.gen_weight(rng, t, M, K)); X = dev(orc.gen_act(rng, N * K))
    G = K // 32 if t == 12 else K // 16
    dots = torch.zeros((N, M, G), dtype=torch.int32, device="cuda")
    a = torch.zeros(N * M, dtype=torch.float16, device="cuda"); b = torch.zeros_like(a)
    jb.gemm_quant_batched(a, W, t, X, M, N, K)
    jb.gemm_quant_batched_int_dots(b, dots, W, t, X, M, N, K)
    ok, md = close_gemm(a.float().cpu().numpy(), b.float().cpu().numpy(), N, M)
    assert ok, md
    assert jb.device_status() == 0


def test_n_equal_one_routes_to_gemv():
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(1005))
    M, K = 77, 1024
    W = dev(orc.gen_weight(rng, 12, M, K)); x = dev(orc.gen_act(rng, K))
    a = torch.zeros(M, dtype=torch.float16, device="cuda"); b = torch.zeros_like(a)
    jb.gemm_quant_batched(a, W, 12, x, M, 1, K)
    jb.gemv_quant(b, W, 12, x, M, K)
    assert torch.equal(a, b)
