"""GPU parity of the K-quant GEMV family against the CPU oracle, through the C ABI.

Bars: integer accumulators bit-exact; fp outputs within 1e-3 relative plus a floor of 2e-3 of the
output RMS (summation order differs from the reference's lane-strided order, and fp16 outputs carry
half an fp16 ULP); q8_1 paths compare against the oracle's q8_1 model, fp16-x paths (gemv_quant_add,
Q6_K logits, Q5_K) against its float model."""
import numpy as np
import pytest

from oracle import oracle as orc
from gpu_util import pkg, dev, close

pytestmark = pytest.mark.gpu

SHAPES = [(12, 1, 256), (12, 3, 512), (12, 129, 1024), (12, 257, 2560), (12, 64, 4096), (12, 33, 9728),
          (14, 1, 256), (14, 5, 512), (14, 127, 1024), (14, 130, 2560), (14, 40, 9728)]


def _run_gemv(t, M, K, seed):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(seed))
    W = orc.gen_weight(rng, t, M, K)
    x = orc.gen_act(rng, K)
    y = torch.full((M + 8,), 7.0, dtype=torch.float16, device="cuda")          # canary tail
    jb.gemv_quant(y, dev(W), t, dev(x), M, K)
    got = y.float().cpu().numpy()
    assert np.all(got[M:] == 7.0), "wrote past the output"
    return W, x, got[:M]


@pytest.mark.parametrize("t,M,K", SHAPES)
def test_gemv_quant_matches_oracle(t, M, K):
    W, x, got = _run_gemv(t, M, K, 100 + M + K + t)
    want = orc.entry_gemv_quant(W, t, x, M, K).astype(np.float32)
    ok, md = close(got, want)
    assert ok, f"max diff {md}"
    assert pkg().device_status() == 0


@pytest.mark.parametrize("t,M,K", [(12, 37, 768), (12, 200, 2560), (14, 37, 768), (14, 64, 9728)])
def test_integer_accumulators_bit_exact(t, M, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(7 + M))
    W = orc.gen_weight(rng, t, M, K)
    x = orc.gen_act(rng, K)
    G = K // 32 if t == 12 else K // 16
    dots = torch.zeros((M, G), dtype=torch.int32, device="cuda")
    y = torch.zeros(M, dtype=torch.float16, device="cuda")
    jb.gemv_quant_int_dots(y, dots, dev(W), t, dev(x), M, K)
    qs, _, _ = orc.quantize_q8_1(x)
    want = orc.q8_int_dots(W, t, M, K, qs)
    assert np.array_equal(dots.cpu().numpy(), want)


@pytest.mark.parametrize("t,M,K", [(12, 2560, 4096), (14, 2560, 9728), (13, 50, 1024), (12, 5, 256),
                                    # the row shards of Wo and W_down at 4 and 8 tensor-parallel ranks
                                    (12, 640, 4096), (14, 640, 9728), (12, 320, 4096), (14, 320, 9728)])
def test_gemv_quant_add(t, M, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(11 + M))
    W = orc.gen_weight(rng, t, M, K)
    x = orc.gen_act(rng, K)
    res = orc.gen_act(rng, M)
    y = torch.zeros(M, dtype=torch.float16, device="cuda")
    jb.gemv_quant_add(y, dev(W), t, dev(x), dev(res), M, K)
    want = orc.entry_gemv_quant_add(W, t, x, res, M, K).astype(np.float32)
    ok, md = close(y.float().cpu().numpy(), want)
    assert ok, f"max diff {md}"


@pytest.mark.parametrize("t,M,K", [(12, 300, 2560), (14, 1000, 2560), (13, 20, 512)])
def test_gemv_quant_f32(t, M, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(13 + M))
    W = orc.gen_weight(rng, t, M, K)
    x = orc.gen_act(rng, K)
    y = torch.zeros(M, dtype=torch.float32, device="cuda")
    jb.gemv_quant_f32(y, dev(W), t, dev(x), M, K)
    want = orc.entry_gemv_quant_f32(W, t, x, M, K)
    ok, md = close(y.cpu().numpy(), want, floor=1e-3 * float(np.sqrt(np.mean(want.astype(np.float64) ** 2))))
    assert ok, f"max diff {md}"


@pytest.mark.parametrize("types,Ms,K", [((12, 12), (9728, 9728), 2560), ((12, 14), (70, 33), 1024), ((12, 12), (5, 3), 256),
                                        ((12, 12), (2432, 2432), 2560), ((12, 12), (1216, 1216), 2560)])      # gate/up shards at 4 / 8 ranks
def test_gemv_quant_pair(types, Ms, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(17 + Ms[0]))
    Ws = [orc.gen_weight(rng, t, m, K) for t, m in zip(types, Ms)]
    x = orc.gen_act(rng, K)
    ys = [torch.zeros(m, dtype=torch.float16, device="cuda") for m in Ms]
    jb.gemv_quant_pair(ys[0], dev(Ws[0]), types[0], Ms[0], ys[1], dev(Ws[1]), types[1], Ms[1], dev(x), K)
    wants = orc.entry_gemv_multi(Ws, list(types), list(Ms), x, K)
    for y, w in zip(ys, wants):
        ok, md = close(y.float().cpu().numpy(), w.astype(np.float32))
        assert ok, f"max diff {md}"


@pytest.mark.parametrize("types,Ms,K", [((12, 12, 14), (4096, 1024, 1024), 2560), ((12, 12, 12), (40, 9, 9), 512),
                                        ((14, 14, 14), (33, 17, 5), 768), ((14, 12, 12), (20, 20, 20), 1024),
                                        ((12, 14, 12), (31, 16, 8), 512)])
def test_gemv_quant_triple(types, Ms, K):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(19 + Ms[0]))
    Ws = [orc.gen_weight(rng, t, m, K) for t, m in zip(types, Ms)]
    x = orc.gen_act(rng, K)
    ys = [torch.zeros(m, dtype=torch.float16, device="cuda") for m in Ms]
    jb.gemv_quant_triple(ys[0], dev(Ws[0]), types[0], Ms[0], ys[1], dev(Ws[1]), types[1], Ms[1], ys[2], dev(Ws[2]), types[2], Ms[2],
                         dev(x), K)
    wants = orc.entry_gemv_multi(Ws, list(types), list(Ms), x, K)
    for y, w in zip(ys, wants):
        ok, md = close(y.float().cpu().numpy(), w.astype(np.float32))
        assert ok, f"max diff {md}"


def test_fused_norm_variants_equal_unfused_sequence():
    """norm_gemv_* == fused_rmsnorm_residual followed by the plain entry point, bit for bit."""
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(23))
    K, Ms, types = 2560, (512, 128, 128), (12, 12, 14)
    Ws = [dev(orc.gen_weight(rng, t, m, K)) for t, m in zip(types, Ms)]
    x = dev(orc.gen_act(rng, K))
    w = dev((1 + 0.02 * rng.standard_normal(K)).astype(np.float32))
    normed = torch.zeros(K, dtype=torch.float16, device="cuda")
    jb.fused_rmsnorm_residual(normed, x, None, w, 1, K, 1e-6, True)
    a = [torch.zeros(m, dtype=torch.float16, device="cuda") for m in Ms]
    b = [torch.zeros(m, dtype=torch.float16, device="cuda") for m in Ms]
    jb.gemv_quant_triple(a[0], Ws[0], types[0], Ms[0], a[1], Ws[1], types[1], Ms[1], a[2], Ws[2], types[2], Ms[2], normed, K)
    jb.norm_gemv_quant_triple(b[0], Ws[0], types[0], Ms[0], b[1], Ws[1], types[1], Ms[1], b[2], Ws[2], types[2], Ms[2], x, w, True, 1e-6, K)
    for p, q in zip(a, b):
        assert torch.equal(p, q)
    # gate/up + SwiGLU epilogue == pair then fused_swiglu
    M = 1000
    Wg, Wu = dev(orc.gen_weight(rng, 12, M, K)), dev(orc.gen_weight(rng, 12, M, K))
    g = torch.zeros(M, dtype=torch.float16, device="cuda"); u = torch.zeros_like(g); s1 = torch.zeros_like(g); s2 = torch.zeros_like(g)
    jb.gemv_quant_pair(g, Wg, 12, M, u, Wu, 12, M, normed, K)
    jb.fused_swiglu(s1, g, u, 1, M)
    jb.norm_gemv_pair_swiglu(s2, Wg, Wu, 12, M, x, w, True, 1e-6, K)
    assert torch.equal(s1, s2)


def test_errors_are_reported_not_hidden():
    import torch
    jb = pkg()
    y = torch.ones(8, dtype=torch.float16, device="cuda")
    W = torch.zeros(8 * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(256, dtype=torch.float16, device="cuda")
    with pytest.raises(jb.JllmError) as e:                      # unsupported type: error + zero fill (gemv_q4.cu:2668)
        jb.gemv_quant(y, W, 2, x, 8, 256)
    assert e.value.code == 2
    torch.cuda.synchronize()
    assert float(y.abs().sum()) == 0.0
    with pytest.raises(jb.JllmError) as e:                      # K not a multiple of 256
        jb.gemv_quant(y, W, 12, x, 8, 200)
    assert e.value.code == 1
    host = np.zeros(8 * 144, np.uint8)
    with pytest.raises(jb.JllmError) as e:                      # host weight pointer with no registered mapping
        jb.gemv_quant(y, host.ctypes.data, 12, x, 8, 256)
    assert e.value.code == 3
    jb.gemv_quant(y, W, 12, x, 0, 256)                          # M == 0 is a no-op
