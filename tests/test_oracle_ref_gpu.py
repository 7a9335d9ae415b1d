"""Pins the CPU oracle against what the reference's OWN GPU kernels returned on a B200 for the seeded benchmark
inputs (tests/golden/ref_gpu.npz, written by tests/golden/make_golden_gpu.py from the reference's unmodified kernel
sources compiled for sm_100a).  Inputs are regenerated from their seeds and checked against the recorded digests.

The reference's dp4a decode GEMV (gemv_quant, _pair, _triple with Q4_K / Q6_K) quantises the activation vector to
q8_1 blocks first.  As nvcc 12.9 compiles that quantiser's packed 36-byte block struct for sm_100a, the blocks it
stores on a B200 carry corrupted scales — d with its low byte zero, s with a wrong low byte; the codes are right (seen
in the recorded blocks, test_q8_1_quantiser) — so the reference's dp4a outputs on the B200 sit up to 0.6 of the output
RMS away from the reference's own CPU golden.  The oracle models the source (full fp16 scales) and is pinned to that
CPU golden elsewhere.  Here the dp4a rows are checked in the way the records allow: fed the very q8_1 blocks the
reference's quantiser produced for each vector (oracle.q8_override), the oracle must reproduce the reference's GPU
results, which pins the integer dots, the scale/min unpacking and the epilogue arithmetic to the reference's GPU
execution.  Everything else (fp16-x GEMVs, batched products, attention, element-wise kernels) is compared as is.

Bars.  The reference builds its kernels with --use_fast_math (approximate division, exp, powf, sinf, cosf), the oracle
uses IEEE arithmetic: the q8_1 quantiser may differ by one code where x/d lands on a rounding tie, fp outputs are held
to 1e-3 relative plus 2e-3 of the output RMS, fp16 element-wise results to 2 fp16 ULP, RoPE to 2 ULP of the larger
magnitude of the rotated pair (the angle at position 32767 carries the fast-math range-reduction error)."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from golden import gpu_cases as gc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu.npz")


@pytest.fixture(scope="module")
def ref():
    return np.load(GOLD)


def f16(a):
    return np.asarray(a).view(np.float16).astype(np.float32)


def close(got, want, rel=1e-3, floor_rms=2e-3, flips=0.0):
    """|got - want| <= rel*|want| + floor_rms*RMS(want) + one fp16 ULP of want (both sides round their fp16 outputs).
    `flips`: fraction of outputs that may lie within TWICE that bound — the reference's activation quantisers divide
    with the fast-math approximation, so a code that sits on a rounding tie can come out one step away from the IEEE
    result and move the outputs of its token by a step of one weight."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    tol = rel * np.abs(want) + floor_rms * np.sqrt(np.mean(want ** 2)) + np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
    err = np.abs(got - want)
    bad = err > tol
    ok = (not bad.any()) or (bad.mean() <= flips and not (err > 2 * tol).any())
    return ok, "max |d| %.4g (rms %.4g), %d outside" % (err.max(), np.sqrt(np.mean(want ** 2)), bad.sum())


def ulp16(a):
    a = np.abs(np.asarray(a, np.float32))
    return np.maximum(np.spacing(a.astype(np.float16)).astype(np.float32), np.float32(2.0 ** -24))


def same_inputs(ref, name, *arrays):
    assert np.array_equal(ref[name + "_in"], gc.digest(*arrays)), f"seeded inputs of {name} drifted from the record"


def test_q8_1_quantiser(ref):
    x = gc.q8_1()["x"]
    same_inputs(ref, "q8_1", x)
    blocks = ref["q8_1_blocks"].reshape(-1, 36)
    qs, d, s = orc.quantize_q8_1(x)
    rq = blocks[:, 4:].view(np.int8).reshape(-1)
    diff = np.abs(qs.astype(np.int32) - rq.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.01, (diff.max(), (diff != 0).mean())
    rd = blocks[:, 0:2].copy().view(np.uint16).reshape(-1)
    rs = blocks[:, 2:4].copy().view(np.uint16).reshape(-1)
    # the record's scales are corrupted in their low byte (see the module docstring); their high bytes are the oracle's
    assert np.all((rd & 0xFF) == 0)
    assert np.mean((d.view(np.uint16) & 0xFF00) == rd) > 0.98
    assert np.mean((s.view(np.uint16) & 0xFF00) == (rs & 0xFF00)) > 0.98


@pytest.mark.parametrize("case", ["gemv_q4k", "gemv_q6k"])
def test_gemv_quant_config_shapes(ref, case):
    c = getattr(gc, case)()
    same_inputs(ref, case, c["W"], c["x"])
    with orc.q8_override(ref[case + "_q8"]):
        got = orc.entry_gemv_quant(c["W"], c["t"], c["x"], c["M"], c["K"]).astype(np.float32)
    ok, msg = close(got, f16(ref[case + "_y"]))
    assert ok, msg


def test_full_precision_scales_are_what_the_cpu_golden_implies(ref):
    """The other half of the argument: with full fp16 q8_1 scales the dp4a model stays within the 8-bit activation
    rounding of the reference's own CPU golden (dequantise + fp32 dot, pinned bit for bit in test_oracle_golden.py);
    with the block scales of the B200 record it does not."""
    c = gc.gemv_q4k()
    M = 512
    W = np.ascontiguousarray(c["W"][:M])
    golden = orc.gemv_float(W, 12, c["x"], M, c["K"])
    rms = float(np.sqrt(np.mean(golden.astype(np.float64) ** 2)))
    full = orc.entry_gemv_quant(W, 12, c["x"], M, c["K"]).astype(np.float32)
    with orc.q8_override(ref["gemv_q4k_q8"]):
        trunc = orc.entry_gemv_quant(W, 12, c["x"], M, c["K"]).astype(np.float32)
    e_full = float(np.sqrt(np.mean((full - golden) ** 2))) / rms
    e_trunc = float(np.sqrt(np.mean((trunc - golden) ** 2))) / rms
    assert e_full < 0.02 and e_trunc > 5 * e_full, (e_full, e_trunc)


@pytest.mark.parametrize("case", ["gemv_add_wo", "gemv_add_down"])
def test_gemv_quant_add(ref, case):
    c = getattr(gc, case)()
    same_inputs(ref, case, c["W"], c["x"], c["res"])
    got = orc.entry_gemv_quant_add(c["W"], c["t"], c["x"], c["res"], c["M"], c["K"]).astype(np.float32)
    ok, msg = close(got, f16(ref[case + "_y"]))
    assert ok, msg


def test_gemv_quant_f32(ref):
    c = gc.gemv_f32()
    same_inputs(ref, "gemv_f32", c["W"], c["x"])
    got = orc.entry_gemv_quant_f32(c["W"], c["t"], c["x"], c["M"], c["K"])
    ok, msg = close(got, ref["gemv_f32_y"])
    assert ok, msg


@pytest.mark.parametrize("case", ["gemv_pair", "gemv_triple"])
def test_gemv_shared_activation(ref, case):
    c = getattr(gc, case)()
    Ws = [c[f"W{i}"] for i in range(len(c["Ms"]))]
    same_inputs(ref, case, *Ws, c["x"])
    with orc.q8_override(ref[case + "_q8"]):
        ys = orc.entry_gemv_multi(Ws, list(c["ts"]), list(c["Ms"]), c["x"], c["K"])
    for i, y in enumerate(ys):
        ok, msg = close(y.astype(np.float32), f16(ref[f"{case}_y{i}"]))
        assert ok, f"matrix {i}: {msg}"


def test_gemm_batch8_q6k(ref):
    c = gc.gemv_q6k()
    same_inputs(ref, "gemm_q6k_b8", c["W"], c["X8"])
    got = orc.entry_gemm_quant_batched(c["W"], 14, c["X8"], c["M"], 8, c["K"]).astype(np.float32)
    ok, msg = close(got, f16(ref["gemm_q6k_b8_y"]))
    assert ok, msg


@pytest.mark.parametrize("t,N", [(12, 512), (12, 2048), (12, 8192), (14, 2048)])
def test_gemm_prefill_shapes(ref, t, N):
    c = gc.gemm(t, N)
    name = f"gemm_t{t}_N{N}"
    same_inputs(ref, name, c["W"], c["X"])
    assert np.array_equal(ref[name + "_sel"], c["sel"])
    Xs = np.ascontiguousarray(c["X"][c["sel"]])          # a token's output depends on that token alone
    got = orc.entry_gemm_quant_batched(c["W"], t, Xs, c["M"], len(c["sel"]), c["K"]).astype(np.float32)
    ok, msg = close(got, f16(ref[name + "_y"]), flips=1e-4)
    assert ok, msg


@pytest.mark.parametrize("L", gc.ATTN_LENGTHS)
def test_decode_attention_int8(ref, L):
    c = gc.attention(L)
    same_inputs(ref, f"attn_L{L}", c["q"], c["k"], c["v"], c["ks"], c["vs"])
    got = orc.attention_decode(c["q"], c["k"], c["v"], gc.NH, gc.NKV, gc.HD, L, gc.SCALE, True, c["ks"], c["vs"]).astype(np.float32)
    want = f16(ref[f"attn_L{L}_out"]).reshape(gc.NH, gc.HD)
    tol = 1e-3 * np.abs(want) + 2e-3 * np.abs(want).max(axis=-1, keepdims=True) + 1e-6
    assert np.all(np.abs(got - want) <= tol), float(np.abs(got - want).max())


@pytest.mark.parametrize("N", [33, 512])
def test_prefill_attention_int8(ref, N):
    c = gc.attention_prefill(N)
    same_inputs(ref, f"prefill_attn_N{N}", c["q"], c["k"], c["v"], c["ks"], c["vs"])
    sel = gc.prefill_sample(N)
    assert np.array_equal(ref[f"prefill_attn_N{N}_sel"], sel)
    got = orc.attention_prefill(c["q"], c["k"], c["v"], gc.NH, gc.NKV, gc.HD, N, 0, gc.SCALE, True, c["ks"], c["vs"]).astype(np.float32)[sel]
    want = f16(ref[f"prefill_attn_N{N}_out"]).reshape(len(sel), gc.NH, gc.HD)
    tol = 1e-3 * np.abs(want) + 2e-3 * np.abs(want).max(axis=-1, keepdims=True) + 1e-6
    assert np.all(np.abs(got - want) <= tol), float(np.abs(got - want).max())


def test_elementwise(ref):
    e = gc.elementwise()
    same_inputs(ref, "elementwise", e["x"], e["res"], e["w"], e["qh"], e["kh"], e["wh"], e["g"], e["u"], e["Wemb"])
    for key, res, x, w, rows, dim in (("rmsnorm_res", e["res"], e["x"], e["w"], 1, gc.H), ("rmsnorm_plain", None, e["x"], e["w"], 1, gc.H),
                                      ("rmsnorm_heads", None, e["qh"], e["wh"], gc.NH, gc.HD)):
        got = orc.rmsnorm(x, res, w, rows, dim, 1e-6).astype(np.float32)
        want = f16(ref[key])
        assert np.all(np.abs(got - want) <= 2 * ulp16(want)), key
    for pos in e["positions"]:
        q, k = orc.rope(e["qh"], e["kh"], gc.NH, gc.NKV, gc.HD, int(pos), 1e6, True)
        for got, key, nh in ((q, f"rope_q_{pos}", gc.NH), (k, f"rope_k_{pos}", gc.NKV)):
            got = got.astype(np.float32).reshape(nh, 2, gc.HD // 2); want = f16(ref[key]).reshape(nh, 2, gc.HD // 2)
            mag = np.maximum(np.abs(want[:, 0]), np.abs(want[:, 1]))[:, None, :]
            # fast-math sinf/cosf: absolute error grows with the angle (up to ~pos * 2^-21 after range reduction)
            bound = 2 * ulp16(mag) + mag * (2e-2 if pos > 10000 else 5e-4)
            assert np.all(np.abs(got - want) <= bound), (key, float(np.abs(got - want).max()))
    codes, scales = orc.fp16_to_int8(e["kh"], gc.NKV, gc.HD)
    assert np.abs(codes.reshape(-1).astype(np.int32) - ref["kvq_codes"].astype(np.int32)).max() <= 1
    assert np.allclose(scales, ref["kvq_scales"], rtol=1e-6)
    got = orc.swiglu(e["g"], e["u"]).astype(np.float32); want = f16(ref["swiglu"])
    assert np.all(np.abs(got - want) <= 2 * ulp16(want))
    got = orc.dequant_embedding_row(e["Wemb"], 12, 37, gc.H).astype(np.float32); want = f16(ref["embedding_row37"])
    assert np.all(np.abs(got - want) <= ulp16(want))
