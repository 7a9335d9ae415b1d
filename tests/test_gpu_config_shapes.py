"""GPU parity at the benchmark configurations' own shapes, through the C ABI, against BOTH checkers: the CPU oracle
and the records of the reference's own GPU kernels on the same seeded inputs (tests/golden/ref_gpu.npz).

The reference's dp4a decode GEMV stores corrupted q8_1 block scales when compiled for sm_100a (see
tests/test_oracle_ref_gpu.py), so for gemv_quant / _pair / _triple the checker is the oracle alone — which
test_oracle_ref_gpu.py ties to the reference's GPU run through the recorded blocks — and the record is compared
wherever the reference's GPU result is sound: fp16-x GEMVs, batched products, attention.

Bars: fp outputs 1e-3 relative plus 2e-3 of the output RMS (attention: of the head's largest output); the batched
products use gpu_util.close_gemm (see its docstring)."""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from golden import gpu_cases as gc
from gpu_util import pkg, dev, close, close_gemm, ulp16

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu.npz")


@pytest.fixture(scope="module")
def ref():
    return np.load(GOLD)


def f16(a):
    return np.asarray(a).view(np.float16).astype(np.float32)


def both(got, oracle_want, ref_want, what):
    for name, want in (("oracle", oracle_want), ("reference GPU record", ref_want)):
        ok, md = close(got, np.asarray(want, np.float32))
        assert ok, f"{what} against the {name}: max diff {md}"


@pytest.mark.parametrize("case", ["gemv_q4k", "gemv_q6k"])
def test_gemv_quant_configs_0_and_1(ref, case):
    import torch
    jb = pkg()
    c = getattr(gc, case)()
    y = torch.zeros(c["M"], dtype=torch.float16, device="cuda")
    jb.gemv_quant(y, dev(c["W"]), c["t"], dev(c["x"]), c["M"], c["K"])
    ok, md = close(y.float().cpu().numpy(), orc.entry_gemv_quant(c["W"], c["t"], c["x"], c["M"], c["K"]).astype(np.float32))
    assert ok, f"{case} against the oracle: max diff {md}"
    assert jb.device_status() == 0


def test_integer_dots_bit_exact_at_config_shapes():
    import torch
    jb = pkg()
    for case in ("gemv_q4k", "gemv_q6k"):
        c = getattr(gc, case)()
        M = 512                                   # rows of the full-width matrix; every row runs the same code
        G = c["K"] // 32 if c["t"] == 12 else c["K"] // 16
        dots = torch.zeros((M, G), dtype=torch.int32, device="cuda")
        y = torch.zeros(M, dtype=torch.float16, device="cuda")
        W = np.ascontiguousarray(c["W"][:M])
        jb.gemv_quant_int_dots(y, dots, dev(W), c["t"], dev(c["x"]), M, c["K"])
        qs, _, _ = orc.quantize_q8_1(c["x"])
        assert np.array_equal(dots.cpu().numpy(), orc.q8_int_dots(W, c["t"], M, c["K"], qs)), case


def test_batch8_q6k_config_1(ref):
    import torch
    jb = pkg()
    c = gc.gemv_q6k()
    y = torch.zeros((8, c["M"]), dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched(y, dev(c["W"]), 14, dev(c["X8"]), c["M"], 8, c["K"])
    got = y.float().cpu().numpy()
    for name, want in (("oracle", orc.entry_gemm_quant_batched(c["W"], 14, c["X8"], c["M"], 8, c["K"]).astype(np.float32)),
                       ("reference GPU record", f16(ref["gemm_q6k_b8_y"]))):
        ok, msg = close_gemm(got, want, 8, c["M"], flips=0.0 if name == "oracle" else 1e-4)
        assert ok, f"batch 8 against the {name}: {msg}"


@pytest.mark.parametrize("case", ["gemv_pair", "gemv_triple"])
def test_shared_activation_gemvs(ref, case):
    import torch
    jb = pkg()
    c = getattr(gc, case)()
    n = len(c["Ms"])
    Ws = [c[f"W{i}"] for i in range(n)]
    ys = [torch.zeros(m, dtype=torch.float16, device="cuda") for m in c["Ms"]]
    x = dev(c["x"])
    if n == 2:
        jb.gemv_quant_pair(ys[0], dev(Ws[0]), c["ts"][0], c["Ms"][0], ys[1], dev(Ws[1]), c["ts"][1], c["Ms"][1], x, c["K"])
    else:
        jb.gemv_quant_triple(ys[0], dev(Ws[0]), c["ts"][0], c["Ms"][0], ys[1], dev(Ws[1]), c["ts"][1], c["Ms"][1],
                             ys[2], dev(Ws[2]), c["ts"][2], c["Ms"][2], x, c["K"])
    want = orc.entry_gemv_multi(Ws, list(c["ts"]), list(c["Ms"]), c["x"], c["K"])
    for i in range(n):
        ok, md = close(ys[i].float().cpu().numpy(), want[i].astype(np.float32))
        assert ok, f"{case}[{i}] against the oracle: max diff {md}"


@pytest.mark.parametrize("case", ["gemv_add_wo", "gemv_add_down"])
def test_residual_gemvs(ref, case):
    import torch
    jb = pkg()
    c = getattr(gc, case)()
    y = torch.zeros(c["M"], dtype=torch.float16, device="cuda")
    jb.gemv_quant_add(y, dev(c["W"]), c["t"], dev(c["x"]), dev(c["res"]), c["M"], c["K"])
    both(y.float().cpu().numpy(), orc.entry_gemv_quant_add(c["W"], c["t"], c["x"], c["res"], c["M"], c["K"]), f16(ref[case + "_y"]), case)


def test_logits_slice_f32(ref):
    import torch
    jb = pkg()
    c = gc.gemv_f32()
    y = torch.zeros(c["M"], dtype=torch.float32, device="cuda")
    jb.gemv_quant_f32(y, dev(c["W"]), c["t"], dev(c["x"]), c["M"], c["K"])
    both(y.cpu().numpy(), orc.entry_gemv_quant_f32(c["W"], c["t"], c["x"], c["M"], c["K"]), ref["gemv_f32_y"], "gemv_quant_f32")


def _attn_check(got, want, what):
    got = np.asarray(got, np.float32).reshape(want.shape)
    tol = 1e-3 * np.abs(want) + 2e-3 * np.abs(want).max(axis=-1, keepdims=True) + ulp16(want)      # + one fp16 ULP of the output
    assert np.all(np.abs(got - want) <= tol), f"{what}: max diff {float(np.abs(got - want).max())}"


@pytest.mark.parametrize("L", gc.ATTN_LENGTHS)
def test_decode_attention_config_2(ref, L):
    import torch
    jb = pkg()
    c = gc.attention(L)
    out = torch.zeros(gc.NH * gc.HD, dtype=torch.float16, device="cuda")
    jb.flash_attention_decode(out, dev(c["q"]), dev(c["k"]), dev(c["v"]), gc.NH, gc.NKV, gc.HD, gc.HD, L, gc.SCALE, True, dev(c["ks"]), dev(c["vs"]), 0)
    got = out.float().cpu().numpy()
    _attn_check(got, orc.attention_decode(c["q"], c["k"], c["v"], gc.NH, gc.NKV, gc.HD, L, gc.SCALE, True, c["ks"], c["vs"]).astype(np.float32), "oracle")
    _attn_check(got, f16(ref[f"attn_L{L}_out"]).reshape(gc.NH, gc.HD), "reference GPU record")
    assert jb.device_status() == 0


def test_decode_attention_64_ragged_sequences():
    """Configuration 2's batch: 64 sequences with lengths drawn uniformly from [256, 8192], each with its own cache."""
    import torch
    jb = pkg()
    lens = gc.ragged_lengths()
    B = len(lens)
    rng = gc.rng_for(2, 8)
    q = orc.gen_act(rng, B * gc.NH * gc.HD).reshape(B, gc.NH * gc.HD)
    host, devs = [], []
    for L in lens:
        k, ks = orc.gen_kv(rng, int(L), gc.NKV, gc.HD); v, vs = orc.gen_kv(rng, int(L), gc.NKV, gc.HD)
        host.append((k, v, ks, vs)); devs.append(tuple(dev(a) for a in (k, v, ks, vs)))
    ptrs = [torch.tensor([d[i].data_ptr() for d in devs], dtype=torch.int64, device="cuda") for i in range(4)]
    out = torch.zeros((B, gc.NH * gc.HD), dtype=torch.float16, device="cuda")
    jb.flash_attention_decode_batched(out, dev(q), ptrs[0], ptrs[1], ptrs[2], ptrs[3], torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                      B, int(lens.max()), gc.NH, gc.NKV, gc.HD, gc.SCALE, True)
    got = out.float().cpu().numpy()
    # the same batch through a plan (tensor maps built once; every cache padded to the longest length)
    Lmax = int(lens.max())
    pad = lambda t: torch.cat([t, torch.zeros((Lmax - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device="cuda")])
    padded = [tuple(pad(t) for t in d) for d in devs]
    plan = jb.AttnPlan([p[0] for p in padded], [p[1] for p in padded], [p[2] for p in padded], [p[3] for p in padded], Lmax, gc.NKV)
    out2 = torch.zeros((B, gc.NH * gc.HD), dtype=torch.float16, device="cuda")
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    plan.decode(out2, dev(q), lens_d, gc.NH, gc.SCALE)
    plan.decode(out2, dev(q), lens_d, gc.NH, gc.SCALE)              # twice: the slice counters must be back at zero
    got2 = out2.float().cpu().numpy()
    plan.close()
    for b in range(B):
        k, v, ks, vs = host[b]
        want = orc.attention_decode(q[b], k, v, gc.NH, gc.NKV, gc.HD, int(lens[b]), gc.SCALE, True, ks, vs).astype(np.float32)
        _attn_check(got[b], want, f"pointer lists, sequence {b} (length {lens[b]})")
        _attn_check(got2[b], want, f"plan, sequence {b} (length {lens[b]})")
    assert jb.device_status() == 0


@pytest.mark.parametrize("t,N", [(12, 512), (12, 2048), (12, 8192), (14, 2048)])
def test_prefill_gemm_config_3(ref, t, N):
    import torch
    jb = pkg()
    c = gc.gemm(t, N)
    y = torch.zeros((N, c["M"]), dtype=torch.float16, device="cuda")
    jb.gemm_quant_batched(y, dev(c["W"]), t, dev(c["X"]), c["M"], N, c["K"])
    sel = c["sel"]
    got = y[torch.from_numpy(sel).long().cuda()].float().cpu().numpy()
    Xs = np.ascontiguousarray(c["X"][sel])
    want = orc.entry_gemm_quant_batched(c["W"], t, Xs, c["M"], len(sel), c["K"]).astype(np.float32)
    for name, w in (("oracle", want), ("reference GPU record", f16(ref[f"gemm_t{t}_N{N}_y"]))):
        ok, msg = close_gemm(got, w, len(sel), c["M"], flips=0.0 if name == "oracle" else 1e-4)
        assert ok, f"M={c['M']} K={c['K']} N={N} against the {name}: {msg}"
    # every token row, not only the sampled ones, must be finite and of the sampled rows' magnitude
    rms_all = y.float().pow(2).mean(dim=1).sqrt().cpu().numpy()
    assert np.all(np.isfinite(rms_all)) and rms_all.min() > 0.2 * np.sqrt(np.mean(want ** 2))
    assert jb.device_status() == 0
