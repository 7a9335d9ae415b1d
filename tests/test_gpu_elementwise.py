"""GPU parity of the element-wise family, KV quantiser, embedding rows and pools (C ABI vs oracle)."""
import numpy as np
import pytest

from oracle import oracle as orc
from gpu_util import pkg, dev, close

pytestmark = pytest.mark.gpu


def _ulp_close(got, want, ulps=1):
    """fp16 results within `ulps` units in the last place of each other."""
    g = np.asarray(got, np.float16).astype(np.float32)
    w = np.asarray(want, np.float16).astype(np.float32)
    ulp = np.maximum(np.abs(np.spacing(np.asarray(want, np.float16))).astype(np.float32), 6e-8)
    return bool(np.all(np.abs(g - w) <= ulps * ulp)), float(np.max(np.abs(g - w) / ulp))


@pytest.mark.parametrize("rows,dim,res,wf32", [(1, 2560, False, True), (32, 128, False, True), (8, 128, True, False), (5, 1024, True, True)])
def test_rmsnorm(rows, dim, res, wf32):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(rows + dim))
    x = orc.gen_act(rng, rows * dim)
    r = orc.gen_act(rng, rows * dim) if res else None
    w = (1 + 0.02 * rng.standard_normal(dim)).astype(np.float32 if wf32 else np.float16)
    out = torch.zeros(rows * dim, dtype=torch.float16, device="cuda")
    jb.fused_rmsnorm_residual(out, dev(x), None if r is None else dev(r), dev(w), rows, dim, 1e-6, wf32)
    want = orc.rmsnorm(x, r, w, rows, dim, 1e-6)
    ok, worst = _ulp_close(out.cpu().numpy(), want, 1)
    assert ok, worst
    # in place (Qwen3 QK-norm calls it with output == x)
    xd = dev(x)
    jb.fused_rmsnorm_residual(xd, xd, None if r is None else dev(r), dev(w), rows, dim, 1e-6, wf32)
    assert torch.equal(xd, out)


def test_rmsnorm_known_answer():
    import torch
    jb = pkg()
    ones = torch.ones(256, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(ones)
    jb.fused_rmsnorm_residual(out, ones, ones, torch.ones(256, dtype=torch.float32, device="cuda"), 1, 256, 1e-6, True)
    assert float((out.float() - 1).abs().max()) < 0.05        # tests/test_kernels.cu:21-48


@pytest.mark.parametrize("pos", [0, 1, 77, 4095, 32767])
@pytest.mark.parametrize("neox", [True, False])
def test_rope(pos, neox):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(pos + 5))
    nh, nkv, hd = 32, 8, 128
    q = orc.gen_act(rng, nh * hd)
    k = orc.gen_act(rng, nkv * hd)
    qd, kd = dev(q), dev(k)
    jb.rope_inplace(qd, kd, nh, nkv, hd, pos, 1e6, neox)
    wq, wk = orc.rope(q, k, nh, nkv, hd, pos, 1e6, neox)
    ok, worst = _ulp_close(qd.cpu().numpy(), wq, 1)
    assert ok, worst
    ok, worst = _ulp_close(kd.cpu().numpy(), wk, 1)
    assert ok, worst
    if pos == 0:
        assert np.array_equal(qd.cpu().numpy(), q)              # tests/test_kernels.cu: position 0 is the identity


def test_rope_table_equals_trig_path():
    """tests/test_rope_table.cu:43-139: table path and trig path give identical bits."""
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(31))
    nh, nkv, hd = 8, 2, 128
    q = orc.gen_act(rng, nh * hd)
    k = orc.gen_act(rng, nkv * hd)
    a_q, a_k = dev(q), dev(k)
    jb.rope_inplace(a_q, a_k, nh, nkv, hd, 123, 10000.0, True)
    jb.rope_precompute_table(512, hd, 10000.0)
    b_q, b_k = dev(q), dev(k)
    jb.rope_inplace(b_q, b_k, nh, nkv, hd, 123, 10000.0, True)
    d_pos = torch.tensor([123], dtype=torch.int32, device="cuda")
    c_q, c_k = dev(q), dev(k)
    jb.rope_inplace_dyn(c_q, c_k, nh, nkv, hd, d_pos, 10000.0, True)
    jb.rope_clear_tables()
    assert torch.equal(a_q, b_q) and torch.equal(a_k, b_k) and torch.equal(a_q, c_q) and torch.equal(a_k, c_k)


def test_rope_store_and_batched_variants():
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(37))
    nh, nkv, hd, N, start = 4, 2, 64, 5, 9
    q = orc.gen_act(rng, N * nh * hd).reshape(N, nh * hd)
    k = orc.gen_act(rng, N * nkv * hd).reshape(N, nkv * hd)
    v = orc.gen_act(rng, N * nkv * hd).reshape(N, nkv * hd)
    qd, kd, vd = dev(q), dev(k), dev(v)
    kc = torch.zeros((start + N, nkv * hd), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    jb.lib.jllm_b200_rope_inplace_store_kv_fp16_batched(
        jb._ptr(qd), jb._ptr(kd), jb._ptr(vd), jb._ptr(kc[start:]), jb._ptr(vc[start:]), nkv * hd, nh, nkv, hd, start, N, nh * hd, nkv * hd,
        __import__("ctypes").c_float(1e4), 1, jb._stream())
    for t in range(N):
        wq, wk = orc.rope(q[t], k[t], nh, nkv, hd, start + t, 1e4, True)
        assert _ulp_close(qd[t].cpu().numpy(), wq)[0] and _ulp_close(kd[t].cpu().numpy(), wk)[0]
        assert torch.equal(kc[start + t], kd[t]) and torch.equal(vc[start + t], vd[t])


def test_swiglu_geglu_scale_softcap_softmax():
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(41))
    n = 9728 + 1                                               # odd length exercises the tail element
    g = (rng.standard_normal(n) * 3).astype(np.float16)
    u = orc.gen_act(rng, n)
    out = torch.zeros(n, dtype=torch.float16, device="cuda")
    jb.fused_swiglu(out, dev(g), dev(u), 1, n)
    assert _ulp_close(out.cpu().numpy(), orc.swiglu(g, u), 1)[0]
    jb.fused_geglu(out, dev(g), dev(u), 1, n)
    assert _ulp_close(out.cpu().numpy(), orc.geglu(g, u), 1)[0]
    # a multiple of eight elements takes the 16-byte form of the kernel: the same bits as the two-element form on a copy
    # whose length is not a multiple of eight
    n8 = 16 * 9728
    g8 = (rng.standard_normal(n8 + 1) * 3).astype(np.float16); u8 = orc.gen_act(rng, n8 + 1)
    for fn in (jb.fused_swiglu, jb.fused_geglu):
        wide = torch.zeros(n8, dtype=torch.float16, device="cuda"); narrow = torch.zeros(n8 + 1, dtype=torch.float16, device="cuda")
        fn(wide, dev(g8[:n8].copy()), dev(u8[:n8].copy()), 16, 9728)
        fn(narrow, dev(g8), dev(u8), 1, n8 + 1)
        assert torch.equal(wide, narrow[:n8])
    assert _ulp_close(wide.cpu().numpy()[:9728], orc.geglu(g8[:9728], u8[:9728]), 1)[0]
    one = torch.tensor([1.0], dtype=torch.float16, device="cuda"); two = torch.tensor([2.0], dtype=torch.float16, device="cuda")
    o1 = torch.zeros(1, dtype=torch.float16, device="cuda")
    jb.fused_swiglu(o1, one, two, 1, 1)
    assert abs(float(o1[0]) - 1.4621) < 0.05                  # tests/test_kernels.cu silu(1)*2
    x = dev(u[:1001].copy())
    jb.vec_scale(x, 1001, 1.5)
    want = (u[:1000].astype(np.float16) * np.float16(1.5)).astype(np.float16)
    assert np.array_equal(x.cpu().numpy()[:1000], want)
    lg = dev(rng.standard_normal(5000).astype(np.float32) * 40)
    ref = 30.0 * np.tanh(lg.cpu().numpy() / 30.0)
    jb.logit_softcap(lg, 5000, 30.0)
    assert np.allclose(lg.cpu().numpy(), ref, rtol=1e-5, atol=1e-5)
    p = dev(rng.standard_normal(151936).astype(np.float32) * 4)
    want = orc.softmax(p.cpu().numpy())
    jb.softmax_inplace(p, 151936)
    got = p.cpu().numpy()
    # a sequential fp32 sum over 151936 terms (the oracle) is itself only good to ~1e-4; both sit within 1e-3 of float64
    assert abs(got.sum() - 1) < 1e-4 and np.allclose(got, want, rtol=1e-3, atol=1e-12)


@pytest.mark.parametrize("rows,cols", [(8, 128), (1, 4096), (3, 100)])
def test_fp16_to_int8_bit_exact(rows, cols):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(rows * cols))
    src = orc.gen_act(rng, rows * cols)
    src[:cols // 2] *= 0                                      # an all-zero stretch
    dst = torch.zeros(rows * cols, dtype=torch.int8, device="cuda")
    sc = torch.zeros(rows, dtype=torch.float32, device="cuda")
    jb.fp16_to_int8(dst, sc, dev(src), rows, cols)
    wq, ws = orc.fp16_to_int8(src, rows, cols)
    assert np.array_equal(dst.cpu().numpy().reshape(rows, cols), wq)
    assert np.array_equal(sc.cpu().numpy(), ws)
    # round trip: tests/test_kv_int8_convert.cu:74-164 (relative error <= 2 % of the row maximum)
    back = wq.astype(np.float32) * ws[:, None]
    s = src.astype(np.float32).reshape(rows, cols)
    assert np.all(np.abs(back - s) <= 0.02 * np.abs(s).max(1, keepdims=True) + 1e-12)
    z = torch.zeros(128, dtype=torch.float16, device="cuda")
    jb.fp16_to_int8(dst, sc, z, 1, 128)                        # zero row: scale 0, codes 0
    assert float(sc[0]) == 0.0 and int(dst[:128].abs().sum()) == 0


@pytest.mark.parametrize("t", [12, 14])
def test_embedding_row_bit_exact(t):
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(t))
    vocab, hidden = 50, 2560
    W = orc.gen_weight(rng, t, vocab, hidden)
    Wd = dev(W)
    for tok in (0, 17, 49):
        dst = torch.zeros(hidden, dtype=torch.float16, device="cuda")
        assert jb.dequant_embedding_row(dst, Wd, t, tok, hidden)
        assert np.array_equal(dst.cpu().numpy().view(np.uint16), orc.dequant_embedding_row(W, t, tok, hidden).view(np.uint16))
    assert not jb.dequant_embedding_row(dst, Wd, 13, 0, hidden)          # unsupported type -> false
    assert not jb.dequant_embedding_row(dst, Wd, t, 0, 100)              # hidden not a multiple of 256 -> false


def test_dense_gemv():
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(43))
    M, N, K = 37, 3, 300
    W = rng.standard_normal((M, K)).astype(np.float32)
    x = orc.gen_act(rng, N * K).reshape(N, K)
    for wt, Wd in ((0, dev(W)), (1, dev(W.astype(np.float16))), (30, dev(W).bfloat16())):
        out = torch.zeros((N, M), dtype=torch.float16, device="cuda")
        jb.gemm_dense_batched(out, Wd, wt, dev(x), M, N, K)
        ref = x.astype(np.float32) @ Wd.float().cpu().numpy().T
        assert np.allclose(out.float().cpu().numpy(), ref, rtol=2e-3, atol=2e-2)


def test_kv_pool_layout_and_scratch_pool():
    """tests/test_kv_scale_storage.cu:32-165 and tests/test_memory.cpp:13-83 restated."""
    import torch
    jb = pkg()
    L, nkv, hd, ctx = 3, 8, 128, 64
    p = jb.KVCachePool()
    assert p.init(L, nkv, hd, ctx, 0, 1)
    assert p.kv_scales_bytes() == 2 * L * ctx * nkv * 4
    assert p.capacity_bytes() == L * ctx * 2 * nkv * hd
    base = p.key_ptr(0, 0)
    assert p.val_ptr(0, 0) - base == ctx * nkv * hd               # values follow all keys of the layer
    assert p.key_ptr(1, 0) - base == 2 * ctx * nkv * hd
    assert p.key_ptr(0, 5) - base == 5 * nkv * hd
    s0 = p.kv_scale_ptr(0, 0, False)
    assert p.kv_scale_ptr(0, 0, True) - s0 == ctx * nkv * 4       # K -> V stride
    assert p.kv_scale_ptr(1, 0, False) - s0 == 2 * ctx * nkv * 4  # layer stride
    assert p.kv_scale_ptr(0, 7, False) - s0 == 7 * nkv * 4
    assert p.kv_scale_ptr(L, 0, False) is None and p.kv_scale_ptr(0, ctx, False) is None
    # gather / scatter round trip
    used = 10
    img = np.random.default_rng(0).integers(-127, 128, p.packed_used_bytes(used), dtype=np.int8)
    assert p.scatter_from_host(img, used, True) and p.used_tokens() == used
    back = np.zeros_like(img)
    assert p.gather_used_to_host(back, used) and np.array_equal(back, img)
    assert not p.gather_used_to_host(back, ctx + 1)
    p.destroy()
    f = jb.KVCachePool()
    assert f.init(2, 2, 64, 16, 0, 2)
    assert f.kv_scale_ptr(0, 0, False) is None and f.kv_scales_bytes() == 0      # FP16 mode has no scales
    f.destroy()
    s = jb.ScratchPool()
    assert s.init(1 << 20) and s.capacity() == 1 << 20 and s.used() == 0
    a = s.get(100); b = s.get(300)
    assert b - a == 256 and s.used() == 256 + 512
    m = s.mark(); s.get(1000); s.rewind_to(m)
    assert s.used() == m
    assert s.get(2 << 20) is None                                  # exhausted -> null
    s.reset()
    assert s.used() == 0
    s.destroy()


def test_qkv_prep_equals_separate_calls():
    import torch
    jb = pkg()
    rng = np.random.Generator(np.random.PCG64(47))
    nh, nkv, hd, ctx, pos = 32, 8, 128, 32, 11
    q = dev(orc.gen_act(rng, nh * hd)); k = dev(orc.gen_act(rng, nkv * hd)); v = dev(orc.gen_act(rng, nkv * hd))
    qn = dev((1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)); kn = dev((1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    q1, k1 = q.clone(), k.clone()
    jb.fused_rmsnorm_residual(q1, q1, None, qn, nh, hd, 1e-6, True)
    jb.fused_rmsnorm_residual(k1, k1, None, kn, nkv, hd, 1e-6, True)
    jb.rope_inplace(q1, k1, nh, nkv, hd, pos, 1e6, True)
    kc1 = torch.zeros((ctx, nkv * hd), dtype=torch.int8, device="cuda"); vc1 = torch.zeros_like(kc1)
    ks1 = torch.zeros((ctx, nkv), dtype=torch.float32, device="cuda"); vs1 = torch.zeros_like(ks1)
    jb.fp16_to_int8(kc1[pos], ks1[pos], k1, nkv, hd)
    jb.fp16_to_int8(vc1[pos], vs1[pos], v, nkv, hd)
    q2 = q.clone()
    kc2 = torch.zeros_like(kc1); vc2 = torch.zeros_like(kc1); ks2 = torch.zeros_like(ks1); vs2 = torch.zeros_like(ks1)
    jb.qkv_prep_int8(q2, k, v, qn, kn, 1e-6, kc2, vc2, ks2, vs2, nh, nkv, hd, pos, None, 1e6, True)
    assert torch.equal(q1, q2) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2) and torch.equal(ks1, ks2) and torch.equal(vs1, vs2)
