"""The allocation-free decode attention entry point, called through the C ABI and compared with the regular
entry point on two calls in a row (the second call finds the built-in scratch full of the first call's values).

Who needs it: hosts that cannot let the library call cudaMalloc — an engine whose pools already own the GPU's
memory, a latency-bound request loop that must not hit a driver call which may stall the device.  The result is also
held against the CPU oracle, and the free device memory is read before and after a call to show that nothing was
allocated.  This file is named so that pytest collects it last: a run that stops at the first failure has then
already run every other test."""
import numpy as np
import pytest

from oracle import oracle as orc
from gpu_util import pkg, dev

pytestmark = pytest.mark.gpu


def _close(a, b):
    a = a.float().cpu().numpy(); b = b.float().cpu().numpy()
    tol = 1e-3 * np.abs(b) + 2e-3 * np.abs(b).max() + 1e-6          # the bar of the attention parity tests
    return bool(np.all(np.abs(a - b) <= tol)), float(np.abs(a - b).max())


def test_noalloc_attention_matches_regular_entry_point_twice():
    import torch
    jb = pkg()
    nh, nkv, hd = 32, 8, 128
    scale = float(1 / np.sqrt(hd))
    rng = np.random.Generator(np.random.PCG64(2024))
    for L in (3000, 700):                                            # 24 slices first, then 6: stale records stay behind
        q = dev(orc.gen_act(rng, nh * hd))
        k, ks = orc.gen_kv(rng, L, nkv, hd); v, vs = orc.gen_kv(rng, L, nkv, hd)
        kd, vd, ksd, vsd = dev(k), dev(v), dev(ks), dev(vs)
        ref = torch.zeros(nh * hd, dtype=torch.float16, device="cuda")
        out = torch.full((nh * hd,), 9.0, dtype=torch.float16, device="cuda")
        jb.flash_attention_decode(ref, q, kd, vd, nh, nkv, hd, hd, L, scale, True, ksd, vsd, 0)
        jb.flash_attention_decode_noalloc(out, q, kd, vd, nh, nkv, hd, hd, L, scale, True, ksd, vsd, 0)
        ok, md = _close(out, ref)
        assert ok, (L, md)
        # ... and against the CPU oracle, the checker of every other attention test
        want = torch.from_numpy(orc.attention_decode(q.cpu().numpy(), k, v, nh, nkv, hd, L, scale, True, ks, vs).astype(np.float32).reshape(-1))
        ok, md = _close(out, want)
        assert ok, ("oracle", L, md)
        # a warm call leaves the amount of free device memory as it found it: nothing is allocated
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        jb.flash_attention_decode_noalloc(out, q, kd, vd, nh, nkv, hd, hd, L, scale, True, ksd, vsd, 0)
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0, (free0, free1)
    # FP16 cache with a sliding window goes through the same built-in scratch
    L, nh2, nkv2, hd2 = 900, 4, 4, 64
    q = dev(orc.gen_act(rng, nh2 * hd2))
    k = dev((rng.standard_normal((L, nkv2, hd2)) * 0.5).astype(np.float16)); v = dev((rng.standard_normal((L, nkv2, hd2)) * 0.5).astype(np.float16))
    ref = torch.zeros(nh2 * hd2, dtype=torch.float16, device="cuda"); out = torch.zeros_like(ref)
    jb.flash_attention_decode(ref, q, k, v, nh2, nkv2, hd2, hd2, L, 0.125, False, None, None, 256)
    jb.flash_attention_decode_noalloc(out, q, k, v, nh2, nkv2, hd2, hd2, L, 0.125, False, None, None, 256)
    ok, md = _close(out, ref)
    assert ok, md


def test_noalloc_attention_rejects_sizes_beyond_the_builtin_scratch():
    import torch
    jb = pkg()
    nh, hd, L = 64, 512, 8192                                        # 64 heads x 32 slices x 514 floats > 256 Ki floats
    t = torch.zeros(nh * hd, dtype=torch.float16, device="cuda")
    kv = torch.zeros(16, dtype=torch.float16, device="cuda")
    with pytest.raises(jb.JllmError) as e:
        jb.flash_attention_decode_noalloc(t, t, kv, kv, nh, nh, hd, hd, L, 1.0, False, None, None, 0)
    assert e.value.code == 6 and "exceed" in str(e.value)
