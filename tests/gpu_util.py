"""Helpers shared by the GPU parity tests."""
import numpy as np

from __graft_entry__ import load_package


def pkg():
    return load_package()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ulp16(a):
    """One fp16 unit in the last place at the magnitude of `a` (both sides of a comparison round their outputs to fp16)."""
    with np.errstate(over="ignore"):
        u = np.spacing(np.abs(np.asarray(a, np.float32)).astype(np.float16)).astype(np.float64)
    return np.where(np.isfinite(u), u, 32.0)


def close(got, want, rel=1e-3, floor=None):
    """|got-want| <= rel*|want| + floor + one fp16 ULP.  The floor (default 2e-3 of the RMS of `want`) covers outputs
    near zero, where a relative bound on an fp16-rounded sum of thousands of terms is meaningless."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if floor is None:
        floor = 2e-3 * float(np.sqrt(np.mean(want ** 2)) + 1e-30)
    bad = np.abs(got - want) > rel * np.abs(want) + floor + ulp16(want)
    return not bad.any(), float(np.abs(got - want).max())


def close_gemm(got, want, N, M, rel=1e-3, floor=3e-3, rms_bound=6e-4, flips=0.0):
    """Bound for a batched product y[t][r] whose error scales with the magnitudes of token t and row r:
    |got-want| <= rel*|want| + one fp16 ULP + floor*s[t][r] with s[t][r] = RMS(want[t,:]) * RMS(want[:,r]) / RMS(want), and the
    RMS of the whole error at most rms_bound of the RMS of `want`.  The tensor-core prefill path rounds each
    operand product to fp16 (2^-11 relative): measured error RMS 3.7e-4 of the output scale, so `floor` is an
    8-sigma bound for the millions of outputs a test holds and `rms_bound` the accuracy statement proper."""
    g = np.asarray(got, np.float64).reshape(N, M)
    w = np.asarray(want, np.float64).reshape(N, M)
    rt = np.sqrt(np.mean(w ** 2, axis=1, keepdims=True)) + 1e-30
    ra = float(np.sqrt(np.mean(w ** 2)) + 1e-30)
    # the magnitude of a row needs enough tokens to be estimated from the outputs; with a handful, use the overall scale
    rr = (np.sqrt(np.mean(w ** 2, axis=0, keepdims=True)) + 1e-30) if N >= 64 else np.full((1, M), ra)
    s = rt * rr / ra
    err = np.abs(g - w)
    bad = err > rel * np.abs(w) + floor * s + ulp16(w)
    e_rms = float(np.sqrt(np.mean((g - w) ** 2))) / ra
    # `flips`: fraction of outputs allowed within twice the bound (comparisons with records of the reference's GPU run, whose
    # fast-math activation quantiser can land one code away from the IEEE result on a rounding tie)
    inside = (not bad.any()) or (bad.mean() <= flips and not (err > 2 * (rel * np.abs(w) + floor * s + ulp16(w))).any())
    return inside and e_rms <= rms_bound, "max |d| %.4g, error rms %.3g of output rms, %d outside" % (float(err.max()), e_rms, int(bad.sum()))
