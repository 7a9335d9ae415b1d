"""Helpers shared by the GPU parity tests."""
import numpy as np

from __graft_entry__ import load_package


def pkg():
    return load_package()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, rel=1e-3, floor=None):
    """|got-want| <= rel*|want| + floor.  The floor (default 2e-3 of the RMS of `want`) covers outputs
    near zero, where a relative bound on an fp16-rounded sum of thousands of terms is meaningless."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if floor is None:
        floor = 2e-3 * float(np.sqrt(np.mean(want ** 2)) + 1e-30)
    bad = np.abs(got - want) > rel * np.abs(want) + floor
    return not bad.any(), float(np.abs(got - want).max())
