"""Shared test plumbing: the `gpu` marker, import paths, tolerance helpers, golden loaders."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "l1-attention_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def rel_err(x, ref):
    """(max|x-ref| / max|ref|, rms(x-ref) / rms(ref)) -- the norm-wise measures every parity test uses.

    Element-wise relative error is meaningless for gradients with near-zero entries, and the
    reference's own fp32 GPU backward is order-dependent (atomic adds), so tolerances are stated
    against the largest / rms magnitude of the reference array.
    """
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert x.shape == ref.shape, (x.shape, ref.shape)
    if ref.size == 0:
        return 0.0, 0.0
    d = x - ref
    mx = np.abs(ref).max()
    rms = np.sqrt((ref ** 2).mean())
    e1 = np.abs(d).max() / mx if mx > 0 else np.abs(d).max()
    e2 = np.sqrt((d ** 2).mean()) / rms if rms > 0 else np.sqrt((d ** 2).mean())
    return float(e1), float(e2)


def assert_close(x, ref, tol, what=""):
    e1, e2 = rel_err(x, ref)
    assert e1 <= tol and e2 <= tol, "%s: max-rel %.3e rms-rel %.3e > tol %.1e" % (what, e1, e2, tol)


def assert_close_torch(x, ref, tol, what=""):
    """assert_close for device tensors too large to move to the host: same two norm-wise measures,
    accumulated in float64 on the device."""
    import torch
    assert x.shape == ref.shape, (x.shape, ref.shape)
    mx = float(ref.abs().max())
    dmax = float((x - ref).abs().max())
    ss_d = ss_r = 0.0
    xf, rf = x.reshape(-1), ref.reshape(-1)
    for i in range(0, xf.numel(), 1 << 26):
        a, b = xf[i:i + (1 << 26)].double(), rf[i:i + (1 << 26)].double()
        ss_d += float(((a - b) ** 2).sum())
        ss_r += float((b ** 2).sum())
    e1 = dmax / mx if mx > 0 else dmax
    e2 = (ss_d / ss_r) ** 0.5 if ss_r > 0 else ss_d ** 0.5
    assert e1 <= tol and e2 <= tol, "%s: max-rel %.3e rms-rel %.3e > tol %.1e" % (what, e1, e2, tol)
    return e1, e2


@pytest.fixture(scope="session")
def golden():
    d = os.path.join(ROOT, "tests", "golden")
    return {n: np.load(os.path.join(d, n + ".npz")) for n in ("kat", "dense", "sparse", "expandcoo", "fused")}
