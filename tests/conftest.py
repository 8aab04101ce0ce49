import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with -m gpu; without a device they are skipped rather than failed
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


# Acceptance rule of the benchmark definition: per element |d| <= 2e-2 + 1e-2 |ref| in binary16.
ATOL, RTOL = 2e-2, 1e-2


def error_report(got, ref):
    g = np.asarray(got, dtype=np.float32)
    r = np.asarray(ref, dtype=np.float32)
    d = np.abs(g - r)
    bad = d > (ATOL + RTOL * np.abs(r))
    return dict(max=float(d.max()) if d.size else 0.0, mean=float(d.mean()) if d.size else 0.0,
                violations=int(bad.sum()), n=int(d.size))


def assert_close(got, ref, what="", max_violation_fraction=0.0):
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(np.asarray(got, dtype=np.float32)).all(), f"{what}: non-finite output"
    rep = error_report(got, ref)
    frac = rep["violations"] / max(1, rep["n"])
    assert frac <= max_violation_fraction, f"{what}: {rep}"
    return rep
