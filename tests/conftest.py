import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Parity tolerances for floating-point results against the fp64 oracle (fp16 inputs, fp32 accumulation).
REL_L2_TOL = 5e-3
MAX_ABS_TOL = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def assert_close(got, want, what=""):
    """rel-L2 <= 5e-3 and max-abs <= 2e-2 against the fp64 oracle."""
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.all(np.isfinite(got)), f"{what}: non-finite values in the result"
    if want.size == 0:
        return
    max_abs = float(np.max(np.abs(got - want)))
    denom = float(np.linalg.norm(want))
    rel = float(np.linalg.norm(got - want)) / denom if denom > 0 else float(np.linalg.norm(got - want))
    assert rel <= REL_L2_TOL, f"{what}: rel-L2 {rel:.3e} > {REL_L2_TOL}"
    assert max_abs <= MAX_ABS_TOL, f"{what}: max-abs {max_abs:.3e} > {MAX_ABS_TOL}"


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_host.npz")
    z = np.load(path)
    cases = {}
    for name in z["names"]:
        name = str(name)
        cases[name] = {k.split("/", 1)[1]: z[k] for k in z.files if k.startswith(name + "/")}
        for key in ("m_vec", "K", "V", "N", "k"):
            cases[name][key] = int(cases[name][key])
    return cases
