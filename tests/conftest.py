import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")

# north-star tolerances for FP16 outputs against the FP32 oracle
REL_FRO_TOL = 1e-3
MAX_ABS_TOL = 5e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def errors(y, ref):
    """(relative Frobenius error, max abs error) of y against ref, both as float64 arrays."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return (np.linalg.norm(y - ref) / den if den > 0 else np.linalg.norm(y - ref)), np.abs(y - ref).max()


def assert_close(y, ref, what=""):
    rel, mx = errors(y, ref)
    assert rel <= REL_FRO_TOL and mx <= MAX_ABS_TOL, f"{what}: rel_fro={rel:.3e} max_abs={mx:.3e}"


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle


def layer_oracle(oracle, layer, x, alpha, impl="port", threads=None):
    """FP32 oracle output for a workloads.Layer and an FP16 input (exact up-casts)."""
    return oracle.forward_csr(layer.base_weight.cpu().numpy(), layer.base_scales.float().cpu().numpy(),
                              layer.row_ptr.cpu().numpy(), layer.col.cpu().numpy(),
                              layer.vals.float().cpu().numpy(), x.float().cpu().numpy(), alpha,
                              impl=impl, threads=threads)
