import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Builds the oracle and the CUDA library when they are missing (nvcc cross-compiles without a GPU)."""
    from llama_cu_awq_b200 import build as b
    from oracle import q4_oracle
    if not os.path.exists(b.LIB) or not os.path.exists(b.TEST_LIB):
        b.build()
    if not os.path.exists(q4_oracle.LIB_PATH):
        q4_oracle.build()


# Tolerances of the floating-point parity tests (fp16 outputs, fp32 accumulation):
MAX_REL = 1e-2     # max |y - ref| / max |ref|
MIN_COS = 0.999    # cosine similarity


def rel_err(y, ref):
    y = np.asarray(y, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def cosine(y, ref):
    y = np.asarray(y, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    return float(y @ ref / max(np.linalg.norm(y) * np.linalg.norm(ref), 1e-30))


def assert_close(y, ref, what="", max_rel=MAX_REL, min_cos=MIN_COS):
    assert np.isfinite(np.asarray(y, np.float32)).all(), f"{what}: non-finite output"
    r, c = rel_err(y, ref), cosine(y, ref)
    assert r <= max_rel and c >= min_cos, f"{what}: max rel err {r:.3e} (limit {max_rel}), cosine {c:.6f} (limit {min_cos})"
    return r, c
