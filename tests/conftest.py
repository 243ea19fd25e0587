import json
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


def golden_manifest():
    with open(os.path.join(GOLDEN, "manifest.json")) as f:
        return json.load(f)


def golden_case(name):
    with np.load(os.path.join(GOLDEN, f"case_{name}.npz")) as z:
        return {k: z[k] for k in z.files}


def golden_codebooks():
    with np.load(os.path.join(GOLDEN, "codebooks.npz")) as z:
        return {k: z[k] for k in z.files}


CASES = golden_manifest()["cases"]
CASE_IDS = [c["name"] for c in CASES]


@pytest.fixture(scope="session")
def lib_built():
    """Build libtq_sm100.so if it is missing or stale (needs nvcc only, no GPU)."""
    from project_tensor_b200 import build
    return build.build()
