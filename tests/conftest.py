import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; the parity tests proper")


def load_build_module():
    """deepwell_b200/_build.py loaded by path (importing the package needs an up-to-date library)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("_dw_build", os.path.join(ROOT, "deepwell_b200", "_build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def native_lib():
    """Builds (if stale) and loads the C-ABI library."""
    b = load_build_module()                # before the package is imported: its import loads the library
    b.build()
    b.build_ext()
    from deepwell_b200 import _native
    return _native.load()


@pytest.fixture(scope="session")
def golden():
    return {name: np.load(os.path.join(GOLDEN, name + ".npz")) for name in ("kat_quant", "config1", "ref_gemm")}


def config1_inputs():
    """The CPU-reference workload: X [2048,4096] N(0,1) with 1% of the entries x50 (outliers), W [4096,4096] N(0,0.02), seed 1234."""
    import torch
    g = torch.Generator("cpu").manual_seed(1234)
    X = torch.randn(2048, 4096, generator=g)
    mask = torch.rand(2048, 4096, generator=g) < 0.01
    X[mask] *= 50
    W = torch.randn(4096, 4096, generator=g) * 0.02
    return X.bfloat16(), W.bfloat16()
