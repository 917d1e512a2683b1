"""Shared test configuration: import paths, the ``gpu`` marker and small helpers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "moe-explore_b200"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

# MOE_TEST_GATHER_IN_GEMM=0/1 runs the whole suite with the other row-gather form of the layer (rows copied into the
# expert-sorted layout first / gathered by the GEMMs' operand loads); unset = the package default.
if os.environ.get("MOE_TEST_GATHER_IN_GEMM") in ("0", "1"):
    import moe_explore.expert_compute as _ec

    _ec.GATHER_IN_GEMM_DEFAULT = os.environ["MOE_TEST_GATHER_IN_GEMM"] == "1"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native():
    """The ctypes binding, with the library built if it is missing (nvcc cross-compiles on CPU hosts)."""
    from moe_explore import _native

    if not os.path.exists(_native.LIB_PATH):
        import importlib.util

        spec = importlib.util.spec_from_file_location("build_native", os.path.join(ROOT, "moe-explore_b200", "build_native.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    _native.load()
    return _native


def load_golden(name):
    import numpy as np

    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
