"""Shared test configuration: markers, import paths, golden-fixture loader."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "flash-attention-legacy_b200")
for p in (PKG, ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "slow: takes more than a few seconds")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Returns a dict of torch tensors / python scalars from tests/golden/<name>.npz."""
    data = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for key in data.files:
        arr = data[key]
        out[key] = arr.item() if arr.shape == () else torch.from_numpy(arr)
    return out


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN_DIR) if f.startswith(prefix) and f.endswith(".npz"))


@pytest.fixture(scope="session", autouse=True)
def _build_library():
    """The shared library must exist before anything imports the binding."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("fal_b200_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if not os.path.exists(mod.LIB_PATH):
        mod.build()
    yield


@pytest.fixture(autouse=True)
def _cuda_sync_after_test(request):
    """Surfaces asynchronous CUDA errors inside the test that caused them."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        torch.cuda.synchronize()
