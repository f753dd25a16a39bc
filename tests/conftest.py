import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without one is skipped, never silently passed.
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
    """The checker libraries and the product library exist before any test runs (both build without a GPU)."""
    import importlib.util

    import oracle.build as ob

    ob.build()
    lib = os.path.join(ROOT, "strixite_b200", "libstrixite_b200.so")
    if not os.path.exists(lib):
        spec = importlib.util.spec_from_file_location("_sb_build", os.path.join(ROOT, "strixite_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    yield
