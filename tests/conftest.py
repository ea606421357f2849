"""Test configuration: the ``gpu`` marker, an in-tree build of the native libraries before the first
test, and the repository root on ``sys.path`` (for ``oracle`` and the package)."""
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _load_build_module():
    spec = importlib.util.spec_from_file_location("_pmoe_build", ROOT / "prime_flash_moe_b200" / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    # build (or reuse) the libraries before any test module imports the package
    _load_build_module().build_all()
    from oracle import build_ref
    build_ref.build_c_oracle()


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import torch
    return torch.load(ROOT / "tests" / "golden" / "reference_vectors.pt", weights_only=False)
