import importlib
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pk():
    """The product package (its directory name is not a Python identifier).  The shared
    library is built first if this is a fresh checkout (nvcc cross-compiles without a GPU)."""
    if not (ROOT / "l4-parakeet-rs_b200" / "libpk100.so").exists():
        spec = importlib.util.spec_from_file_location("pk100_build", ROOT / "l4-parakeet-rs_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return importlib.import_module("l4-parakeet-rs_b200")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible (there is no CPU fallback)")
    return torch.device("cuda:0")
