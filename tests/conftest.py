import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG_DIR = os.path.join(ROOT, "24ppopp-liger_b200")


def load_package():
    """The package directory name is not a Python identifier; import it under the alias liger_b200."""
    if "liger_b200" in sys.modules:
        return sys.modules["liger_b200"]
    spec = importlib.util.spec_from_file_location(
        "liger_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["liger_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def liger():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def gpu(liger):
    """The loaded CUDA library on a machine with a GPU; GPU tests never fall back to anything else."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    lib = liger.lib()
    return lib
