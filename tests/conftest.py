import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "cuda-kernel-qwen3-8b-awq_b200")
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def load_package():
    """The package directory name is not an identifier: load it under the name qw3awq_b200."""
    if "qw3awq_b200" in sys.modules:
        return sys.modules["qw3awq_b200"]
    spec = importlib.util.spec_from_file_location("qw3awq_b200", os.path.join(PKG_DIR, "__init__.py"),
                                                  submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["qw3awq_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def orc():
    import orc as _orc
    _orc.lib()
    return _orc


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu was run without a CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def ops(pkg, cuda):
    import importlib
    return importlib.import_module("qw3awq_b200.ops")
