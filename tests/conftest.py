"""pytest configuration: the `gpu` marker and shared loaders."""
import importlib.util
import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_binding():
    """Loads sd3.c_b200/sd3_b200.py (the package directory name has a dot)."""
    name = "sd3_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(REPO, "sd3.c_b200", "sd3_b200.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def sd3():
    return load_binding()


def golden(name):
    import torch
    return torch.load(os.path.join(REPO, "tests", "golden", name), map_location="cpu")
