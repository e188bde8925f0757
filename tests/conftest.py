"""Shared fixtures: the ctypes package, the CPU oracle, the compiled reference.

Markers: ``gpu`` tests need a B200 and call the CUDA path through the C ABI;
everything else runs on CPU (oracle pins, host logic, ABI surface).
"""
import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_package():
    name = "bmb_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "bare-metal-bard_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def bmb():
    mod = load_package()
    if not os.path.exists(mod.LIB_PATH):
        # Build on demand where nvcc exists (no GPU needed to compile).
        subprocess.check_call([sys.executable, os.path.join(ROOT, "bare-metal-bard_b200", "build.py")])
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def orc():
    import helpers
    return helpers.load_oracle()


@pytest.fixture(scope="session")
def ref():
    import helpers
    r = helpers.load_reference()
    if r is None:
        pytest.skip("oracle/_ref/libbmbref.so not built (needs the reference checkout at build time)")
    return r


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch
