"""Shared fixtures.  Tests marked `gpu` need a B200; everything else runs on a CPU box."""

import importlib.util
import os
import shutil
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "cuda-kernel-library_b200")
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs an sm_100 (B200) GPU")


def load_package():
    """Import the package directory (its name has a hyphen) under the module name ckl_b200."""
    if "ckl_b200" in sys.modules:
        return sys.modules["ckl_b200"]
    lib = os.path.join(PKG_DIR, "libckl_gemm.so")
    if not os.path.exists(lib) and shutil.which("nvcc"):
        spec = importlib.util.spec_from_file_location("ckl_b200_build", os.path.join(PKG_DIR, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    spec = importlib.util.spec_from_file_location(
        "ckl_b200", os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ckl_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def ckl():
    return load_package()


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    return oracle


@pytest.fixture(scope="session")
def orc(oracle_mod):
    return oracle_mod.Oracle()
