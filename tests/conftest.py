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


def reference_tree():
    """The reference library's source tree, or None where it is not mounted."""
    path = os.environ.get("CKL_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    return path if os.path.isdir(os.path.join(path, "include", "ckl")) else None


def dropin_binary(name: str) -> str:
    """Path of a reference driver built unchanged against this library (oracle/_ref/<name>).
    Where the reference tree is mounted a missing binary is built, and a failure to build it
    fails the test; only a machine with neither the tree nor a prebuilt binary skips."""
    exe = os.path.join(ROOT, "oracle", "_ref", name)
    if os.path.exists(exe):
        return exe
    ref = reference_tree()
    if ref is None:
        pytest.skip(f"oracle/_ref/{name} was not shipped and the reference tree is not mounted")
    import subprocess
    load_package()  # the drivers link libckl_gemm.so
    out = subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "dropin", f"REFERENCE={ref}"],
                         capture_output=True, text=True)
    if out.returncode != 0 or not os.path.exists(exe):
        pytest.fail(f"could not build oracle/_ref/{name} from {ref}:\n{out.stderr[-2000:]}")
    return exe


def tool_binary(name: str) -> str:
    """Path of a command-line tool of this library (cuda-kernel-library_b200/build/<name>);
    built on demand, and a tool that cannot be built fails the test."""
    exe = os.path.join(PKG_DIR, "build", name)
    if os.path.exists(exe):
        return exe
    import subprocess
    load_package()
    out = subprocess.run(["make", "-s", "-C", os.path.join(PKG_DIR, "tools")], capture_output=True, text=True)
    if out.returncode != 0 or not os.path.exists(exe):
        pytest.fail(f"could not build {exe}:\n{out.stderr[-2000:]}")
    return exe


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
