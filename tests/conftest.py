"""Shared fixtures.  Tests marked ``gpu`` need a CUDA device and the built library; the
rest run on a CPU-only box (oracle vs golden vectors, host logic, ABI surface)."""
from __future__ import annotations

import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

PKG_NAME = "optimize_inference_gpt-oss_b200"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The ctypes binding.  Where nvcc is around the library is rebuilt first if any source or
    header is newer than it (the build is incremental), so the tests never run a stale binary;
    without nvcc a missing library is an error and a present one is used as it is."""
    mod = importlib.import_module(PKG_NAME)
    build = importlib.import_module(PKG_NAME + ".build")
    if os.path.exists(build.NVCC):
        build.build()
    mod.load()
    return mod


@pytest.fixture(scope="session", autouse=True)
def _checked_build_report(request):
    """When the session runs on the checked build of the library (GPTOSS_B200_LIB pointing at
    libgptoss_b200_bounds.so), its closing line says how many pointer arguments were held
    against their allocations and how many violations were seen."""
    yield
    mod = sys.modules.get(PKG_NAME)
    if mod is None or getattr(mod, "_lib", None) is None:
        return
    lib = mod._lib
    if lib.gptoss_bounds_enabled():
        import json
        rec = {"enabled": 1, "violations": int(lib.gptoss_bounds_violations()),
               "checked_spans": int(lib.gptoss_bounds_checked_spans())}
        with request.config.pluginmanager.getplugin("capturemanager").global_and_fixture_disabled():
            print("\n[bounds]" + json.dumps(rec))


@pytest.fixture(scope="session")
def orc():
    import oracle
    import shutil
    if shutil.which("gcc") or not os.path.exists(oracle.ORACLE_SO):
        oracle.build(ref=None)  # make: rebuilt only when a source is newer
    return oracle.Oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own compiled CPU functions; skipped where never built."""
    import oracle
    if not oracle.have_reference():
        if os.path.exists(os.path.join(oracle.REFERENCE_CHECKOUT, "run.cpp")):
            oracle.build(ref=True)
        else:
            pytest.skip("oracle/_ref/libgptoss_ref.so not built and no reference checkout here")
    return oracle.Reference()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "golden.npz"))


@pytest.fixture(scope="session")
def gpu(pkg):
    """Selects device 0; fails (does not skip) when a gpu-marked test finds no device."""
    n = pkg.device_count()
    assert n > 0, "gpu-marked test without a CUDA device"
    pkg.set_device(0)
    return pkg


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({4: np.uint32, 2: np.uint16, 8: np.uint64}[a.dtype.itemsize])


def assert_bit_equal(a, b, what=""):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    ne = bits(a) != bits(b)
    assert not ne.any(), f"{what}: {int(ne.sum())} of {ne.size} elements differ; first at {np.argwhere(ne)[0]}"


def rel_err(got, want, floor):
    """max |got - want| / max(|want|, floor)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor))) if got.size else 0.0
