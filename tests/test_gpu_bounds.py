"""The checked build of the library (-DGPTOSS_BOUNDS, libgptoss_b200_bounds.so) as the stand-in
for a memory checker: the small parity cases of the kernel tests run through it in a child
process and must finish with no refused call and no skipped access, and a probe makes the
mistakes the build exists to catch and checks that each one is refused or skipped -- never
executed."""
from __future__ import annotations

import importlib
import json
import os
import subprocess
import sys

import pytest

from conftest import PKG_NAME, ROOT

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bounds_lib():
    build = importlib.import_module(PKG_NAME + ".build")
    if os.path.exists(build.NVCC):
        build.build_bounds()
    assert os.path.exists(build.BOUNDS_LIB), "libgptoss_b200_bounds.so is not built and there is no nvcc here"
    return build.BOUNDS_LIB


def _env(lib):
    env = dict(os.environ, GPTOSS_B200_LIB=lib)
    env.pop("PYTEST_CURRENT_TEST", None)
    return env


def test_parity_cases_run_clean_under_the_checked_build(gpu, bounds_lib):
    """Kernel and small chain cases through the checked library: every test passes, and the
    session's closing line (printed by conftest.py for a checked build) reports spans checked
    and zero violations."""
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_kernels.py"),
           os.path.join(ROOT, "tests", "test_gpu_chain.py"), "-m", "gpu", "-q", "-x", "-p", "no:cacheprovider",
           "-k", "not 8192 and not 100000 and not full_depth and not config and not 4096 and not producer"]
    r = subprocess.run(cmd, env=_env(bounds_lib), capture_output=True, text=True, cwd=ROOT)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    line = [l for l in r.stdout.splitlines() if l.startswith("[bounds]")]
    assert line, tail
    rec = json.loads(line[-1][len("[bounds]"):])
    assert rec["enabled"] == 1 and rec["violations"] == 0 and rec["checked_spans"] > 1000, rec


def test_the_checked_build_refuses_or_skips_what_it_should(gpu, bounds_lib):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "bounds_probe.py")], env=_env(bounds_lib),
                       capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    got = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    pkg = gpu
    assert got["enabled"] == 1
    assert got["short_out_status"] == pkg.ERR_BAD_ARG and got["short_out_untouched"]
    assert got["violations_after_short_out"] == 1
    assert got["short_strided_status"] == pkg.ERR_BAD_ARG and got["violations_after_strided"] == 2
    for form in ("vector", "scalar"):
        assert got[f"oob_rows_{form}_status"] == pkg.OK and got[f"oob_rows_{form}_exact"]
        assert got[f"oob_rows_{form}_counted"] == 7, got
    assert got["good_call_status"] == pkg.OK and got["good_call_counted"] == 0


def test_the_ordinary_build_reports_no_checking(gpu):
    lib = gpu.load()
    assert lib.gptoss_bounds_enabled() == 0 and lib.gptoss_bounds_violations() == 0
