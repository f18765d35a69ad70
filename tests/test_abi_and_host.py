"""CPU-side checks of the shipped library: it loads, exports every symbol the headers
declare, validates arguments before touching CUDA, and its host-side pieces (RoPE table
builder, synthetic generator, sharding) behave.  No kernel is launched here."""
from __future__ import annotations

import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT, assert_bit_equal


def _declared(header: str):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"GPTOSS_API\s+[\w\s\*]+?\b(gptoss_\w+)\s*\(", text)))


def test_headers_and_exports_agree(pkg):
    declared = _declared("gptoss_kernels.h") + _declared("gptoss_engine.h")
    assert len(declared) >= 40
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    missing = [d for d in declared if d not in exported]
    assert not missing, f"declared in include/ but not exported: {missing}"
    extra = sorted(e for e in exported if e.startswith("gptoss_") and e not in declared)
    assert not extra, f"exported but not declared: {extra}"
    # the Python prototypes cover the same surface
    assert sorted(pkg.PROTOTYPES) == sorted(declared)


def test_headers_compile_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "gptoss_kernels.h"\n#include "gptoss_engine.h"\nint main(void){return GPTOSS_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src),
                    "-o", str(tmp_path / "t.o")], check=True)


def test_version_and_status_strings(pkg):
    lib = pkg.load()
    assert re.match(rb"\d+\.\d+\.\d+", lib.gptoss_version())
    assert lib.gptoss_status_string(pkg.OK) == b"ok"
    assert b"argument" in lib.gptoss_status_string(pkg.ERR_BAD_ARG)


def test_bad_arguments_are_refused_before_any_launch(pkg):
    """Every entry point checks sizes, dtypes and null pointers first and returns a status
    instead of aborting (the reference exits the process in HIP_CHECK)."""
    lib, P = pkg.load(), 0x1000  # a fake non-null address; never dereferenced
    B, U = pkg.ERR_BAD_ARG, pkg.ERR_UNSUPPORTED
    assert lib.gptoss_embed(None, -1, P, 1, 10, P, P, 0, 64, 0) == B
    assert lib.gptoss_embed(None, 4, None, 1, 10, P, P, 0, 64, 0) == B
    assert lib.gptoss_embed(None, 4, P, 7, 10, P, P, 0, 64, 0) == B
    assert lib.gptoss_embed(None, 4, P, 0, 10, P, P, 1, 64, 0) == U      # fp32 table -> bf16 rows
    assert lib.gptoss_embed(None, 0, None, 1, 10, None, None, 0, 64, 0) == pkg.OK  # empty batch
    assert lib.gptoss_add_rmsnorm(None, 4, None, None, 0, P, P, 0, 64, 0) == B
    assert lib.gptoss_add_rmsnorm(None, 4, P, None, 0, P, P, 0, 0, 0) == B
    assert lib.gptoss_add_rmsnorm(None, 4, P, None, 0, P, P, 1, 64, 0) == B  # in place needs fp32 out
    assert lib.gptoss_add_rmsnorm(None, 0, None, None, 0, None, None, 0, 64, 0) == pkg.OK
    assert lib.gptoss_qkv_bias_rope(None, 4, P, 0, 100, None, None, 0, P, P, 16, 64, 8, 64, P, 0, 5120, 0) == B  # stride < row
    assert lib.gptoss_qkv_bias_rope(None, 4, P, 0, 5120, None, None, 0, P, P, 16, 64, 8, 63, P, 0, 5120, 0) == B  # odd head
    assert lib.gptoss_qkv_bias_rope(None, 4, P, 0, 5120, None, None, 0, P, P, 16, 64, 8, 64, P, 1, 5120, 0) == B  # in place, dtype change
    assert lib.gptoss_qkv_bias_rope(None, 4, P, 0, 5120, None, None, 0, None, P, 16, 64, 8, 64, P + 64, 0, 5120, 0) == B
    assert lib.gptoss_router_topk(None, 4, P, 0, 32, 0, P, P, None, None, 0) == B
    assert lib.gptoss_router_topk(None, 4, P, 0, 32, 33, P, P, None, None, 0) == B
    assert lib.gptoss_router_topk(None, 4, P, 0, 512, 4, P, P, None, None, 0) == U
    assert lib.gptoss_router_topk(None, 4, P, 0, 32, 9, P, P, None, None, 0) == U
    assert lib.gptoss_swiglu(None, None, 0, P, 0, 4, 64, 7.0, 0) == B
    assert lib.gptoss_swiglu(None, P, 0, P, 0, 4, 0, 7.0, 0) == B
    assert lib.gptoss_swiglu(None, P, 0, P, 0, 4, 64, -1.0, 0) == B
    assert lib.gptoss_swiglu(None, None, 0, None, 0, 0, 64, 7.0, 0) == pkg.OK
    assert lib.gptoss_moe_combine(None, 4, P, P, 0, None, P, None, 4, 64, None, None, None, 0, 0) == B
    assert lib.gptoss_moe_combine(None, 4, P, P, 0, None, P, P, 9, 64, None, None, None, 0, 0) == U
    assert lib.gptoss_moe_combine(None, 4, P, P, 0, None, P, P, 4, 64, None, P, None, 0, 0) == B  # norm without out
    assert lib.gptoss_argmax(None, 4, P, 0, 0, 0, None, P, 0) == B
    assert lib.gptoss_argmax(None, 4, P, 0, 100, 50, None, P, 0) == B  # stride < V
    assert lib.gptoss_argmax(None, 4, P, 0, 100, 100, None, None, 0) == B
    assert lib.gptoss_argmax(None, 0, None, 0, 100, 100, None, None, 0) == pkg.OK
    assert lib.gptoss_chain_create(None, 4, 1, None) == B
    assert lib.gptoss_build_rope_tables(0, 64, 150000.0, 32.0, 4096.0, 32.0, 1.0, P, P) == B


def test_missing_library_is_loud(pkg, monkeypatch):
    import importlib
    mod = importlib.reload(importlib.import_module("optimize_inference_gpt-oss_b200"))
    monkeypatch.setattr(mod, "LIB_PATH", "/nonexistent/libgptoss_b200.so")
    monkeypatch.setattr(mod, "_lib", None)
    with pytest.raises(mod.GptossError, match="no fallback"):
        mod.load()


def test_rope_tables_match_the_oracle_bit_for_bit(pkg, orc):
    cs, sn = pkg.build_rope_tables(4096)
    oc, os_ = orc.yarn_table(4096)
    assert_bit_equal(cs, oc, "cos table")
    assert_bit_equal(sn, os_, "sin table")
    cs, sn = pkg.build_rope_tables(300, head_dim=128, factor=1.0)
    oc, os_ = orc.yarn_table(300, head_dim=128, factor=1.0)
    assert_bit_equal(cs, oc)
    assert_bit_equal(sn, os_)


def test_bf16_host_helpers(pkg):
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.0, -0.0, np.inf, 3.4e38], np.float32)
    b = pkg.to_bf16_bits(x)
    assert b[0] == 0x3F80 and b[1] == 0x3F80           # tie rounds to even (down)
    assert b[2] == 0x3F82                               # tie rounds to even (up)
    assert b[5] == 0x8000 and b[6] == 0x7F80 and b[7] == 0x7F80  # overflow rounds to inf
    assert np.isnan(pkg.from_bf16_bits(pkg.to_bf16_bits(np.array([np.nan], np.float32))))[0]
    r = np.random.default_rng(0).standard_normal(10000).astype(np.float32)
    q = pkg.bf16_round(r)
    assert np.max(np.abs(q - r) / np.abs(r)) <= 2.0 ** -8
    assert_bit_equal(pkg.bf16_round(q), q)


def test_synthetic_generator(pkg):
    a = pkg.synth_normal(200001, pkg.F32, seed=7, stream_id=3, threads=1)
    b = pkg.synth_normal(200001, pkg.F32, seed=7, stream_id=3, threads=5)
    assert_bit_equal(a, b, "thread count must not change the bits")
    assert abs(float(a.mean())) < 0.01 and abs(float(a.std()) - 1.0) < 0.01
    c = pkg.synth_normal(200001, pkg.F32, seed=7, stream_id=4)
    assert not np.array_equal(a, c)
    h = pkg.synth_normal(4096, pkg.BF16, seed=7, stream_id=3, mean=1.0, sd=0.1)
    f = pkg.synth_normal(4096, pkg.F32, seed=7, stream_id=3, mean=1.0, sd=0.1)
    assert np.array_equal(h, pkg.to_bf16_bits(f))
    ids = pkg.synth_uniform_int(100000, 1, 0, 0, 201088)
    assert ids.min() >= 0 and ids.max() < 201088 and ids.max() > 200000 and len(np.unique(ids)) > 70000


def test_shard_ranges(pkg):
    import importlib
    sh = importlib.import_module("optimize_inference_gpt-oss_b200.sharding")
    for total, world, gran in [(4096, 8, 1), (16384, 8, 1024), (16384, 4, 1024), (7, 4, 1), (3, 8, 1), (0, 2, 1)]:
        prev = 0
        for r in range(world):
            b, e = sh.shard_range(total, world, r, gran)
            assert b == prev and e >= b and b % gran == 0
            prev = e
        assert prev == total
    assert sh.shard_range(4096, 8, 3) == (1536, 2048)
    sizes = [sh.shard_range(7, 4, r) for r in range(4)]
    assert [e - b for b, e in sizes] == [2, 2, 2, 1]
    with pytest.raises(ValueError):
        sh.shard_range(1000, 4, 0, 1024)
    with pytest.raises(ValueError):
        sh.shard_range(8, 4, 4)


def test_reference_named_launchers_compile_as_plain_cxx(tmp_path):
    """include/gptoss_launchers.hpp (the reference's launcher names over the C ABI) and the demo
    that uses it build with g++ alone and link against the library."""
    out = tmp_path / "launcher_demo"
    pkg_dir = os.path.join(ROOT, "optimize_inference_gpt-oss_b200")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "launcher_demo.cpp"), "-o", str(out), "-L", pkg_dir,
                    "-lgptoss_b200", f"-Wl,-rpath,{pkg_dir}"], check=True)
    assert out.exists()


def test_exp2_table_of_the_device_expf():
    """The 32-entry table in csrc/exact_math.cuh is bits(2^(i/32)) - (i << 47), with 2^(i/32)
    correctly rounded to double: recomputed here at 60 decimal digits."""
    import decimal
    import re
    import struct
    src = open(os.path.join(ROOT, "optimize_inference_gpt-oss_b200", "csrc", "exact_math.cuh")).read()
    body = src[src.index("kExp2Tab32[32]"):]
    body = body[:body.index("};")]
    table = [int(h, 16) for h in re.findall(r"0x([0-9a-f]{16})ull", body)]
    assert len(table) == 32
    decimal.getcontext().prec = 60
    for i, t in enumerate(table):
        exact = decimal.Decimal(2) ** (decimal.Decimal(i) / 32)
        want = struct.unpack("<Q", struct.pack("<d", float(exact)))[0]   # float(Decimal) rounds correctly
        assert (t + (i << 47)) & 0xFFFFFFFFFFFFFFFF == want, i
