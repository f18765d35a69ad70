"""The reference's launcher names (include/gptoss_launchers.hpp) used from a plain C++ program,
as a port of the reference engine would use them, against the oracle: add_rmsnorm_bf16,
rope_kv_bf16 (keys only, as the engine calls it), router_topk_wave, moe_combine_rmsnorm."""
from __future__ import annotations

import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from gpu_util import TOL_BF16, n_bit_diff, rel_err

pytestmark = pytest.mark.gpu


def test_engine_launch_sites_through_the_reference_names(gpu, orc, tmp_path):
    pkg = gpu
    exe = tmp_path / "launcher_demo"
    pkg_dir = os.path.dirname(pkg.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "launcher_demo.cpp"), "-o", str(exe), "-L", pkg_dir,
                    "-lgptoss_b200", f"-Wl,-rpath,{pkg_dir}"], check=True)
    B, H, E, k, slots, slot = 37, 2880, 32, 4, 128, 77
    NQ, NKV, QKV = 64, 8, 5120
    r = np.random.default_rng(5)
    x = r.standard_normal((B, H)).astype(np.float32)
    y = r.standard_normal((B, H)).astype(np.float32)
    w = (1 + 0.1 * r.standard_normal(H)).astype(np.float32)
    qkv = r.standard_normal((B, QKV)).astype(np.float32)
    ct, st = pkg.build_rope_tables(slot + 1)
    logits = r.standard_normal((B, E)).astype(np.float32)
    Z = r.standard_normal((B * k, H)).astype(np.float32)
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(np.array([B, H, E, k, slots, slot], np.int32).tobytes())
        for a in (x, y, w, qkv, ct[slot], st[slot], logits, Z):
            f.write(np.ascontiguousarray(a, np.float32).tobytes())
    subprocess.run([str(exe), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], check=True, timeout=300)
    raw = open(tmp_path / "out.bin", "rb").read()
    at = 0

    def take(dtype, shape):
        nonlocal at
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        a = np.frombuffer(raw, dtype, int(np.prod(shape)), at).reshape(shape)
        at += n
        return a

    kv = B * slots * NKV * 64
    x1, t1 = take(np.float32, (B, H)), take(np.uint16, (B, H))
    q1, kc, vq, vs = take(np.float32, (B, QKV)), take(np.uint16, kv), take(np.int8, kv), take(np.float32, kv // 64)
    tw, te = take(np.float32, (B, k)), take(np.int32, (B, k))
    x2, t2 = take(np.float32, (B, H)), take(np.uint16, (B, H))
    assert at == len(raw)

    want_x1, want_n1 = orc.add_rmsnorm_rows(x, y, w)
    assert n_bit_diff(x1, want_x1) == 0
    assert rel_err(pkg.from_bf16_bits(t1).reshape(B, H), want_n1) <= TOL_BF16
    # rope_kv_bf16 with rotate_q = false: queries untouched, keys rotated, values untouched
    assert n_bit_diff(q1[:, :NQ * 64], qkv[:, :NQ * 64]) == 0
    assert n_bit_diff(q1[:, (NQ + NKV) * 64:], qkv[:, (NQ + NKV) * 64:]) == 0
    k_rot = orc.rotate_heads(qkv[0, NQ * 64:(NQ + NKV) * 64], ct[slot], st[slot], NKV, 64)
    assert rel_err(q1[0, NQ * 64:(NQ + NKV) * 64], k_rot) <= 1e-5  # FMA rounding (the reference's GPU form) vs separate products
    want_k = np.full(kv, 0x5555, np.uint16)
    want_q = np.full(kv, 0x55, np.int8)
    want_s = np.frombuffer(bytes([0x55]) * (kv // 64 * 4), np.float32).copy()
    orc.kv_cache_write(q1, NQ, NKV, want_k, want_q, want_s, slots, np.full(B, slot, np.int32))
    assert np.array_equal(kc, want_k) and np.array_equal(vq, want_q) and n_bit_diff(vs, want_s) == 0
    want_w, want_e = orc.router_rows(logits, k)
    assert np.array_equal(te, want_e) and n_bit_diff(tw, want_w) == 0
    want_x2 = orc.combine_rows(want_x1, Z, np.arange(B * k, dtype=np.int32).reshape(B, k), want_w, want_e, E)
    assert rel_err(x2, want_x2) <= 1e-4
    assert rel_err(pkg.from_bf16_bits(t2).reshape(B, H), orc.add_rmsnorm_rows(want_x2, None, w)[1]) <= TOL_BF16
