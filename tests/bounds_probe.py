"""Helper of test_gpu_bounds.py, run as a child process with GPTOSS_B200_LIB pointing at the
checked build of the library: makes a few calls whose buffers are too small for their shape
arguments, or whose row map points past the end of its array, and prints what the library did
about them as one JSON line.  Nothing here can fault: the checked build refuses the
mis-sized calls before launching and skips the out-of-range rows."""
from __future__ import annotations

import importlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    pkg = importlib.import_module("optimize_inference_gpt-oss_b200")
    lib = pkg.load()
    import oracle
    orc = oracle.Oracle()
    out = {"enabled": int(lib.gptoss_bounds_enabled())}
    if not out["enabled"]:  # the ordinary build would run these calls as given: never do that
        print(json.dumps(out))
        sys.exit("not the checked build of the library; nothing was called")
    pkg.set_device(0)
    D = pkg.DeviceBuffer
    T, H, k = 40, 2880, 4
    r = np.random.default_rng(7)
    x = r.standard_normal((T, H)).astype(np.float32)
    gain = np.ones(H, np.float32)
    v0 = lib.gptoss_bounds_violations()

    # 1. an output buffer one row short: refused, nothing launched, the buffer keeps its fill
    dx, dw = D.from_numpy(x), D.from_numpy(gain)
    short = D.filled((T - 1) * H * 4, 0x5A)
    st = lib.gptoss_add_rmsnorm(None, T, dx.ptr, None, pkg.F32, dw.ptr, short.ptr, pkg.F32, H, 0)
    pkg.synchronize()
    out["short_out_status"] = int(st)
    out["short_out_untouched"] = bool((short.numpy(np.uint8, (T - 1) * H * 4) == 0x5A).all())
    out["violations_after_short_out"] = int(lib.gptoss_bounds_violations() - v0)

    # 2. a strided input whose last row runs past the end
    row, stride = 5120, 5200
    qkv = D((T - 1) * stride * 2 + row * 2 - 16)
    qo = D(T * row * 2)
    ct, sn = pkg.build_rope_tables(64, 64)
    dct, dsn = D.from_numpy(ct), D.from_numpy(sn)
    st = lib.gptoss_qkv_bias_rope(None, T, qkv.ptr, pkg.BF16, stride, None, None, 3, dct.ptr, dsn.ptr, 64, 64, 8, 64,
                                  qo.ptr, pkg.BF16, row, 0)
    out["short_strided_status"] = int(st)
    out["violations_after_strided"] = int(lib.gptoss_bounds_violations() - v0)

    # 3. a row map with entries past the end of Z: those pairs are skipped and counted
    w, e = orc.router_rows(r.standard_normal((T, 32)).astype(np.float32), k)
    z_rows = T * k - 7
    z = r.standard_normal((z_rows, H)).astype(np.float32)
    own = np.arange(T * k, dtype=np.int32)                    # the last 7 point past the end
    want_map = np.where(own < z_rows, own, -1).astype(np.int32).reshape(T, k)
    for name, Hd in (("vector", H), ("scalar", 77)):
        zz, xx = np.ascontiguousarray(z[:, :Hd]), np.ascontiguousarray(x[:, :Hd])
        before = lib.gptoss_bounds_violations()
        dxx = D.from_numpy(xx)
        dz, do, dww, de = D.from_numpy(zz), D.from_numpy(own), D.from_numpy(w), D.from_numpy(e)
        st = lib.gptoss_moe_combine(None, T, dxx.ptr, dz.ptr, pkg.F32, do.ptr, dww.ptr, de.ptr, k, Hd, None, None,
                                    None, pkg.F32, pkg.EXACT)
        pkg.synchronize()
        got = dxx.numpy(np.float32, (T, Hd))
        ref = orc.combine_rows(xx, zz, want_map, w, e, 32)
        out[f"oob_rows_{name}_status"] = int(st)
        out[f"oob_rows_{name}_exact"] = bool(np.array_equal(got.view(np.uint32), ref.view(np.uint32)))
        out[f"oob_rows_{name}_counted"] = int(lib.gptoss_bounds_violations() - before)

    # 4. the same call with a map that fits: nothing counted
    before = lib.gptoss_bounds_violations()
    dxx, dz = D.from_numpy(x), D.from_numpy(z)
    fit = D.from_numpy(np.where(own < z_rows, own, 0).astype(np.int32))
    dww, de = D.from_numpy(w), D.from_numpy(e)  # named: a buffer lives as long as its Python object
    st = lib.gptoss_moe_combine(None, T, dxx.ptr, dz.ptr, pkg.F32, fit.ptr, dww.ptr, de.ptr, k,
                                H, None, None, None, pkg.F32, 0)
    pkg.synchronize()
    out["good_call_status"] = int(st)
    out["good_call_counted"] = int(lib.gptoss_bounds_violations() - before)
    out["checked_spans"] = int(lib.gptoss_bounds_checked_spans())
    print(json.dumps(out))


if __name__ == "__main__":
    main()
