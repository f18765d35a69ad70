"""The kernels at the full sizes of the benchmark configurations (prefill T = 16,384 with
positions 0..1023 per sequence; 128-expert router; vocabulary-sized argmax and gather).
Inputs come from the library's seeded host generator; results are checked against the
oracle run over the same data (in row blocks where the tensor is large)."""
from __future__ import annotations

import numpy as np
import pytest

from gpu_util import Dev, TOL_BF16, n_bit_diff, rel_err

pytestmark = pytest.mark.gpu

H, QKV, V = 2880, 5120, 201088


def _normal_bf16(pkg, shape, seed, sid, mean=0.0, sd=1.0):
    return pkg.synth_normal(int(np.prod(shape)), pkg.BF16, seed, sid, mean, sd).reshape(shape)


def test_prefill_add_rmsnorm_rope_router(gpu, orc):
    """16 sequences x 1024 positions: contiguous positions walk the whole YaRN table."""
    pkg, d = gpu, Dev(gpu)
    T = 16384
    pos = (np.arange(T) % 1024).astype(np.int32)
    x = pkg.synth_normal(T * H, pkg.F32, 21, 0).reshape(T, H)
    y = _normal_bf16(pkg, (T, H), 21, 1)
    gain = pkg.synth_normal(H, pkg.F32, 21, 2, 1.0, 0.1)
    xb, o = d.put_inout(x), d.out((T, H), pkg.BF16)
    pkg.add_rmsnorm(T, xb, d.put(y), pkg.BF16, d.put(gain), o, pkg.BF16, H)
    want_x, want_o = orc.add_rmsnorm_rows(x, pkg.from_bf16_bits(y).reshape(T, H), gain, threads=0)
    assert n_bit_diff(xb.get(), want_x) == 0
    assert rel_err(o.get(), want_o) <= TOL_BF16

    qkv = _normal_bf16(pkg, (T, QKV), 21, 3)
    bias = pkg.bf16_round(pkg.synth_normal(QKV, pkg.F32, 21, 4, 0.0, 0.02))
    ct, st = pkg.build_rope_tables(1024)
    q = d.out((T, QKV), pkg.BF16)
    pkg.qkv_bias_rope(T, d.put(qkv), pkg.BF16, QKV, d.put(bias), d.put(pos), 0, d.put(ct), d.put(st), 1024,
                      64, 8, 64, q, pkg.BF16, QKV)
    want_q = orc.bias_rope_rows_table(pkg.from_bf16_bits(qkv).reshape(T, QKV), bias, pos, ct, st, threads=0)
    assert rel_err(q.get(), want_q) <= TOL_BF16
    # and against the per-token angles forward() computes, on a sample of rows
    rows = np.arange(0, T, 97)
    want_s = orc.bias_rope_rows(pkg.from_bf16_bits(qkv).reshape(T, QKV)[rows], bias, pos[rows], threads=0)
    assert n_bit_diff(want_s, want_q[rows]) == 0

    for E, sid in ((32, 5), (128, 6)):
        s = _normal_bf16(pkg, (T, E), 21, sid)
        wb, eb = d.out((T, 4), pkg.F32), d.out((T, 4), np.int32)
        pkg.router_topk(T, d.put(s), pkg.BF16, E, 4, wb, eb)
        want_w, want_e = orc.router_rows(pkg.from_bf16_bits(s).reshape(T, E), 4, threads=0)
        assert np.array_equal(eb.get(), want_e)
        assert n_bit_diff(wb.get(), want_w) == 0


def test_decode_swiglu_and_combine_4096_tokens(gpu, orc):
    pkg, d = gpu, Dev(gpu)
    T, K = 4096, 4
    y = _normal_bf16(pkg, (K * T, 2 * H), 22, 0, 0.0, 2.0)
    g = d.out((K * T, H), pkg.BF16)
    pkg.swiglu(d.put(y), pkg.BF16, g, pkg.BF16, K * T, H, 7.0)
    assert rel_err(g.get(), orc.swiglu_rows(pkg.from_bf16_bits(y).reshape(K * T, 2 * H), threads=0)) <= TOL_BF16
    del y

    x = pkg.synth_normal(T * H, pkg.F32, 22, 1).reshape(T, H)
    Z = _normal_bf16(pkg, (K * T, H), 22, 2)
    s = pkg.from_bf16_bits(_normal_bf16(pkg, (T, 128), 22, 3)).reshape(T, 128)
    w, e = orc.router_rows(s, K, threads=0)
    gain = pkg.synth_normal(H, pkg.F32, 22, 4, 1.0, 0.1)
    xb, o = d.put_inout(x), d.out((T, H), pkg.BF16)
    pkg.moe_combine(T, xb, d.put(Z), pkg.BF16, None, d.put(w), d.put(e), K, H, norm_w=d.put(gain), out=o,
                    out_dtype=pkg.BF16)
    want_x = orc.combine_rows(x, pkg.from_bf16_bits(Z).reshape(K * T, H),
                              np.arange(K * T, dtype=np.int32).reshape(T, K), w, e, 128, threads=0)
    assert rel_err(xb.get(), want_x) <= 1e-4
    assert rel_err(o.get(), orc.add_rmsnorm_rows(want_x, None, gain, threads=0)[1]) <= TOL_BF16


def test_vocab_argmax_4096_rows(gpu, orc):
    """bf16 [4096, 201088] N(0,3): 1.65 GB of logits; bf16's coarse grid makes exact ties at
    the maximum common, so the lowest-index rule is exercised on many rows."""
    pkg = gpu
    T = 4096
    buf = pkg.DeviceBuffer(T * V * 2)
    block = 256
    want = np.empty(T, np.int32)
    ties = 0
    for b in range(0, T, block):
        lg = _normal_bf16(pkg, (block, V), 23, b // block, 0.0, 3.0)
        pkg.check(pkg.load().gptoss_upload(buf.ptr + b * V * 2, lg.ctypes.data, lg.nbytes, None))
        pkg.synchronize()
        f = pkg.from_bf16_bits(lg).reshape(block, V)
        want[b:b + block] = orc.argmax_rows(f, threads=0)
        ties += int(np.count_nonzero((f == f.max(axis=1, keepdims=True)).sum(axis=1) > 1))
    assert ties > 0, "the data should contain rows whose maximum occurs more than once"
    keys = pkg.DeviceBuffer.from_numpy(np.zeros(T, np.uint64))
    out = pkg.DeviceBuffer(T * 4)
    pkg.argmax(T, buf, pkg.BF16, V, V, keys, out)
    assert np.array_equal(out.numpy(np.int32, T), want)
    # a 512-row shard is cut into several slices per row and merged through the keys
    assert pkg.load().gptoss_argmax_slices(512, V, pkg.BF16, 1) > 1
    pkg.argmax(512, buf, pkg.BF16, V, V, keys, out)
    assert np.array_equal(out.numpy(np.int32, 512), want[:512])
    assert not keys.numpy(np.uint64, T).any()
    for b in (buf, keys, out):
        b.free()


def test_vocab_embedding_gather_8192_ids(gpu):
    pkg = gpu
    table = _normal_bf16(pkg, (V, H), 24, 0, 0.0, 0.02)
    ids = pkg.synth_uniform_int(8192, 24, 1, 0, V)
    tb = pkg.DeviceBuffer.from_numpy(table)
    x32, x16 = pkg.DeviceBuffer(8192 * H * 4), pkg.DeviceBuffer(8192 * H * 2)
    ib = pkg.DeviceBuffer.from_numpy(ids)
    pkg.embed(8192, tb, pkg.BF16, V, ib, x32, pkg.F32, H)
    pkg.embed(8192, tb, pkg.BF16, V, ib, x16, pkg.BF16, H)
    rows = table[ids]
    assert np.array_equal(x16.numpy(np.uint16, (8192, H)), rows)
    assert np.array_equal(x32.numpy(np.uint32, (8192, H)), rows.astype(np.uint32) << 16)
    # the gather fused with the first norm, from the same table: the two launches' bits
    gain = pkg.DeviceBuffer.from_numpy(pkg.synth_normal(H, pkg.F32, 24, 2, 1.0, 0.1))
    xf, of, o2 = pkg.DeviceBuffer(8192 * H * 4), pkg.DeviceBuffer(8192 * H * 2), pkg.DeviceBuffer(8192 * H * 2)
    pkg.embed_rmsnorm(8192, tb, pkg.BF16, V, ib, xf, gain, of, pkg.BF16, H)
    pkg.add_rmsnorm(8192, x32, None, pkg.F32, gain, o2, pkg.BF16, H)
    assert np.array_equal(xf.numpy(np.uint32, (8192, H)), rows.astype(np.uint32) << 16)
    assert np.array_equal(of.numpy(np.uint16, (8192, H)), o2.numpy(np.uint16, (8192, H)))
    for b in (tb, x32, x16, ib, gain, xf, of, o2):
        b.free()


def test_decode_rotation_with_cache_write_4096_rows(gpu):
    """One decode step of 4096 sequences at the model's head counts, 128 cache slots each:
    rotation + cache write in one launch against the two launches, fp32 rows, every byte of
    the 0.8 GB of caches."""
    pkg = gpu
    T, nq, nkv, slots, n_pos = 4096, 64, 8, 128, 4096
    kv_dim = nkv * 64
    qkv = pkg.synth_normal(T * QKV, pkg.F32, 26, 0).reshape(T, QKV)
    bias = pkg.synth_normal(QKV, pkg.F32, 26, 1, 0.0, 0.02)
    pos = pkg.synth_uniform_int(T, 26, 2, 0, n_pos)
    slot = pkg.synth_uniform_int(T, 26, 3, 0, slots)
    ct, st = pkg.build_rope_tables(n_pos)
    dev = lambda a: pkg.DeviceBuffer.from_numpy(np.ascontiguousarray(a))
    qb, bb, pb, sb, cb, tb = dev(qkv), dev(bias), dev(pos), dev(slot), dev(ct), dev(st)
    n_k = T * slots * kv_dim
    caches = [[pkg.DeviceBuffer.filled(n_k * 2, 0x11), pkg.DeviceBuffer.filled(n_k, 0x11),
               pkg.DeviceBuffer.filled(n_k // 64 * 4, 0x11)] for _ in range(2)]
    o1, o2 = pkg.DeviceBuffer(T * QKV * 4), pkg.DeviceBuffer(T * QKV * 4)
    pkg.qkv_bias_rope_kv(T, qb, pkg.F32, QKV, bb, pb, 0, cb, tb, n_pos, nq, nkv, 64, o1, pkg.F32, QKV,
                         caches[0][0], caches[0][1], caches[0][2], slots, slot_of_row=sb)
    pkg.qkv_bias_rope(T, qb, pkg.F32, QKV, bb, pb, 0, cb, tb, n_pos, nq, nkv, 64, o2, pkg.F32, QKV)
    pkg.kv_cache_write(T, o2, pkg.F32, QKV, nq, nkv, 64, caches[1][0], caches[1][1], caches[1][2], slots,
                       slot_of_row=sb)
    assert np.array_equal(o1.numpy(np.uint32, T * QKV), o2.numpy(np.uint32, T * QKV))
    for a, b, dt in zip(caches[0], caches[1], (np.uint16, np.uint8, np.uint32)):
        got, want = a.numpy(dt, a.nbytes // np.dtype(dt).itemsize), b.numpy(dt, b.nbytes // np.dtype(dt).itemsize)
        assert np.array_equal(got, want)
    written = caches[0][0].numpy(np.uint16, n_k) != 0x1111
    assert T * kv_dim * 0.99 <= written.sum() <= T * kv_dim  # one slot per sequence (a key may happen to equal the fill)
    for b in [qb, bb, pb, sb, cb, tb, o1, o2] + caches[0] + caches[1]:
        b.free()


def test_final_norm_4096_rows(gpu, orc):
    pkg, d = gpu, Dev(gpu)
    T = 4096
    x = pkg.synth_normal(T * H, pkg.F32, 25, 0).reshape(T, H)
    gain = pkg.synth_normal(H, pkg.F32, 25, 1, 1.0, 0.1)
    o = d.out((T, H), pkg.BF16)
    pkg.add_rmsnorm(T, d.put(x), None, pkg.F32, d.put(gain), o, pkg.BF16, H)
    assert rel_err(o.get(), orc.add_rmsnorm_rows(x, None, gain, threads=0)[1]) <= TOL_BF16
