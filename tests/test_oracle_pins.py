"""Pins the restated CPU oracle: (1) against the golden vectors the reference's compiled
functions produced (always), (2) against the reference's functions themselves, bit for
bit, on seeded inputs (where oracle/_ref/libgptoss_ref.so is present)."""
from __future__ import annotations

import os

import numpy as np
import pytest

import golden_inputs as gi
import oracle
from conftest import ROOT, assert_bit_equal


# ---- (1) golden known answers -------------------------------------------------------

def test_golden_rmsnorm(orc, golden):
    x, delta, gain = gi.case_rmsnorm()
    xa, normed = orc.add_rmsnorm_rows(x, delta, gain)
    assert_bit_equal(xa, golden["rmsnorm_x"], "x after add")
    assert_bit_equal(normed, golden["rmsnorm_out"], "normed")
    assert_bit_equal(orc.add_rmsnorm_rows(x, None, gain)[1], golden["rmsnorm_only"], "norm only")


def test_golden_yarn_and_rope(orc, golden):
    conc, inv = orc.yarn_inv_freq()
    assert np.float32(conc) == golden["yarn_conc"]
    assert_bit_equal(inv, golden["yarn_inv_freq"], "inv_freq")
    # anchors of the YaRN blend (gpt-oss parameters): concentration, the last
    # pure-extrapolation pair (8) and the first pure-interpolation pair (18)
    assert float(conc).hex() == "0x1.58b90c0000000p+0"
    assert float(inv[0]) == 1.0
    assert float(inv[8]).hex() == "0x1.a043280000000p-5"
    assert float(inv[18]).hex() == "0x1.415b8c0000000p-15"
    assert float(inv[31]).hex() == "0x1.44a5a60000000p-22"
    qkv, bias, pos = gi.case_rope()
    for i, p in enumerate(pos):
        c, s = orc.yarn_cos_sin(int(p))
        assert_bit_equal(c, golden["yarn_cos"][i], f"cos pos {p}")
        assert_bit_equal(s, golden["yarn_sin"][i], f"sin pos {p}")
    assert_bit_equal(orc.bias_rope_rows(qkv, bias, pos), golden["rope_out"], "rope")
    # the table form (what the GPU engine uses) gives the same bits
    ct, st = orc.yarn_table(4096)
    assert_bit_equal(orc.bias_rope_rows_table(qkv, bias, pos, ct, st), golden["rope_out"], "rope via table")


def test_golden_router(orc, golden):
    a, b = gi.case_router()
    w, e = orc.router_rows(a)
    assert np.array_equal(e, golden["router20_e"])
    assert_bit_equal(w, golden["router20_w"], "weights E=32")
    w, e = orc.router_rows(b)
    assert np.array_equal(e, golden["router120_e"])
    assert_bit_equal(w, golden["router120_w"], "weights E=128")


def test_golden_argmax(orc, golden):
    lg = gi.case_argmax()
    got = orc.argmax_rows(lg)
    assert np.array_equal(got, golden["argmax"])
    assert got[1] == 777 and got[2] == 0


def test_golden_forward(orc, golden):
    m = gi.tiny_model()
    cfg = oracle.OrcConfig(*m.values())
    w = gi.uniform(71, (oracle.flat_weight_count(cfg),), 0.35)
    toks = gi.small_ints(72, (10,), 0, m["vocab"])
    assert_bit_equal(orc.forward_seq(cfg, w, toks), golden["forward_logits"], "tiny-model logits")


def test_golden_swiglu_combine_regression(orc, golden):
    assert_bit_equal(orc.swiglu_rows(gi.case_swiglu()), golden["swiglu_out"], "swiglu")
    x, Z, row_of, w, e = gi.case_combine()
    assert_bit_equal(orc.combine_rows(x, Z, row_of, w, e, gi.E20), golden["combine_x"], "combine")


def test_golden_cache_layout_and_bf16_rounding(orc, golden):
    """Where a key element, a value code and a value scale go in the chunk64 caches, and how
    fp32 becomes bf16: the reference's own functions wrote these vectors."""
    b, slot, g, i, slots, kv_dim = gi.case_cache_layout()
    k_at, vq_at, vs_at = orc.cache_indices(b, slot, g, i, slots, kv_dim)
    assert np.array_equal(k_at, golden["cache_k_at"])
    assert np.array_equal(vq_at, golden["cache_vq_at"])
    assert np.array_equal(vs_at, golden["cache_vs_at"])
    assert np.array_equal(orc.f32_to_bf16(gi.case_bf16_rounding()), golden["bf16_bits"])


def test_cache_layout_is_what_the_cache_writer_uses(orc):
    """orc_kv_cache_write places every element where the index functions say."""
    T, n_q, n_kv, slots = 5, 2, 3, 128
    kv_dim = n_kv * 64
    r = np.random.default_rng(5)
    qkv = r.standard_normal((T, (n_q + 2 * n_kv) * 64)).astype(np.float32)
    slot_of = np.array([0, 17, 63, 64, 127], np.int32)
    kc = np.full(T * slots * kv_dim, 0xAAAA, np.uint16)
    vq = np.full(T * slots * kv_dim, 0x55, np.int8)
    vs = np.full(T * slots * n_kv, -1.0, np.float32)
    orc.kv_cache_write(qkv, n_q, n_kv, kc, vq, vs, slots, slot_of)
    bb, gg, ii = np.meshgrid(np.arange(T), np.arange(n_kv), np.arange(64), indexing="ij")
    k_at, vq_at, vs_at = orc.cache_indices(bb.ravel(), slot_of[bb.ravel()], gg.ravel(), ii.ravel(), slots, kv_dim)
    k = qkv[:, n_q * 64:n_q * 64 + kv_dim].reshape(T, n_kv, 64)
    v = qkv[:, n_q * 64 + kv_dim:].reshape(T, n_kv, 64)
    assert np.array_equal(kc[k_at], orc.f32_to_bf16(k).ravel())
    amax = np.abs(v).max(axis=2, keepdims=True)
    codes = np.clip(np.rint(v * (np.float32(127.0) / amax)), -127, 127).astype(np.int8)
    assert np.array_equal(vq[vq_at], codes.ravel())
    assert np.array_equal(vs[vs_at].reshape(T, n_kv, 64)[:, :, 0], (amax / np.float32(127.0))[:, :, 0])
    touched = np.zeros(kc.size, bool)
    touched[k_at] = True
    assert (kc[~touched] == 0xAAAA).all() and len(np.unique(k_at)) == k_at.size == len(np.unique(vq_at))


def test_topk_ties_go_to_the_lowest_index(orc):
    """Guards the one place the CPU program leans on the C library: qsort leaving equal
    scores in index order."""
    v, i = orc.topk(np.array([1, 3, 3, -0.0, 0, 3, 2, 2], np.float32), 4)
    assert list(i) == [1, 2, 5, 6] and list(v) == [3, 3, 3, 2]
    v, i = orc.topk(np.zeros(32, np.float32), 4)
    assert list(i) == [0, 1, 2, 3]
    s = np.zeros(32, np.float32)
    s[5], s[9] = -0.0, 0.0
    assert list(orc.topk(s, 4)[1]) == [0, 1, 2, 3]


def test_argmax_nan_rules(orc):
    nan = np.float32("nan")
    assert orc.argmax(np.array([1, nan, 3, 3], np.float32)) == 2
    assert orc.argmax(np.array([nan, 5, 7], np.float32)) == 0      # NaN in front sticks
    assert orc.argmax(np.array([-np.inf, -np.inf], np.float32)) == 0
    assert orc.argmax(np.array([-0.0, 0.0], np.float32)) == 0


# ---- (2) the reference's own functions, bit for bit ----------------------------------

@pytest.mark.parametrize("n", [1, 7, 64, 1000, 2880, 4096])
def test_ref_rmsnorm(orc, ref, n):
    rng = np.random.default_rng(n)
    for scale in (1e-3, 1.0, 50.0):
        x = (rng.standard_normal(n) * scale).astype(np.float32)
        g = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        assert_bit_equal(orc.rmsnorm(x, g), ref.rmsnorm(x, g), f"rmsnorm n={n} scale={scale}")


@pytest.mark.parametrize("n", [1, 2, 4, 8, 33, 130])
def test_ref_softmax(orc, ref, n):
    rng = np.random.default_rng(100 + n)
    for scale in (0.1, 4.0, 60.0):
        x = (rng.standard_normal(n) * scale).astype(np.float32)
        assert_bit_equal(orc.softmax(x), ref.softmax(x), f"softmax n={n}")


@pytest.mark.parametrize("E,k", [(16, 8), (32, 4), (128, 4), (200, 2), (32, 2)])
def test_ref_topk_with_planted_ties(orc, ref, E, k):
    rng = np.random.default_rng(E * 10 + k)
    for t in range(40):
        s = rng.standard_normal(E).astype(np.float32)
        if t % 3 == 0:
            s[E - 1] = s[rng.integers(0, E - 1)]
        if t % 5 == 0:
            s[1], s[E // 2], s[0], s[E - 2] = 0.0, -0.0, 50.0, 50.0
        if t % 7 == 0:
            s = np.trunc(s * 2).astype(np.float32)
        (v0, i0), (v1, i1) = orc.topk(s, k), ref.topk(s, k)
        assert np.array_equal(i0, i1), (t, i0, i1)
        assert_bit_equal(v0, v1)


def test_ref_yarn(orc, ref):
    assert orc.yarn_inv_freq()[0] == ref.yarn_inv_freq()[0]
    assert_bit_equal(orc.yarn_inv_freq()[1], ref.yarn_inv_freq()[1])
    # unscaled RoPE branch and another head size
    assert_bit_equal(orc.yarn_inv_freq(factor=1.0)[1], ref.yarn_inv_freq(factor=1.0)[1])
    assert_bit_equal(orc.yarn_inv_freq(head_dim=128)[1], ref.yarn_inv_freq(head_dim=128)[1])
    for p in (0, 1, 2, 37, 127, 128, 1023, 1024, 4095, 4096, 131071):
        (c0, s0), (c1, s1) = orc.yarn_cos_sin(p), ref.yarn_cos_sin(p)
        assert_bit_equal(c0, c1, f"cos {p}")
        assert_bit_equal(s0, s1, f"sin {p}")


@pytest.mark.parametrize("heads", [(64, 8), (8, 1), (32, 4)])
def test_ref_bias_rope_rows(orc, ref, heads):
    nq, nkv = heads
    rng = np.random.default_rng(nq)
    T, row = 9, (nq + 2 * nkv) * 64
    qkv = rng.standard_normal((T, row)).astype(np.float32)
    bias = (0.02 * rng.standard_normal(row)).astype(np.float32)
    pos = rng.integers(0, 4096, T).astype(np.int32)
    assert_bit_equal(orc.bias_rope_rows(qkv, bias, pos, nq, nkv), ref.bias_rope_rows(qkv, bias, pos, nq, nkv))
    assert_bit_equal(orc.bias_rope_rows(qkv, None, pos, nq, nkv), ref.bias_rope_rows(qkv, None, pos, nq, nkv))


def test_ref_batched_rows(orc, ref):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((17, 2880)).astype(np.float32)
    d = rng.standard_normal((17, 2880)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(2880)).astype(np.float32)
    for a, b in zip(orc.add_rmsnorm_rows(x, d, g, threads=3), ref.add_rmsnorm_rows(x, d, g, threads=2)):
        assert_bit_equal(a, b)
    s = rng.standard_normal((65, 128)).astype(np.float32)
    (w0, e0), (w1, e1) = orc.router_rows(s, 4, threads=2), ref.router_rows(s, 4, threads=3)
    assert np.array_equal(e0, e1)
    assert_bit_equal(w0, w1)
    lg = rng.standard_normal((5, 50000)).astype(np.float32)
    lg[2, 40000] = lg[2, 123] = 77.0
    assert np.array_equal(orc.argmax_rows(lg), ref.argmax_rows(lg))
    assert orc.argmax_rows(lg)[2] == 123


def test_ref_cache_layout_and_bf16_rounding(orc, ref):
    if not ref.has_cache_layout:
        pytest.skip("reference library built without the kernels' headers")
    r = np.random.default_rng(9)
    for slots, n_kv in ((64, 1), (192, 8), (4096, 8)):
        n = 20000
        b, slot, g, i = r.integers(0, 7, n), r.integers(0, slots, n), r.integers(0, n_kv, n), r.integers(0, 64, n)
        for got, want in zip(orc.cache_indices(b, slot, g, i, slots, n_kv * 64),
                             ref.cache_indices(b, slot, g, i, slots, n_kv * 64)):
            assert np.array_equal(got, want)
    bits = r.integers(0, 2**32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    assert np.array_equal(orc.f32_to_bf16(bits), ref.f32_to_bf16(bits))
    assert np.array_equal(orc.f32_to_bf16(gi.case_bf16_rounding()), ref.f32_to_bf16(gi.case_bf16_rounding()))


def _assert_same_wave(got, want):
    for g, w, what in zip(got, want, ("rows", "generated", "steps run", "done", "fed", "mask")):
        assert np.array_equal(np.asarray(g), np.asarray(w)), what


def test_golden_value_codes_and_wave(orc, golden):
    codes, scales = orc.value_codes(gi.case_value_heads())
    assert np.array_equal(codes, golden["value_codes"])
    assert_bit_equal(scales, golden["value_scales"], "value scales")
    for j, (prompts, picked, steps) in enumerate(gi.case_wave()):
        rows, total, ran, done, fed, mask = orc.wave_bookkeeping(prompts, picked, steps)
        assert np.array_equal(rows, golden[f"wave{j}_rows"]), j
        assert [total, ran] == list(golden[f"wave{j}_counts"]), j
        assert np.array_equal(done, golden[f"wave{j}_done"]) and np.array_equal(fed, golden[f"wave{j}_fed"]), j
        assert np.array_equal(mask, golden[f"wave{j}_mask"]), j


def test_ref_value_codes_of_the_cache(orc, ref):
    """The int8 value rule against quantize_v of the reference's attention test
    (tests/attn_test.cpp:218-226), bit for bit: random heads over 30 orders of magnitude, the
    committed corner heads, heads made of exact halves at random power-of-two scales."""
    if not ref.has_value_codes:
        pytest.skip("reference library built without tests/attn_test.cpp")
    r = np.random.default_rng(17)
    v = r.standard_normal((20000, 64)).astype(np.float32) * np.float32(10.0) ** r.integers(-15, 15, (20000, 1)).astype(np.float32)
    v[::7] = np.round(v[::7] * 4) / 4
    for heads in (v, gi.case_value_heads()):
        (c0, s0), (c1, s1) = orc.value_codes(heads), ref.value_codes(heads)
        assert np.array_equal(c0, c1)
        assert_bit_equal(s0, s1, "scales")
    k = r.integers(-126, 127, (4000, 64)).astype(np.float32) + np.float32(0.5)
    k[:, 0] = 127.0
    k = (k * np.float32(2.0) ** r.integers(-60, 60, (4000, 1)).astype(np.float32)).astype(np.float32)
    (c0, s0), (c1, s1) = orc.value_codes(k), ref.value_codes(k)
    assert np.array_equal(c0, c1) and np.array_equal(s0.view(np.uint32), s1.view(np.uint32))
    assert (np.abs(c0.astype(np.int32)) % 2 == 0)[:, 1:].all(), "halves go to the even neighbour"


def test_ref_wave_bookkeeping(orc, ref):
    """The wave bookkeeping, restated row by row, against the reference's own statements
    (engine/gpu_engine.hpp:696-701, 802-838) driven with recorded picks: output rows, the
    generated-token count, steps run, the finished mask, and per step the tokens fed and the
    mask the device held."""
    if not ref.has_wave:
        pytest.skip("reference library built without engine/gpu_engine.hpp")
    for prompts, picked, steps in gi.case_wave():
        _assert_same_wave(orc.wave_bookkeeping(prompts, picked, steps), ref.wave_bookkeeping(prompts, picked, steps))
    r = np.random.default_rng(23)
    for trial in range(300):
        n, steps = int(r.integers(1, 40)), int(r.integers(0, 30))
        prompts = [list(r.integers(0, 199000, int(r.integers(1, 12)))) for _ in range(n)]
        picked = r.integers(0, 199000, (steps, n)).astype(np.int32)
        ends = r.random((steps, n)) < (0.0, 0.05, 0.3)[trial % 3]
        picked[ends] = np.where(r.random(int(ends.sum())) < 0.5, 199999, 200002)
        for b in range(n):
            if r.random() < 0.1:
                prompts[b][int(r.integers(0, len(prompts[b])))] = 199999
        _assert_same_wave(orc.wave_bookkeeping(prompts, picked, steps), ref.wave_bookkeeping(prompts, picked, steps))


def _group_of_a_range(full, e, e_begin, e_count):
    """What grouping for experts e_begin .. e_begin+e_count-1 alone must give, derived from a
    grouping over all experts: that range's rows, renumbered from zero, and -1 for every pair
    whose expert lies outside it (kernels/moe_ep.hpp:44-49, :118-127)."""
    off, rp, pr = full
    lo, hi = off[e_begin], off[e_begin + e_count]
    inside = (e.ravel() >= e_begin) & (e.ravel() < e_begin + e_count)
    return off[e_begin:e_begin + e_count + 1] - lo, rp[lo:hi], np.where(inside, pr - lo, -1).astype(np.int32)


def test_golden_group_and_gather(orc, golden):
    for j, (e, E) in enumerate(gi.case_group()):
        counts, off, rp, own = orc.moe_group(e, 0, E)
        assert np.array_equal(off, golden[f"group{j}_offsets"]), j
        assert np.array_equal(rp, golden[f"group{j}_row_pair"]), j
        assert np.array_equal(own, golden[f"group{j}_pair_row"]), j
        assert np.array_equal(counts, np.diff(off)), j
        full = (golden[f"group{j}_offsets"], golden[f"group{j}_row_pair"], golden[f"group{j}_pair_row"])
        for i, (e_begin, e_count) in enumerate(gi.group_ranges(E)):
            c2, off2, rp2, own2 = orc.moe_group(e, e_begin, e_count)
            w_off, w_rp, w_own = _group_of_a_range(full, e, e_begin, e_count)
            assert np.array_equal(off2, w_off) and np.array_equal(rp2, w_rp) and np.array_equal(own2, w_own), (j, e_begin)
            if j < 2:   # the reference's own kernels for part of the experts
                for got, name in ((c2, "counts"), (off2, "offsets"), (rp2, "row_pair"), (own2, "own_row")):
                    assert np.array_equal(got, golden[f"group{j}_part{i}_{name}"]), (j, i, name)
    e, E = gi.case_group()[0]
    rows = orc.moe_gather(gi.uniform(610, (e.shape[0], 64)), golden["group0_row_pair"], e.shape[1])
    assert_bit_equal(rows, golden["group0_rows"], "gathered rows")


def test_ref_group_and_gather(orc, ref):
    """The grouping step against the reference's moe_group_kernel and the row gather against its
    moe_gather_kernel (kernels/moe.hpp:142-171, 175-182), whose bodies the reference library
    runs on host threads (one per GPU thread, a barrier for __syncthreads): offsets, the pair in
    each row and the row of each pair, bit for bit; pairs of finished tokens keep the caller's
    -1.  A grouping for part of the experts is held to the same run, restricted to that range."""
    if not ref.has_group:
        pytest.skip("reference library built without kernels/moe.hpp")
    r = np.random.default_rng(29)
    cases = list(gi.case_group())
    for trial in range(40):
        E, k = ((32, 4), (128, 4), (16, 8), (1024, 4), (7, 2))[trial % 5]
        T = int(r.integers(1, 400)) if E < 1024 else 33
        e = np.stack([r.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        if trial % 2:
            e[r.random(T) < 0.2] = -1
        if trial % 7 == 3:
            e[:] = e[0]   # every token picks the same experts
        cases.append((e, E))
    for e, E in cases:
        full = ref.moe_group(e, E)
        counts, off, rp, own = orc.moe_group(e, 0, E)
        assert np.array_equal(off, full[0]) and np.array_equal(rp, full[1]) and np.array_equal(own, full[2])
        if E >= 8:
            for e_begin, e_count in ((0, E // 2), (E // 2, E - E // 2), (3, 4)):
                got = orc.moe_group(e, e_begin, e_count)[1:]
                for g, w in zip(got, _group_of_a_range(full, e, e_begin, e_count)):
                    assert np.array_equal(g, w)
        H = 24
        t = r.standard_normal((e.shape[0], H)).astype(np.float32)
        assert_bit_equal(orc.moe_gather(t, full[1], e.shape[1]), ref.moe_gather(t, full[1], e.shape[1]), "rows")


def _with_done_and_slots(w, e, done, slot_of):
    """What finished rows and a renumbering table do to a router result (kernels/moe.hpp:60-63): a
    finished row gets expert -1 and weight 0 for every choice; the others the table's number for
    each chosen expert, the choice and the weights unchanged."""
    live = (np.asarray(done) == 0)[:, None]
    return np.where(live, w, np.float32(0)).astype(np.float32), np.where(live, np.asarray(slot_of)[e], -1).astype(np.int32)


def test_golden_router_finished_rows_and_slots(orc, golden):
    for sc, tag in zip(gi.case_router(), ("router20", "router120")):
        done, slot_of = gi.router_done_and_slots(*sc.shape)
        w, e = _with_done_and_slots(*orc.router_rows(sc, 4), done, slot_of)
        assert np.array_equal(e, golden[tag + "_wave_e"])
        assert_bit_equal(w, golden[tag + "_wave_w"], tag)


def test_ref_router_wave_kernel(orc, ref):
    """The router the engine launches, router_topk_wave_kernel (kernels/moe.hpp:64-136, with
    expf_cpu of kernels/exact_math.hpp), run on host threads with a 64-wide wave's shuffles
    emulated: experts and weights equal the oracle's (that is, topk() + softmax() of run.cpp) bit
    for bit, planted ties included, and finished rows and the renumbering table act as the GPU
    tests assume."""
    if not ref.has_router_wave:
        pytest.skip("reference library built without kernels/moe.hpp's router")
    r = np.random.default_rng(41)
    for E, k, B in ((32, 4, 41), (128, 4, 22), (200, 2, 9), (16, 8, 6), (256, 8, 5)):
        s = r.standard_normal((B, E)).astype(np.float32)
        s[::3, E - 1] = s[::3, 2]
        s[::5] = np.trunc(s[::5] * 2)
        s[1, 1], s[1, E // 2] = 0.0, -0.0
        w, e = orc.router_rows(s, k)
        w_ref, e_ref = ref.router_topk_wave(s, k)
        assert np.array_equal(e, e_ref), (E, k)
        assert_bit_equal(w, w_ref, "weights")
        done = (r.random(B) < 0.3).astype(np.int32)
        slot_of = r.permutation(E).astype(np.int32)
        w_ref, e_ref = ref.router_topk_wave(s, k, done, slot_of)
        w_want, e_want = _with_done_and_slots(w, e, done, slot_of)
        assert np.array_equal(e_want, e_ref), (E, k)
        assert_bit_equal(w_want, w_ref, "weights of live rows, zeros of finished ones")


def test_golden_contracted_rotation_and_combine(orc, golden):
    qkv, bias, pos = gi.case_rope()
    ct, st = orc.yarn_table(4096)
    assert_bit_equal(orc.bias_rope_rows_table(qkv, bias, pos, ct, st, fma=True), golden["rope_fma_out"], "rope, fma")
    xc, Z, row_of, wt, e = gi.case_combine()
    assert_bit_equal(orc.combine_rows_fma(xc, Z, row_of, wt, e), golden["combine_fma_x"], "combine, fma")
    assert not np.array_equal(golden["rope_fma_out"], golden["rope_out"]), "the two flavours differ somewhere"


def test_ref_exact_kernels_pin_the_contracted_forms(orc, ref):
    """The fused-multiply-add flavour of the rotation and of the combine (GPTOSS_EXACT | GPTOSS_FMA)
    against the reference's GPU exact kernels rope_exact (kernels/misc.hpp:55-70) and
    moe_combine_exact (kernels/moe.hpp:210-236), whose bodies -- plain C per thread, every rounding
    step named -- the reference library runs on the host: bit for bit."""
    if not ref.has_exact_kernels:
        pytest.skip("reference library built without its exact kernels, or with contraction on")
    r = np.random.default_rng(37)
    for nq, nkv, hd in ((64, 8, 64), (5, 2, 32), (1, 1, 128)):
        B, row = 7, (nq + 2 * nkv) * hd
        rows = (r.standard_normal((B, row)) * 10.0 ** r.integers(-3, 4, (B, 1))).astype(np.float32)
        if hd == 64:
            c, s_ = orc.yarn_table(128)
        else:  # any table will do for the rounding sequence
            c, s_ = (r.uniform(-1.4, 1.4, (128, hd // 2)).astype(np.float32) for _ in range(2))
        for p in (0, 1, 77):
            want = ref.rope_exact(rows, c[p], s_[p], nq + nkv, hd)
            got = orc.bias_rope_rows_table(rows, None, np.full(B, p, np.int32), c, s_, nq, nkv, hd, fma=True)
            assert_bit_equal(got, want, f"rope {nq}/{nkv}/{hd} at {p}")
    for T, k, Hd, E in ((33, 4, 2880, 32), (9, 8, 100, 16), (5, 1, 64, 4), (12, 4, 77, 128)):
        x = r.standard_normal((T, Hd)).astype(np.float32)
        Z = (r.standard_normal((T * k, Hd)) * 3).astype(np.float32)
        w = r.random((T, k)).astype(np.float32)
        e = np.stack([r.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        row_of = r.permutation(T * k).astype(np.int32).reshape(T, k)
        assert_bit_equal(orc.combine_rows_fma(x, Z, row_of, w, e), ref.moe_combine_exact(x, Z, row_of, w, e), "combine")


def _rope_kv_of_the_oracle(orc, rows, ct, st, p, nq, nkv, slots, slot, rotate_q=True):
    """Rotation (contracted form) then cache write, as two oracle calls; the rows come back as
    the reference's kernel leaves them: rotated queries, keys and values untouched."""
    B, kv = rows.shape[0], nkv * 64
    rotated = orc.bias_rope_rows_table(rows, None, np.full(B, p, np.int32), ct, st, nq, nkv, 64, fma=True)
    kc, vq, vs = np.zeros(B * slots * kv, np.uint16), np.zeros(B * slots * kv, np.int8), np.zeros(B * slots * nkv, np.float32)
    orc.kv_cache_write(rotated, nq, nkv, kc, vq, vs, slots, np.full(B, slot, np.int32))
    after = rows.copy()
    if rotate_q:
        after[:, :nq * 64] = rotated[:, :nq * 64]
    return after, kc, vq, vs


def test_golden_rope_kv(orc, golden):
    rows, p, slots, slot = gi.case_rope_kv()
    ct, st = orc.yarn_table(64)
    after, kc, vq, vs = _rope_kv_of_the_oracle(orc, rows, ct, st, p, 64, 8, slots, slot)
    assert_bit_equal(after, golden["rope_kv_rows"], "rows")
    assert np.array_equal(kc, golden["rope_kv_keys"]) and np.array_equal(vq, golden["rope_kv_codes"])
    assert_bit_equal(vs, golden["rope_kv_scales"], "scales")


def test_ref_rope_kv_kernel(orc, ref):
    """The engine's rotation + KV-cache write in one launch, rope_kv_bf16_kernel
    (kernels/fast_misc.hpp:48-108, instantiated as its launcher does at :110-127), run on host
    threads: rotated queries, bf16 keys, int8 value codes, scales and where each lands equal the
    oracle's contracted rotation followed by its cache write, bit for bit -- with the queries
    rotated or left to the attention, for both models' head counts and the kernel's widest case."""
    if not ref.has_rope_kv:
        pytest.skip("reference library built without kernels/fast_misc.hpp's rope_kv_bf16_kernel")
    r = np.random.default_rng(43)
    ct, st = orc.yarn_table(300)
    for nq, nkv, rotate_q, slots, slot in ((64, 8, True, 128, 77), (64, 8, False, 64, 63), (5, 2, True, 64, 0),
                                           (100, 16, True, 128, 16)):
        B, row = 4, (nq + 2 * nkv) * 64
        rows = (r.standard_normal((B, row)) * 10.0 ** r.integers(-2, 3, (B, 1))).astype(np.float32)
        rows[1, (nq + nkv) * 64:(nq + nkv) * 64 + 64] = 0.0
        p = int(r.integers(0, 300))
        kv = nkv * 64
        kc, vq, vs = np.zeros(B * slots * kv, np.uint16), np.zeros(B * slots * kv, np.int8), np.zeros(B * slots * nkv, np.float32)
        after = ref.rope_kv_bf16(rows, ct[p], st[p], nq, nkv, kc, vq, vs, slots, slot, rotate_q)
        w_after, w_kc, w_vq, w_vs = _rope_kv_of_the_oracle(orc, rows, ct, st, p, nq, nkv, slots, slot, rotate_q)
        assert_bit_equal(after, w_after, "rows")
        assert np.array_equal(kc, w_kc) and np.array_equal(vq, w_vq), (nq, nkv)
        assert_bit_equal(vs, w_vs, "scales")


def test_ref_exact_gpu_kernels_agree_with_the_oracle(orc, ref):
    """The rest of the GPU engine's bit-exact path -- embed_kernel, add_inplace_kernel, argmax_kernel
    (kernels/misc.hpp), router_topk_exact and swiglu_exact (kernels/moe.hpp) -- bodies run on the
    host, against the oracle (which is run.cpp's arithmetic): bit for bit.  One corner differs by
    the reference's own choice and is held as such: a NaN in a row's first logit makes
    sample_argmax answer 0, while argmax_kernel skips it like any other NaN."""
    if not ref.has_exact_rows:
        pytest.skip("reference library built without the exact kernels of kernels/misc.hpp and kernels/moe.hpp")
    r = np.random.default_rng(53)
    table = r.integers(0, 2 ** 16, (300, 96), dtype=np.uint16)
    ids = r.integers(0, 300, 41).astype(np.int32)
    want = (table[ids].astype(np.uint32) << 16).view(np.float32)
    assert_bit_equal(ref.exact_rows("embed", table, ids), want, "embedding rows")
    x, y = (r.standard_normal(1000) * 10.0 ** r.integers(-5, 6, 1000)).astype(np.float32), r.standard_normal(1000).astype(np.float32)
    assert_bit_equal(ref.exact_rows("add", x, y), (x + y).astype(np.float32), "residual add")
    for E, k in ((32, 4), (128, 4), (200, 2), (16, 8)):
        lg = r.standard_normal((37, E)).astype(np.float32)
        lg[::3, E - 1] = lg[::3, 2]
        lg[::5] = np.trunc(lg[::5] * 2)
        w, e = ref.exact_rows("router", lg, k)
        w2, e2 = orc.router_rows(lg, k)
        assert np.array_equal(e, e2), (E, k)
        assert_bit_equal(w, w2, "router weights")
    yy = (r.standard_normal((9, 2 * 333)) * np.float32(4)).astype(np.float32)
    yy[0, :8] = 100.0, -100.0, 7.0, -7.0, -60.0, 3.0, 0.0, -0.0
    assert_bit_equal(ref.exact_rows("swiglu", yy, 7.0), orc.swiglu_rows(yy), "SwiGLU")
    lg = np.trunc(r.standard_normal((6, 5001)) * 3).astype(np.float32)   # many equal maxima: the first one wins
    lg[2, :] = -np.inf
    lg[3, 17] = np.nan
    lg[4, 4000] = lg[4].max() + 1
    assert np.array_equal(ref.exact_rows("argmax", lg), orc.argmax_rows(lg))
    lg[5, 0] = np.nan
    assert orc.argmax_rows(lg)[5] == 0 and ref.exact_rows("argmax", lg)[5] == int(np.nanargmax(lg[5]))


def test_ref_fast_kernels_sit_inside_the_bf16_tolerance(orc, ref, golden):
    """The reference's fast-path kernels (rmsnorm_bf16_kernel, swiglu_bf16_kernel,
    moe_combine_kernel, kernels/fast_misc.hpp), run on the host, against the fp32 oracle: they
    differ by the bf16 rounding of their outputs and their own summation order, inside the 2e-2
    that the bf16 mode is held to.  Their outputs on the committed inputs are golden vectors for
    the GPU's bf16 mode."""
    if not ref.has_fast_kernels:
        pytest.skip("reference library built without kernels/fast_misc.hpp's fast-path kernels")
    widen = lambda bits: (np.asarray(bits, np.uint32) << 16).view(np.float32)
    rel = lambda got, want: float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 0.01 * np.sqrt(np.mean(want * want)))))
    x, delta, gain = gi.case_rmsnorm()
    bits = ref.rmsnorm_bf16((x + delta).astype(np.float32), gain)
    assert np.array_equal(bits, golden["fast_norm_bits"])
    assert rel(widen(bits), orc.add_rmsnorm_rows(x, delta, gain)[1]) <= 2e-2
    y = gi.case_swiglu()
    bits = ref.swiglu_bf16(y)
    assert np.array_equal(bits, golden["fast_swiglu_bits"])
    assert rel(widen(bits), orc.swiglu_rows(y)) <= 2e-2
    xc, Z, row_of, wt, e = gi.case_combine()
    got = ref.moe_combine_fast(xc, Z, row_of, wt)
    assert_bit_equal(got, golden["fast_combine_x"], "fast combine")
    assert rel(got, orc.combine_rows(xc, Z, row_of, wt, e, gi.E20)) <= 1e-5


def test_ref_fused_fast_kernels_give_their_unfused_pairs_bits(ref, golden):
    """add_rmsnorm_bf16_kernel (kernels/fast_misc.hpp:237-256) and moe_combine_rmsnorm_kernel
    (kernels/moe_ep.hpp:479-515), run on host threads (a block barrier, then shuffles inside each
    64-wide wave, for the row sum): the reference says each equals its unfused pair bit for bit,
    and run here they do -- which also checks the emulated shuffles.  A finished token keeps its
    x and still gets its norm."""
    if not (ref.has_fused_kernels and ref.has_fast_kernels):
        pytest.skip("reference library built without the fast path's fused kernels")
    x, delta, gain = gi.case_rmsnorm()
    xa, bits = ref.add_rmsnorm_bf16(x, delta, gain)
    assert_bit_equal(xa, (x + delta).astype(np.float32), "x + delta")
    assert np.array_equal(bits, ref.rmsnorm_bf16(xa, gain)) and np.array_equal(bits, golden["fast_norm_bits"])
    xc, Z, row_of, wt, e, gain = gi.case_combine_norm()
    x2, bits2 = ref.moe_combine_rmsnorm(xc, Z, row_of, wt, e, gain)
    unfused = ref.moe_combine_fast(xc, Z, row_of, wt)
    unfused[2] = xc[2]
    assert_bit_equal(x2, unfused, "combine")
    assert np.array_equal(bits2, ref.rmsnorm_bf16(x2, gain))
    assert_bit_equal(x2, golden["fast_combine_norm_x"], "golden x")
    assert np.array_equal(bits2, golden["fast_combine_norm_bits"])
    r = np.random.default_rng(59)   # an odd width takes the launchers' general instantiations
    xo, yo, go = (r.standard_normal((3, 1000)).astype(np.float32) for _ in range(3))
    xa, bits = ref.add_rmsnorm_bf16(xo, yo, go[0])
    assert np.array_equal(bits, ref.rmsnorm_bf16(xa, go[0]))


def test_argmax_key_header_is_the_reference_key(ref, tmp_path):
    """include/gptoss_argmax_key.cuh, compiled for the host (tests/cpp/argmax_key_host.cpp), against
    the reference's argmax_key (kernels/fast_gemm.hpp:94-104): the same 64-bit word for every
    (value, column) -- random bit patterns, both zeros, infinities, NaNs, denormals, columns up to
    2^31 - 1 -- so a producer written against either folds into the same words; and the merged
    word names its column."""
    if not ref.has_argmax_key:
        pytest.skip("reference library built without kernels/fast_gemm.hpp's argmax_key")
    import ctypes as C
    import subprocess
    so = tmp_path / "argmax_key_host.so"
    subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"), "-x", "c++",
                    os.path.join(ROOT, "tests", "cpp", "argmax_key_host.cpp"), "-o", str(so)], check=True)
    host = C.CDLL(str(so))
    r = np.random.default_rng(47)
    x = r.integers(0, 2 ** 32, 400000, dtype=np.uint64).astype(np.uint32).view(np.float32).copy()
    x[:12] = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -np.nan, 1e-45, -1e-45, 3.4e38, -3.4e38, 1.0, -1.0], np.float32)
    col = r.integers(0, 2 ** 31, x.size).astype(np.int32)
    col[:4] = 0, 1, 2 ** 31 - 1, 201087
    got = np.empty(x.size, np.uint64)
    host.host_argmax_keys(C.c_long(x.size), x.ctypes.data_as(C.c_void_p), col.ctypes.data_as(C.c_void_p),
                          got.ctypes.data_as(C.c_void_p))
    assert np.array_equal(got, ref.argmax_keys(x, col))
    back = np.empty(x.size, np.int32)
    host.host_argmax_columns(C.c_long(x.size), got.ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p))
    number = ~np.isnan(x)
    assert np.array_equal(back[number], col[number]) and (got[~number] == 0).all() and (back[~number] == 0).all()


def test_ref_group_for_part_of_the_experts(orc, ref):
    """Grouping for experts e_begin .. e_begin + e_count - 1 against the reference's
    moe_count_ep_kernel + moe_place_ep_kernel (kernels/moe_ep.hpp:55-127; the pair moe_group_ep
    launches at :250-254) with no partner, run on host threads with a 64-wide wavefront's ballot
    and shuffle emulated: counts, offsets, the pair in each row, and the row of each pair with -1
    for every pair whose expert lies outside the range or whose token has finished."""
    if not ref.has_group_ep:
        pytest.skip("reference library built without kernels/moe_ep.hpp")
    r = np.random.default_rng(31)
    cases = [(gi.case_group()[0][0], 32, (0, 16)), (gi.case_group()[0][0], 32, (16, 16)),
             (gi.case_group()[1][0][:120], 128, (96, 32)), (gi.case_group()[4][0], 32, (8, 8))]
    for E, k, T, rng in ((32, 4, 333, (5, 3)), (32, 4, 1, (0, 32)), (16, 8, 70, (8, 8)), (128, 4, 90, (31, 33))):
        e = np.stack([r.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
        e[r.random(T) < 0.15] = -1
        cases.append((e, E, rng))
    for e, E, (e_begin, e_count) in cases:
        want = ref.moe_group_ep(e, e_begin, e_count)
        got = orc.moe_group(e, e_begin, e_count)
        for g, w, name in zip(got, want, ("counts", "offsets", "row_pair", "own_row")):
            assert np.array_equal(g, w), (name, E, e_begin, e_count)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_ref_forward_pins_the_inline_loops(orc, ref, seed):
    """forward() of a tiny model: bias adds, SwiGLU (with clamping hit by the large
    weights), the expert combine in increasing expert order and both residual adds only
    exist inside it."""
    m = gi.tiny_model()
    if seed == 2:
        m.update(window=0, top_k=2, n_experts=4)
    if seed == 3:
        m.update(n_layers=3, inter=80, hidden=96)
    cfg = oracle.OrcConfig(*m.values())
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(oracle.flat_weight_count(cfg)) * (0.2 if seed < 3 else 0.6)).astype(np.float32)
    toks = rng.integers(0, m["vocab"], 8).astype(np.int32)
    assert_bit_equal(orc.forward_seq(cfg, w, toks), ref.forward_seq(cfg, w, toks), "logits")
