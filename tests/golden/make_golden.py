"""Regenerates tests/golden/golden.npz.

Run where the reference checkout is available (it builds oracle/_ref/libgptoss_ref.so
from the reference's own run.cpp and calls the reference's functions):

    python tests/golden/make_golden.py

Inputs come from golden_inputs.py (integer hashing, reproducible anywhere); the file
stores the expected outputs:

  * rmsnorm / add, rope (bias + per-token YaRN cos/sin + rotation), router top-4 + softmax,
    argmax, YaRN anchors: produced by the REFERENCE's compiled functions;
  * logits of a tiny 2-layer model over 10 decode steps: the REFERENCE's forward(), which
    is what pins the loops that only exist inline in it (bias add, SwiGLU, expert combine,
    residual);
  * the chunk64 KV-cache index functions and the fp32 -> bf16 rounding rule: the REFERENCE's
    host-callable definitions in its kernel headers;
  * the int8 codes and scales of value heads: the REFERENCE's quantize_v (tests/attn_test.cpp);
  * the wave bookkeeping (output rows, counts, finished mask, tokens fed and mask seen per
    step): the REFERENCE's statements of gpu_run_wave (engine/gpu_engine.hpp) around recorded
    picks;
  * the grouping of pairs by expert (offsets, row of each pair, pair of each row) and the
    gathered rows: the REFERENCE's moe_group_kernel / moe_gather_kernel (kernels/moe.hpp), their
    bodies run on host threads; for part of the experts its moe_count_ep_kernel +
    moe_place_ep_kernel (kernels/moe_ep.hpp) the same way, 64 host threads to a wavefront;
  * rotated rows, bf16 keys, int8 value codes and scales of the engine's rotation + cache write: the
    REFERENCE's rope_kv_bf16_kernel (kernels/fast_misc.hpp), run on host threads;
  * the bf16 mode's norm, SwiGLU and combine as the REFERENCE's fast-path kernels compute them
    (rmsnorm_bf16_kernel, swiglu_bf16_kernel, moe_combine_kernel of kernels/fast_misc.hpp), run on the host;
  * the router's output for finished rows and with an expert renumbering table: the REFERENCE's
    router_topk_wave_kernel (kernels/moe.hpp), run on host threads;
  * the rotation and the combine with the GPU exact path's rounding (fused multiply-adds): the
    REFERENCE's rope_exact (kernels/misc.hpp) and moe_combine_exact (kernels/moe.hpp), run on the host;
  * SwiGLU rows and combine rows: produced by the restated oracle (the reference has no
    callable form of those loops); they are regression vectors for the oracle, whose
    agreement with forward() is checked separately.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import golden_inputs as gi  # noqa: E402
import oracle  # noqa: E402


def main():
    oracle.build(ref=True)
    ref, orc = oracle.Reference(), oracle.Oracle()
    out = {}

    x, delta, gain = gi.case_rmsnorm()
    xa, normed = ref.add_rmsnorm_rows(x, delta, gain)
    out["rmsnorm_x"], out["rmsnorm_out"] = xa, normed
    out["rmsnorm_only"] = ref.add_rmsnorm_rows(x, None, gain)[1]

    qkv, bias, pos = gi.case_rope()
    out["rope_out"] = ref.bias_rope_rows(qkv, bias, pos)
    conc, inv = ref.yarn_inv_freq()
    out["yarn_conc"], out["yarn_inv_freq"] = np.float32(conc), inv
    cs = [ref.yarn_cos_sin(int(p)) for p in pos]
    out["yarn_cos"] = np.stack([c for c, _ in cs])
    out["yarn_sin"] = np.stack([s for _, s in cs])

    a, b = gi.case_router()
    out["router20_w"], out["router20_e"] = ref.router_rows(a)
    out["router120_w"], out["router120_e"] = ref.router_rows(b)

    # finished rows and renumbered experts: the REFERENCE's router_topk_wave_kernel (kernels/moe.hpp), the router
    # its engine launches, run on host threads (64 to a wave)
    for sc, tag in ((a, "router20"), (b, "router120")):
        done, slot_of = gi.router_done_and_slots(*sc.shape)
        out[tag + "_wave_w"], out[tag + "_wave_e"] = ref.router_topk_wave(sc, 4, done, slot_of)

    out["argmax"] = ref.argmax_rows(gi.case_argmax())

    m = gi.tiny_model()
    cfg = oracle.OrcConfig(*m.values())
    w = gi.uniform(71, (oracle.flat_weight_count(cfg),), 0.35)
    toks = gi.small_ints(72, (10,), 0, m["vocab"])
    out["forward_logits"] = ref.forward_seq(cfg, w, toks)

    out["swiglu_out"] = orc.swiglu_rows(gi.case_swiglu())
    xc, Z, row_of, wt, e = gi.case_combine()
    out["combine_x"] = orc.combine_rows(xc, Z, row_of, wt, e, gi.E20)

    # the KV-cache layout and the bf16 rounding rule: host-callable functions of the
    # reference's kernel headers (kernels/fast_attention.hpp, kernels/fast_common.hpp)
    b, slot, g, i, slots, kv_dim = gi.case_cache_layout()
    k_at, vq_at, vs_at = ref.cache_indices(b, slot, g, i, slots, kv_dim)
    out["cache_k_at"], out["cache_vq_at"], out["cache_vs_at"] = (a.astype(np.int32) for a in (k_at, vq_at, vs_at))
    out["bf16_bits"] = ref.f32_to_bf16(gi.case_bf16_rounding())

    out["value_codes"], out["value_scales"] = ref.value_codes(gi.case_value_heads())
    for j, (prompts, picked, steps) in enumerate(gi.case_wave()):
        rows, total, ran, done, fed, mask = ref.wave_bookkeeping(prompts, picked, steps)
        out[f"wave{j}_rows"], out[f"wave{j}_counts"] = rows, np.array([total, ran], np.int64)
        out[f"wave{j}_done"], out[f"wave{j}_fed"], out[f"wave{j}_mask"] = done, fed, mask.astype(np.int8)

    # the contracted (fused multiply-add) flavour of the rotation and the combine: the REFERENCE's GPU
    # exact kernels rope_exact (kernels/misc.hpp) and moe_combine_exact (kernels/moe.hpp), bodies run on the host
    qkv, bias, pos = gi.case_rope()
    biased = (qkv + bias).astype(np.float32)
    out["rope_fma_out"] = np.concatenate([ref.rope_exact(biased[t:t + 1], *ref.yarn_cos_sin(int(pos[t])), 64 + 8, 64)
                                          for t in range(len(pos))])
    xc, Z, row_of, wt, e = gi.case_combine()
    out["combine_fma_x"] = ref.moe_combine_exact(xc, Z, row_of, wt, e)

    # the engine's rotation + KV-cache write in one launch: the REFERENCE's rope_kv_bf16_kernel
    # (kernels/fast_misc.hpp), run on host threads
    rows, p_, slots, slot = gi.case_rope_kv()
    n_k = rows.shape[0] * slots * 512
    kc, vq, vs = np.zeros(n_k, np.uint16), np.zeros(n_k, np.int8), np.zeros(n_k // 64, np.float32)
    out["rope_kv_rows"] = ref.rope_kv_bf16(rows, *ref.yarn_cos_sin(p_), 64, 8, kc, vq, vs, slots, slot)
    out["rope_kv_keys"], out["rope_kv_codes"], out["rope_kv_scales"] = kc, vq, vs

    # the fast (bf16-activation) path's own answers: the REFERENCE's rmsnorm_bf16_kernel (behind the float
    # add of add_inplace_kernel), swiglu_bf16_kernel and moe_combine_kernel (kernels/fast_misc.hpp), bodies
    # run on the host; the device's approximate __expf is the C library's expf here
    x, delta, gain = gi.case_rmsnorm()
    out["fast_norm_bits"] = ref.rmsnorm_bf16((x + delta).astype(np.float32), gain)
    out["fast_swiglu_bits"] = ref.swiglu_bf16(gi.case_swiglu())
    xc, Z, row_of, wt, e = gi.case_combine()
    out["fast_combine_x"] = ref.moe_combine_fast(xc, Z, row_of, wt)

    # the fast path's fused combine + next norm: the REFERENCE's moe_combine_rmsnorm_kernel (kernels/moe_ep.hpp)
    out["fast_combine_norm_x"], out["fast_combine_norm_bits"] = ref.moe_combine_rmsnorm(*gi.case_combine_norm())

    for j, (e, E) in enumerate(gi.case_group()):
        off, rp, pr = ref.moe_group(e, E)
        out[f"group{j}_offsets"], out[f"group{j}_row_pair"], out[f"group{j}_pair_row"] = off, rp, pr
        if j == 0:
            out["group0_rows"] = ref.moe_gather(gi.uniform(610, (e.shape[0], 64)), rp, e.shape[1])
        if j < 2:   # for part of the experts: moe_count_ep_kernel + moe_place_ep_kernel, no partner
            for i, (e_begin, e_count) in enumerate(gi.group_ranges(E)):
                c, o, rp2, own = ref.moe_group_ep(e, e_begin, e_count)
                out[f"group{j}_part{i}_counts"], out[f"group{j}_part{i}_offsets"] = c, o
                out[f"group{j}_part{i}_row_pair"], out[f"group{j}_part{i}_own_row"] = rp2, own

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes;", ", ".join(f"{k}{list(np.shape(v))}" for k, v in out.items()))


if __name__ == "__main__":
    main()
