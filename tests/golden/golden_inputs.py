"""Inputs of the golden known-answer cases.

Every input is derived from integer hashing and IEEE division only, so the same bits
come out on any machine and numpy version; the fixture files then only need to hold the
expected OUTPUTS, which ``make_golden.py`` obtained from the reference's own compiled
CPU functions.
"""
from __future__ import annotations

import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (x.astype(np.uint64) + np.uint64(0x9E3779B97F4A7C15)) & _M
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M
        return z ^ (z >> np.uint64(31))


def hashed(seed: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = splitmix64(np.array([seed], np.uint64))[0]
        return splitmix64(np.arange(n, dtype=np.uint64) * np.uint64(0xD1342543DE82EF95) + base)


def uniform(seed: int, shape, scale: float = 1.0, levels: int = 200001) -> np.ndarray:
    """fp32 values on a grid of `levels` points spanning [-scale, scale]."""
    n = int(np.prod(shape))
    h = hashed(seed, n) % np.uint64(levels)
    half = (levels - 1) // 2
    v = (h.astype(np.int64) - half).astype(np.float64) * (scale / half)
    return v.astype(np.float32).reshape(shape)


def small_ints(seed: int, shape, lo: int, hi: int) -> np.ndarray:
    n = int(np.prod(shape))
    return (lo + (hashed(seed, n) % np.uint64(hi - lo)).astype(np.int64)).astype(np.int32).reshape(shape)


def coarse(seed: int, shape, step: float = 0.125, span: int = 128) -> np.ndarray:
    """Multiples of `step` in [-span*step, span*step): few distinct values, so ties abound
    and every value is exact in bf16."""
    n = int(np.prod(shape))
    h = hashed(seed, n) % np.uint64(2 * span)
    return ((h.astype(np.int64) - span).astype(np.float32) * np.float32(step)).reshape(shape)


# ---- the cases --------------------------------------------------------------------

H, QKV, E20, E120, V = 2880, 5120, 32, 128, 201088


def case_rmsnorm():
    x = uniform(11, (4, H), 3.0)
    delta = uniform(12, (4, H), 1.0)
    gain = (1.0 + uniform(13, (H,), 0.3)).astype(np.float32)
    return x, delta, gain


def case_rope():
    qkv = uniform(21, (4, QKV), 2.0)
    bias = uniform(22, (QKV,), 0.05)
    pos = np.array([0, 37, 1023, 4095], np.int32)
    return qkv, bias, pos


def case_router():
    a = uniform(31, (48, E20), 2.0)
    b = uniform(32, (16, E120), 2.0)
    for s in (a, b):  # planted ties, signed zeros, many-equal rows
        T, E = s.shape
        for t in range(T):
            if t % 3 == 0:
                s[t, E - 1] = s[t, (7 * t) % (E - 1)]
            if t % 5 == 0:
                s[t, 1], s[t, E // 2] = 0.0, -0.0
                s[t, 0] = s[t, E - 2] = 50.0
            if t % 7 == 0:
                s[t] = np.trunc(s[t] * 2)
    return a, b


def case_swiglu():
    y = uniform(41, (4, 2 * H), 12.0)  # beyond the clamp at 7 on both sides
    y[0, :8] = [7.0, 7.0, -7.0, -7.0, 7.5, -7.5, 0.0, -0.0]
    return y


def case_combine():
    T, k = 6, 4
    x = uniform(51, (T, H), 2.0)
    Z = uniform(52, (T * k, H), 1.5)
    w = np.abs(uniform(53, (T, k), 1.0)) + np.float32(0.01)
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    e = np.stack([np.argsort(hashed(60 + t, E20))[:k] for t in range(T)]).astype(np.int32)
    row_of = np.argsort(hashed(54, T * k)).astype(np.int32).reshape(T, k)  # a permutation
    return x, Z, row_of, w, e


def case_argmax():
    lg = coarse(61, (3, V))
    lg[1, 777] = lg[1, 150000] = 99.0   # planted tie across far-apart columns
    lg[2, :] = 0.0                      # all equal: column 0
    lg[2, 5] = -0.0
    return lg


def tiny_model():
    """A 2-layer model small enough for the CPU forward pass (field order of run.cpp's Config)."""
    cfg = dict(vocab=97, hidden=64, n_experts=8, top_k=4, inter=48, n_layers=2, head_dim=64,
               n_q_heads=4, n_kv_heads=2, seq_len=16, orig_ctx=4096, theta=150000.0, factor=32.0,
               window=4, limit=7.0)
    return cfg


def case_cache_layout():
    """(b, slot, g, i) tuples for the KV-cache index functions: every slot of three chunks for
    a few (sequence, head, element) corners, plus hashed tuples; slots = 192, 8 heads of 64."""
    slots, kv_dim = 192, 512
    grid = [(b, s, g, i) for b in (0, 3) for s in range(slots) for g in (0, 7) for i in (0, 1, 5, 63)]
    n = 4000
    extra = np.stack([small_ints(81, (n,), 0, 6), small_ints(82, (n,), 0, slots), small_ints(83, (n,), 0, 8),
                      small_ints(84, (n,), 0, 64)], axis=1)
    t = np.concatenate([np.array(grid, np.int32), extra.astype(np.int32)])
    return t[:, 0].copy(), t[:, 1].copy(), t[:, 2].copy(), t[:, 3].copy(), slots, kv_dim


def case_bf16_rounding():
    """fp32 bit patterns around every rounding case of fp32 -> bf16: ties (even and odd), just
    above and below a tie, carries into the exponent, the largest finite value, infinities,
    NaNs with and without payload in the kept bits, denormals, zeros."""
    hi = np.array([0x0000, 0x0001, 0x007F, 0x0080, 0x3F80, 0x3F81, 0x7F7E, 0x7F7F, 0x7F80, 0x7F81, 0x7FC0, 0x7FFF],
                  np.uint32)
    lo = np.array([0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF], np.uint32)
    bits = ((hi[:, None] << 16) | lo[None, :]).ravel()
    bits = np.concatenate([bits, bits | np.uint32(0x80000000), (hashed(85, 2000) & 0xFFFFFFFF).astype(np.uint32)])
    return bits.astype(np.uint32).view(np.float32)


def case_value_heads():
    """Value heads of 64 floats for the int8 rule of the KV cache: hashed heads at several
    magnitudes, a head of zeros, the maximum shared by +x and -x, a head whose scaled values
    are exact halves (round-half-to-even decides every code), one large value among tiny
    ones, all values equal, and a head whose maximum is denormal with no zero in it (the
    inverse overflows: every code saturates).  Every value is finite, and no head mixes a
    maximum below 127 / FLT_MAX with a zero: there v * inv is 0 * inf, and the reference's
    host form converts that NaN to int8, which C++ leaves undefined."""
    heads = [uniform(91 + j, (64,), sc) for j, sc in enumerate((1.0, 3.0, 0.02, 1000.0, 1e-6, 2.5, 7.0, 0.3))]
    heads.append(np.zeros(64, np.float32))
    h = uniform(101, (64,), 1.0)
    h[3], h[40] = 2.0, -2.0
    heads.append(h)
    halves = (np.arange(64, dtype=np.float32) - 32.0) + np.float32(0.5)   # -31.5 .. 31.5
    halves[0], halves[63] = 127.0, -127.0                                 # max 127: inv is exactly 1
    heads.append(halves)
    heads.append((halves * np.float32(2.0 ** -20)).astype(np.float32))    # the same, scaled by a power of two
    lone = np.full(64, 1e-4, np.float32)
    lone[17] = -5000.0
    heads.append(lone)
    heads.append(np.full(64, -0.75, np.float32))
    den = np.full(64, 1e-41, np.float32)
    den[::2] = -2e-41
    heads.append(den)
    heads.append(np.float32(3.0e38) * uniform(102, (64,), 1.0))
    return np.stack(heads).astype(np.float32)


def case_wave():
    """Scenarios (prompts, picked [steps, n], steps) for the wave bookkeeping: prompts of 1 to
    7 tokens, an end token inside a prompt, a prompt longer than the wave, rows that pick an
    end token at once, late or never, both end tokens, a wave that every row leaves early, a
    wave of one step and a wave of none."""
    EOS = (199999, 200002)
    out = []
    n, steps = 23, 9
    prompts = [list(small_ints(200 + b, (1 + b % 7,), 0, 199000)) for b in range(n)]
    prompts[3] = [11, 22, 200002, 33, 44]
    prompts[9] = list(small_ints(300, (steps + 6,), 0, 199000))
    prompts[12] = list(small_ints(301, (steps,), 0, 199000))
    picked = small_ints(302, (steps, n), 0, 199000)
    picked[:, 0] = EOS[0]
    picked[4:, 5] = EOS[1]
    picked[steps - 1, 7] = EOS[0]
    picked[2, 8] = EOS[0]     # while row 8 is still inside its prompt: not looked at
    picked[0, 14] = EOS[1]    # row 14 has a one-token prompt: finishes in the first pass
    out.append((prompts, picked, steps))
    n, steps = 10, 20         # everybody finishes by step 6: the wave stops there
    prompts = [list(small_ints(400 + b, (1 + b % 3,), 0, 199000)) for b in range(n)]
    picked = small_ints(401, (steps, n), 0, 199000)
    for b in range(n):
        picked[b % 6:, b] = EOS[b % 2]
    out.append((prompts, picked, steps))
    n = 5
    prompts = [list(small_ints(500 + b, (1 + b,), 0, 199000)) for b in range(n)]
    out.append((prompts, small_ints(501, (1, n), 0, 199000), 1))
    out.append((prompts, np.zeros((0, n), np.int32), 0))
    return out


def case_group():
    """Routings (topk_e [T, k], n_experts) for the grouping step: 32 and 128 experts with four
    distinct choices per token, finished tokens (all four -1) scattered and in a run, an expert
    nobody picks, an expert everybody picks, one token, and a batch with every token finished."""
    out = []
    for j, (T, E, k) in enumerate(((257, 32, 4), (300, 128, 4), (1, 32, 4), (64, 32, 2))):
        order = np.argsort(hashed(600 + j, T * E).reshape(T, E), axis=1, kind="stable").astype(np.int32)
        e = np.ascontiguousarray(order[:, :k])
        if T > 1:
            e[e == 5] = 6 + (np.nonzero(e == 5)[0] % 3 == 0) * 20   # expert 5 is never picked ...
            e[:, 0] = np.where((e[:, 1:] == 7).any(axis=1), e[:, 0], 7)  # ... and 7 by everybody
            e[::9] = -1
            e[40:52] = -1
        out.append((e, E))
    out.append((np.full((16, 4), -1, np.int32), 32))
    return out


def group_ranges(E):
    """(e_begin, e_count) of the groupings for part of the experts that the golden file holds."""
    return ((0, E // 2), (E // 2, E // 2), (5, 3), (E - 1, 1))


def router_done_and_slots(T, E):
    """The finished-row flags and the expert renumbering table of the golden router cases."""
    done = (np.arange(T) % 5 == 0).astype(np.int32)
    slot_of = ((np.arange(E) * 37 + 5) % E).astype(np.int32)
    return done, slot_of


def case_rope_kv():
    """The engine's rotation + KV-cache write call: rows [3, 5120] at one position, one cache slot."""
    rows = uniform(81, (3, QKV), 2.5)
    rows[1, (64 + 8) * 64:(64 + 8) * 64 + 64] = 0.0   # a value head of zeros
    return rows, 37, 64, 21   # rows, position, slots, slot


def case_combine_norm():
    """The combine case with token 2 finished (expert -1 for every choice) and the gain of the norm case:
    inputs of the fused combine + next norm."""
    x, Z, row_of, w, e = case_combine()
    e = e.copy()
    e[2] = -1
    return x, Z, row_of, w, e, case_rmsnorm()[2]
