"""ctypes bindings for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two libraries live here:

* ``libgptoss_oracle.so`` -- the restated CPU oracle (``gptoss_oracle.c``), built by
  ``make -C oracle oracle``.  Always available (gcc is the only requirement).
* ``_ref/libgptoss_ref.so`` -- the reference's own CPU functions compiled from its
  checkout (``make -C oracle ref``).  Only buildable where the reference checkout is
  present; the built file is carried along to machines that do not have it.

Only the test suite, the smoke check and the bench's CPU-baseline legs import this
package.  The shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libgptoss_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libgptoss_ref.so")
# where the reference project is checked out (only needed to build _ref/libgptoss_ref.so):
# GPTOSS_REFERENCE, or a directory named "reference" beside this repository
REFERENCE_CHECKOUT = os.environ.get("GPTOSS_REFERENCE") or os.path.abspath(
    os.path.join(_HERE, os.pardir, os.pardir, "reference"))

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_opt = C.c_void_p  # optional array arguments are passed as raw addresses


def build(ref: bool | None = None) -> None:
    """Compile the oracle, and the reference checker when its checkout is present."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    if ref is None:
        ref = os.path.exists(os.path.join(REFERENCE_CHECKOUT, "run.cpp"))
    if ref:
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={REFERENCE_CHECKOUT}"], check=True)


def _addr(a):
    return None if a is None else a.ctypes.data


class OrcConfig(C.Structure):
    """Byte image shared by the oracle's orc_config_t and the reference's Config."""

    _fields_ = [
        ("vocab", C.c_int), ("hidden", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int),
        ("inter", C.c_int), ("n_layers", C.c_int), ("head_dim", C.c_int), ("n_q_heads", C.c_int),
        ("n_kv_heads", C.c_int), ("seq_len", C.c_int), ("orig_ctx", C.c_int),
        ("theta", C.c_float), ("factor", C.c_float), ("window", C.c_int), ("limit", C.c_float),
    ]


def flat_weight_count(c: OrcConfig) -> int:
    """Number of floats memory_map_weights() walks over for this config."""
    qkv = (c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim
    L, H, E, I, V = c.n_layers, c.hidden, c.n_experts, c.inter, c.vocab
    return (2 * V * H + 2 * L * H + H + L * H * qkv + L * qkv + L * c.n_q_heads * c.head_dim * H
            + L * H + L * c.n_q_heads + L * H * E + L * E + L * E * 2 * I * H + L * E * 2 * I
            + L * E * H * I + L * E * H)


class _Lib:
    def __init__(self, path: str, prefix: str):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built (run `make -C oracle`)")
        self.lib = C.CDLL(path)
        self.p = prefix
        L = self.lib
        p = prefix

        def sig(name, res, *args):
            fn = getattr(L, p + name)
            fn.restype = res
            fn.argtypes = list(args)
            return fn

        self._rmsnorm = sig("rmsnorm", None, _f32p, _f32p, _f32p, C.c_int)
        self._softmax = sig("softmax", None, _f32p, C.c_int)
        self._topk = sig("topk", None if p == "ref_" else C.c_int, _f32p, _i32p, _f32p, C.c_int, C.c_int)
        self._inv_freq = sig("yarn_inv_freq", None, C.c_float, C.c_int, C.c_float, C.c_float,
                             C.c_float, C.c_float, C.POINTER(C.c_float), _f32p)
        self._cos_sin = sig("yarn_cos_sin", None, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                            C.c_float, C.c_float, _f32p, _f32p)
        self._rotate = sig("rotate_heads", None, _f32p, _f32p, _f32p, C.c_int, C.c_int)
        self._argmax = sig("argmax", C.c_int, _f32p, C.c_int)
        self._add_rmsnorm_rows = sig("add_rmsnorm_rows", None, _f32p, _opt, _f32p, _f32p, C.c_int,
                                     C.c_int, C.c_int)
        self._bias_rope_rows = sig("bias_rope_rows", None, _f32p, _opt, _i32p, C.c_int, C.c_int,
                                   C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_float,
                                   C.c_float, C.c_int)
        self._router_rows = sig("router_rows", None, _f32p, _i32p, _f32p, C.c_int, C.c_int, C.c_int,
                                C.c_int)
        self._argmax_rows = sig("argmax_rows", None, _i32p, _f32p, C.c_int, C.c_long, C.c_int)
        self._forward_seq = sig("forward_seq", C.c_int, C.c_void_p, _f32p, _i32p, C.c_int, _f32p)
        self._max_threads = sig("max_threads", C.c_int)
        # the KV-cache index functions and the bf16 rounding rule (the reference library has
        # them when it was built from a checkout that holds the kernels' headers)
        self.has_cache_layout = p == "orc_" or bool(sig("has_cache_layout", C.c_int)())
        if self.has_cache_layout:
            _i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
            _u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
            self._cache_indices = sig("cache_indices", None, C.c_long, _i32p, _i32p, _i32p, _i32p, C.c_int, C.c_int,
                                      _i64p, _i64p, _i64p)
            self._f32_to_bf16 = sig("f32_to_bf16", None, C.c_long, _f32p, _u16p)

        # the int8 value rule of the KV cache and the wave bookkeeping (reference library: when it
        # was built from a checkout that holds tests/attn_test.cpp and engine/gpu_engine.hpp)
        self.has_value_codes = p == "orc_" or (hasattr(L, "ref_has_value_codes") and bool(L.ref_has_value_codes()))
        if self.has_value_codes:
            _i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
            self._value_codes = sig("value_codes", None, C.c_long, _f32p, _i8p, _f32p)
        self.has_wave = p == "orc_" or (hasattr(L, "ref_has_wave") and bool(L.ref_has_wave()))
        if self.has_wave:
            self._wave = sig("wave_bookkeeping", C.c_longlong, C.c_int, _i32p, _i32p, C.c_int, _i32p, C.c_int,
                             _i32p, _i32p, C.POINTER(C.c_int), _i32p, _i32p)

    def value_codes(self, v):
        """int8 codes [n, 64] and scales [n] of n value heads of 64 floats."""
        v = np.ascontiguousarray(v, np.float32).reshape(-1, 64)
        codes, scales = np.empty(v.shape, np.int8), np.empty(v.shape[0], np.float32)
        self._value_codes(v.shape[0], v, codes, scales)
        return codes, scales

    def wave_bookkeeping(self, prompts, picked, steps):
        """A wave of len(prompts) requests served for at most `steps` steps, where step s picked
        token picked[s, b] for row b.  Returns (out_rows [n, steps + 2] with -1 wherever nothing
        was written, n_generated, steps_run, done [n], fed [steps_run, n], mask [steps_run, n])."""
        n = len(prompts)
        offsets = np.zeros(n + 1, np.int32)
        offsets[1:] = np.cumsum([len(p) for p in prompts])
        flat = np.ascontiguousarray(np.concatenate([np.asarray(p, np.int32) for p in prompts]) if n else [], np.int32)
        picked = np.ascontiguousarray(picked, np.int32).reshape(max(steps, 0), n)
        width = steps + 2
        out = np.full((n, width), -1, np.int32)
        done = np.zeros(n, np.int32)
        fed = np.full((max(steps, 1), n), -9, np.int32)
        mask = np.full((max(steps, 1), n), -9, np.int32)
        ran = C.c_int(0)
        total = self._wave(n, flat if flat.size else np.zeros(1, np.int32), offsets, steps,
                           picked if picked.size else np.zeros(1, np.int32), width, out, done, C.byref(ran), fed, mask)
        return out, int(total), int(ran.value), done, fed[:ran.value], mask[:ran.value]

    # -- single-row primitives ------------------------------------------------
    def max_threads(self) -> int:
        return int(self._max_threads())

    def cache_indices(self, b, slot, g, i, slots, kv_dim):
        """For tuples (b, slot, g, i): element offsets of the key element, the value code and
        the value scale in the chunk64 caches."""
        b, slot, g, i = (np.ascontiguousarray(a, np.int32) for a in (b, slot, g, i))
        k_at, vq_at, vs_at = (np.empty(b.size, np.int64) for _ in range(3))
        self._cache_indices(b.size, b, slot, g, i, slots, kv_dim, k_at, vq_at, vs_at)
        return k_at, vq_at, vs_at

    def f32_to_bf16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self._f32_to_bf16(x.size, x, out)
        return out

    def rmsnorm(self, x, gain):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self._rmsnorm(out, x, np.ascontiguousarray(gain, np.float32), x.size)
        return out

    def softmax(self, x):
        x = np.array(x, np.float32, copy=True)
        self._softmax(x, x.size)
        return x

    def topk(self, scores, k):
        scores = np.array(scores, np.float32, copy=True)
        v = np.empty(k, np.float32)
        i = np.empty(k, np.int32)
        self._topk(v, i, scores, scores.size, k)
        return v, i

    def yarn_inv_freq(self, theta=150000.0, head_dim=64, factor=32.0, orig_ctx=4096.0,
                      beta_fast=32.0, beta_slow=1.0):
        conc = C.c_float()
        inv = np.empty(head_dim // 2, np.float32)
        self._inv_freq(theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, C.byref(conc), inv)
        return float(conc.value), inv

    def yarn_cos_sin(self, pos, theta=150000.0, head_dim=64, factor=32.0, orig_ctx=4096.0,
                     beta_fast=32.0, beta_slow=1.0):
        c = np.empty(head_dim // 2, np.float32)
        s = np.empty(head_dim // 2, np.float32)
        self._cos_sin(pos, theta, head_dim, factor, orig_ctx, beta_fast, beta_slow, c, s)
        return c, s

    def rotate_heads(self, x, cos_row, sin_row, n_heads, head_dim):
        x = np.array(x, np.float32, copy=True)
        self._rotate(x, np.ascontiguousarray(cos_row, np.float32),
                     np.ascontiguousarray(sin_row, np.float32), n_heads, head_dim)
        return x

    def argmax(self, p):
        p = np.ascontiguousarray(p, np.float32)
        return int(self._argmax(p, p.size))

    # -- row-batched forms ------------------------------------------------------
    def add_rmsnorm_rows(self, x, delta, gain, threads=1, inplace_norm=False):
        """Returns (x_after_add, normed).  delta may be None (norm only)."""
        x = np.array(x, np.float32, copy=True)
        T, H = x.shape
        d = None if delta is None else np.ascontiguousarray(delta, np.float32)
        normed = x if inplace_norm else np.empty_like(x)
        self._add_rmsnorm_rows(x, _addr(d), np.ascontiguousarray(gain, np.float32), normed, T, H, threads)
        return x, normed

    def bias_rope_rows(self, qkv, bias, pos, n_q=64, n_kv=8, head_dim=64, theta=150000.0,
                       factor=32.0, orig_ctx=4096.0, beta_fast=32.0, beta_slow=1.0, threads=1):
        qkv = np.array(qkv, np.float32, copy=True)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        pos = np.ascontiguousarray(pos, np.int32)
        self._bias_rope_rows(qkv, _addr(b), pos, qkv.shape[0], n_q, n_kv, head_dim, theta, factor,
                             orig_ctx, beta_fast, beta_slow, threads)
        return qkv

    def router_rows(self, scores, k=4, threads=1):
        scores = np.array(scores, np.float32, copy=True)
        T, E = scores.shape
        w = np.empty((T, k), np.float32)
        e = np.empty((T, k), np.int32)
        self._router_rows(w, e, scores, T, E, k, threads)
        return w, e

    def argmax_rows(self, logits, threads=1):
        logits = np.ascontiguousarray(logits, np.float32)
        T, V = logits.shape
        out = np.empty(T, np.int32)
        self._argmax_rows(out, logits, T, V, threads)
        return out

    def forward_seq(self, cfg: OrcConfig, flat_weights, tokens):
        flat_weights = np.ascontiguousarray(flat_weights, np.float32)
        assert flat_weights.size == flat_weight_count(cfg)
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((tokens.size, cfg.vocab), np.float32)
        rc = self._forward_seq(C.addressof(cfg), flat_weights, tokens, tokens.size, out)
        assert rc == 0
        return out


class Oracle(_Lib):
    """The restated CPU oracle, plus the row loops that only it has."""

    def __init__(self):
        super().__init__(ORACLE_SO, "orc_")
        L = self.lib
        L.orc_embed_rows.restype = None
        L.orc_embed_rows.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int]
        L.orc_swiglu_rows.restype = None
        L.orc_swiglu_rows.argtypes = [_f32p, _f32p, C.c_long, C.c_int, C.c_float, C.c_int]
        L.orc_combine_rows.restype = None
        L.orc_combine_rows.argtypes = [_f32p, _f32p, _i32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int]
        L.orc_bias_rope_rows_table.restype = None
        L.orc_bias_rope_rows_table.argtypes = [_f32p, _opt, _i32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                               _f32p, _f32p, C.c_int]
        L.orc_bias_rope_rows_table_fma.restype = None
        L.orc_bias_rope_rows_table_fma.argtypes = L.orc_bias_rope_rows_table.argtypes
        L.orc_combine_rows_fma.restype = None
        L.orc_combine_rows_fma.argtypes = [_f32p, _f32p, _i32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_yarn_table.restype = None
        L.orc_yarn_table.argtypes = [_f32p, _f32p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                                     C.c_float, C.c_float, C.c_int]
        L.orc_moe_group.restype = None
        L.orc_moe_group.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, _i32p, _i32p, _i32p, _i32p]
        L.orc_moe_gather.restype = None
        L.orc_moe_gather.argtypes = [_f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int]
        L.orc_kv_cache_write.restype = None
        L.orc_kv_cache_write.argtypes = [_f32p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int, _i32p]
        L.orc_expf_array.restype = None
        L.orc_expf_array.argtypes = [_f32p, _f32p, C.c_long]

    def embed_rows(self, table, ids, threads=1):
        table = np.ascontiguousarray(table, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty((ids.size, table.shape[1]), np.float32)
        self.lib.orc_embed_rows(out, table, ids, ids.size, table.shape[1], threads)
        return out

    def swiglu_rows(self, gate_up, limit=7.0, threads=1):
        gate_up = np.ascontiguousarray(gate_up, np.float32)
        R, two_i = gate_up.shape
        out = np.empty((R, two_i // 2), np.float32)
        self.lib.orc_swiglu_rows(out, gate_up, R, two_i // 2, limit, threads)
        return out

    def combine_rows(self, x, Z, row_of, weights, experts, n_experts, threads=1):
        x = np.array(x, np.float32, copy=True)
        T, H = x.shape
        k = weights.shape[1]
        self.lib.orc_combine_rows(x, np.ascontiguousarray(Z, np.float32),
                                  np.ascontiguousarray(row_of, np.int32),
                                  np.ascontiguousarray(weights, np.float32),
                                  np.ascontiguousarray(experts, np.int32), T, k, H, n_experts, threads)
        return x

    def combine_rows_fma(self, x, Z, row_of, weights, experts, threads=1):
        """The combine with the GPU exact path's rounding: fused multiply-adds in increasing expert order."""
        x = np.array(x, np.float32, copy=True)
        T, H = x.shape
        k = weights.shape[1]
        self.lib.orc_combine_rows_fma(x, np.ascontiguousarray(Z, np.float32), np.ascontiguousarray(row_of, np.int32),
                                      np.ascontiguousarray(weights, np.float32),
                                      np.ascontiguousarray(experts, np.int32), T, k, H, threads)
        return x

    def bias_rope_rows_table(self, qkv, bias, pos, cos_tab, sin_tab, n_q=64, n_kv=8, head_dim=64,
                             threads=1, fma=False):
        qkv = np.array(qkv, np.float32, copy=True)
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        fn = self.lib.orc_bias_rope_rows_table_fma if fma else self.lib.orc_bias_rope_rows_table
        fn(qkv, _addr(b), np.ascontiguousarray(pos, np.int32), qkv.shape[0], n_q, n_kv, head_dim,
           np.ascontiguousarray(cos_tab, np.float32), np.ascontiguousarray(sin_tab, np.float32), threads)
        return qkv

    def yarn_table(self, n_pos, theta=150000.0, head_dim=64, factor=32.0, orig_ctx=4096.0,
                   beta_fast=32.0, beta_slow=1.0, threads=0):
        c = np.empty((n_pos, head_dim // 2), np.float32)
        s = np.empty((n_pos, head_dim // 2), np.float32)
        self.lib.orc_yarn_table(c, s, n_pos, theta, head_dim, factor, orig_ctx, beta_fast, beta_slow,
                                threads)
        return c, s

    def moe_group(self, topk_e, e_begin, e_count):
        """Returns (counts[e_count], offsets[e_count+1], row_pair[n_local], own_row[n_pairs])."""
        te = np.ascontiguousarray(topk_e, np.int32).ravel()
        counts = np.empty(e_count, np.int32)
        offsets = np.empty(e_count + 1, np.int32)
        row_pair = np.full(te.size, -1, np.int32)
        own_row = np.full(te.size, -7, np.int32)
        self.lib.orc_moe_group(te, te.size, e_begin, e_count, counts, offsets, row_pair, own_row)
        return counts, offsets, row_pair[:offsets[-1]], own_row

    def moe_gather(self, t, row_pair, k):
        t = np.ascontiguousarray(t, np.float32)
        rp = np.ascontiguousarray(row_pair, np.int32)
        out = np.empty((rp.size, t.shape[1]), np.float32)
        self.lib.orc_moe_gather(out, t, rp, rp.size, k, t.shape[1])
        return out

    def kv_cache_write(self, qkv, n_q, n_kv, kc, vq, vs, slots, slot_of_row):
        """Writes into the given cache arrays (uint16 kc, int8 vq, float32 vs) in place."""
        qkv = np.ascontiguousarray(qkv, np.float32)
        assert kc.dtype == np.uint16 and vq.dtype == np.int8 and vs.dtype == np.float32
        self.lib.orc_kv_cache_write(qkv, qkv.shape[1], qkv.shape[0], n_q, n_kv, kc.ctypes.data, vq.ctypes.data,
                                    vs.ctypes.data, slots, np.ascontiguousarray(slot_of_row, np.int32))

    def expf(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty_like(x)
        self.lib.orc_expf_array(out, x, x.size)
        return out


class Reference(_Lib):
    """The reference's own compiled CPU functions (present only when built)."""

    def __init__(self):
        super().__init__(REF_SO, "ref_")
        assert self.lib.ref_config_size() == C.sizeof(OrcConfig)
        L = self.lib
        self.has_group = hasattr(L, "ref_has_group") and bool(L.ref_has_group())
        if self.has_group:
            L.ref_moe_group.restype = None
            L.ref_moe_group.argtypes = [_i32p, C.c_int, C.c_int, _i32p, _i32p, _i32p]
            L.ref_moe_gather.restype = None
            L.ref_moe_gather.argtypes = [_f32p, _i32p, C.c_int, C.c_int, _f32p, C.c_int]

        self.has_exact_kernels = hasattr(L, "ref_has_exact_kernels") and bool(L.ref_has_exact_kernels())
        if self.has_exact_kernels:
            L.ref_rope_exact.restype = None
            L.ref_rope_exact.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _f32p, C.c_int, C.c_int]
            L.ref_moe_combine_exact.restype = None
            L.ref_moe_combine_exact.argtypes = [_f32p, C.c_int, _f32p, _i32p, _f32p, _i32p, C.c_int, C.c_int]
        self.has_router_wave = hasattr(L, "ref_has_router_wave") and bool(L.ref_has_router_wave())
        if self.has_router_wave:
            L.ref_router_topk_wave.restype = None
            L.ref_router_topk_wave.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _i32p, C.c_int, _opt, _opt]
        self.has_rope_kv = hasattr(L, "ref_has_rope_kv") and bool(L.ref_has_rope_kv())
        if self.has_rope_kv:
            L.ref_rope_kv_bf16.restype = None
            L.ref_rope_kv_bf16.argtypes = [C.c_int, _f32p, C.c_int, _f32p, _f32p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                           C.c_void_p, C.c_int, C.c_int, C.c_int]
        self.has_argmax_key = hasattr(L, "ref_has_argmax_key") and bool(L.ref_has_argmax_key())
        if self.has_argmax_key:
            L.ref_argmax_keys.restype = None
            L.ref_argmax_keys.argtypes = [C.c_long, _f32p, _i32p, np.ctypeslib.ndpointer(np.uint64, flags="C")]
        self.has_fast_kernels = hasattr(L, "ref_has_fast_kernels") and bool(L.ref_has_fast_kernels())
        if self.has_fast_kernels:
            _u16p = np.ctypeslib.ndpointer(np.uint16, flags="C")
            L.ref_rmsnorm_bf16.restype = None
            L.ref_rmsnorm_bf16.argtypes = [C.c_int, _f32p, _f32p, _u16p, C.c_int]
            L.ref_swiglu_bf16.restype = None
            L.ref_swiglu_bf16.argtypes = [_f32p, _u16p, C.c_long, C.c_int, C.c_float]
            L.ref_moe_combine_fast.restype = None
            L.ref_moe_combine_fast.argtypes = [C.c_int, _f32p, _f32p, _i32p, _f32p, C.c_int, C.c_int]
        self.has_exact_rows = hasattr(L, "ref_has_exact_rows") and bool(L.ref_has_exact_rows())
        if self.has_exact_rows:
            _u16 = np.ctypeslib.ndpointer(np.uint16, flags="C")
            for name, args in (("ref_embed", [C.c_int, _u16, _i32p, _f32p, C.c_int]),
                               ("ref_add_inplace", [_f32p, _f32p, C.c_long]),
                               ("ref_router_topk_exact", [_f32p, C.c_int, C.c_int, _f32p, _i32p, C.c_int]),
                               ("ref_swiglu_exact", [_f32p, _f32p, C.c_long, C.c_int, C.c_float]),
                               ("ref_argmax_kernel", [C.c_int, _f32p, C.c_int, _i32p])):
                getattr(L, name).restype = None
                getattr(L, name).argtypes = args
        self.has_fused_kernels = hasattr(L, "ref_has_fused_kernels") and bool(L.ref_has_fused_kernels())
        if self.has_fused_kernels:
            _u16o = np.ctypeslib.ndpointer(np.uint16, flags="C")
            L.ref_add_rmsnorm_bf16.restype = None
            L.ref_add_rmsnorm_bf16.argtypes = [C.c_int, _f32p, _f32p, _f32p, _u16o, C.c_int]
            L.ref_moe_combine_rmsnorm.restype = None
            L.ref_moe_combine_rmsnorm.argtypes = [C.c_int, _f32p, _f32p, _i32p, _f32p, _i32p, C.c_int, C.c_int, _f32p, _u16o]
        self.has_group_ep = hasattr(L, "ref_has_group_ep") and bool(L.ref_has_group_ep())
        if self.has_group_ep:
            L.ref_moe_group_ep.restype = None
            L.ref_moe_group_ep.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, _i32p, _i32p, _i32p, _i32p]

    def router_topk_wave(self, logits, k, done=None, slot_of=None):
        """router_topk_wave_kernel (kernels/moe.hpp:64-136), the router the engine launches: (weights, experts);
        outputs start from a fill so that anything the kernel leaves unwritten shows."""
        lg = np.ascontiguousarray(logits, np.float32)
        B, E = lg.shape
        w = np.full((B, k), -7.0, np.float32)
        e = np.full((B, k), -7, np.int32)
        dn = None if done is None else np.ascontiguousarray(done, np.int32)
        so = None if slot_of is None else np.ascontiguousarray(slot_of, np.int32)
        self.lib.ref_router_topk_wave(lg, E, k, w, e, B, _addr(dn), _addr(so))
        return w, e

    def exact_rows(self, op, *a):
        """The GPU engine's bit-exact kernels, bodies run on the host: 'embed' (bf16 table bits, ids),
        'add' (x, y), 'router' (logits, k), 'swiglu' (Y, limit), 'argmax' (logits)."""
        L = self.lib
        if op == "embed":
            table, ids = np.ascontiguousarray(a[0], np.uint16), np.ascontiguousarray(a[1], np.int32)
            x = np.zeros((ids.size, table.shape[1]), np.float32)
            L.ref_embed(ids.size, table, ids, x, table.shape[1])
            return x
        if op == "add":
            x = np.array(a[0], np.float32, copy=True)
            L.ref_add_inplace(x, np.ascontiguousarray(a[1], np.float32), x.size)
            return x
        if op == "router":
            lg, k = np.ascontiguousarray(a[0], np.float32), a[1]
            w, e = np.zeros((lg.shape[0], k), np.float32), np.zeros((lg.shape[0], k), np.int32)
            L.ref_router_topk_exact(lg, lg.shape[1], k, w, e, lg.shape[0])
            return w, e
        if op == "swiglu":
            y = np.ascontiguousarray(a[0], np.float32)
            g = np.zeros((y.shape[0], y.shape[1] // 2), np.float32)
            L.ref_swiglu_exact(y, g, y.shape[0], y.shape[1] // 2, a[1])
            return g
        if op == "argmax":
            lg = np.ascontiguousarray(a[0], np.float32)
            out = np.full(lg.shape[0], -7, np.int32)
            L.ref_argmax_kernel(lg.shape[0], lg, lg.shape[1], out)
            return out
        raise ValueError(op)

    def add_rmsnorm_bf16(self, x, y, weight):
        """add_rmsnorm_bf16_kernel (kernels/fast_misc.hpp:237-256) as its launcher instantiates it:
        (x + y, bf16 bits of the normalised rows)."""
        x = np.array(x, np.float32, copy=True)
        out = np.zeros(x.shape, np.uint16)
        self.lib.ref_add_rmsnorm_bf16(x.shape[0], x, np.ascontiguousarray(y, np.float32),
                                      np.ascontiguousarray(weight, np.float32), out, x.shape[1])
        return x, out

    def moe_combine_rmsnorm(self, x, Z, own_row, weights, experts, norm_w):
        """moe_combine_rmsnorm_kernel (kernels/moe_ep.hpp:479-515) as its launcher instantiates it:
        (updated x, bf16 bits of the next norm's output)."""
        x = np.array(x, np.float32, copy=True)
        out = np.zeros(x.shape, np.uint16)
        self.lib.ref_moe_combine_rmsnorm(x.shape[0], x, np.ascontiguousarray(Z, np.float32),
                                         np.ascontiguousarray(own_row, np.int32), np.ascontiguousarray(weights, np.float32),
                                         np.ascontiguousarray(experts, np.int32), weights.shape[1], x.shape[1],
                                         np.ascontiguousarray(norm_w, np.float32), out)
        return x, out

    def rmsnorm_bf16(self, x, weight):
        """rmsnorm_bf16_kernel (kernels/fast_misc.hpp:11-30): bf16 bits of the normalised rows."""
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape, np.uint16)
        self.lib.ref_rmsnorm_bf16(x.shape[0], x, np.ascontiguousarray(weight, np.float32), out, x.shape[1])
        return out

    def swiglu_bf16(self, y, limit=7.0):
        """swiglu_bf16_kernel (kernels/fast_misc.hpp:130-141) with the C library's expf: bf16 bits."""
        y = np.ascontiguousarray(y, np.float32)
        R, I = y.shape[0], y.shape[1] // 2
        out = np.zeros((R, I), np.uint16)
        self.lib.ref_swiglu_bf16(y, out, R, I, limit)
        return out

    def moe_combine_fast(self, x, Z, pair_row, weights):
        """moe_combine_kernel (kernels/fast_misc.hpp:154-166): fused multiply-adds in choice order."""
        x = np.array(x, np.float32, copy=True)
        self.lib.ref_moe_combine_fast(x.shape[0], x, np.ascontiguousarray(Z, np.float32),
                                      np.ascontiguousarray(pair_row, np.int32), np.ascontiguousarray(weights, np.float32),
                                      weights.shape[1], x.shape[1])
        return x

    def argmax_keys(self, x, col):
        """argmax_key (kernels/fast_gemm.hpp:94-104) of each (value, column)."""
        x = np.ascontiguousarray(x, np.float32).ravel()
        col = np.ascontiguousarray(col, np.int32).ravel()
        keys = np.empty(x.size, np.uint64)
        self.lib.ref_argmax_keys(x.size, x, col, keys)
        return keys

    def rope_kv_bf16(self, rows, cos_row, sin_row, n_q, n_kv, kc, vq, vs, slots, slot, rotate_q=True):
        """rope_kv_bf16_kernel (kernels/fast_misc.hpp:48-108) as its launcher instantiates it: rotates the rows
        in place (a copy is returned) and writes row b's keys and values into the caches at (b, slot)."""
        rows = np.array(rows, np.float32, copy=True)
        assert kc.dtype == np.uint16 and vq.dtype == np.int8 and vs.dtype == np.float32
        self.lib.ref_rope_kv_bf16(rows.shape[0], rows, rows.shape[1], np.ascontiguousarray(cos_row, np.float32),
                                  np.ascontiguousarray(sin_row, np.float32), n_q, n_kv, kc.ctypes.data, vq.ctypes.data,
                                  vs.ctypes.data, slots, slot, int(rotate_q))
        return rows

    def rope_exact(self, rows, cos_row, sin_row, n_heads, head_dim):
        """rope_exact (kernels/misc.hpp:55-70) on biased rows [B, row_stride]: the first n_heads heads of each
        row rotated by one position's cos/sin, one block per row."""
        rows = np.array(rows, np.float32, copy=True)
        self.lib.ref_rope_exact(rows, rows.shape[0], rows.shape[1], np.ascontiguousarray(cos_row, np.float32),
                                np.ascontiguousarray(sin_row, np.float32), n_heads, head_dim)
        return rows

    def moe_combine_exact(self, x, Z, pair_row, weights, experts):
        """moe_combine_exact (kernels/moe.hpp:210-236): one block per token."""
        x = np.array(x, np.float32, copy=True)
        k = weights.shape[1]
        self.lib.ref_moe_combine_exact(x, x.shape[0], np.ascontiguousarray(Z, np.float32),
                                       np.ascontiguousarray(pair_row, np.int32), np.ascontiguousarray(weights, np.float32),
                                       np.ascontiguousarray(experts, np.int32), k, x.shape[1])
        return x

    def moe_group_ep(self, topk_e, e_begin, e_count):
        """moe_count_ep_kernel + moe_place_ep_kernel for experts e_begin .. e_begin + e_count - 1 with no
        partner: (counts[e_count], offsets[e_count + 1], row_pair[rows], own_row[n_pairs]); own_row starts
        from a fill that the kernels must overwrite for every pair."""
        te = np.ascontiguousarray(topk_e, np.int32).ravel()
        counts = np.full(e_count, -7, np.int32)
        offsets = np.full(e_count + 1, -7, np.int32)
        row_pair = np.full(max(te.size, 1), -7, np.int32)
        own_row = np.full(max(te.size, 1), -7, np.int32)
        self.lib.ref_moe_group_ep(te, te.size, e_begin, e_count, counts, offsets, row_pair, own_row)
        return counts, offsets, row_pair[:offsets[-1]], own_row[:te.size]

    def moe_group(self, topk_e, n_experts):
        """moe_group_kernel over all experts: (offsets[E+1], row_pair[n_routed], pair_row[n_pairs], -1 where
        the kernel writes nothing: pairs of finished tokens)."""
        te = np.ascontiguousarray(topk_e, np.int32).ravel()
        offsets = np.full(n_experts + 1, -7, np.int32)
        row_pair = np.full(te.size, -7, np.int32)
        pair_row = np.full(te.size, -1, np.int32)
        self.lib.ref_moe_group(te, te.size, n_experts, offsets, row_pair, pair_row)
        return offsets, row_pair[:offsets[-1]], pair_row

    def moe_gather(self, t, row_pair, k):
        t = np.ascontiguousarray(t, np.float32)
        rp = np.ascontiguousarray(row_pair, np.int32)
        out = np.full((rp.size, t.shape[1]), np.nan, np.float32)
        self.lib.ref_moe_gather(t, rp, rp.size, k, out, t.shape[1])
        return out


def have_reference() -> bool:
    return os.path.exists(REF_SO)
