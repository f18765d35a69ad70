"""gptoss-b200-fused: ctypes binding of libgptoss_b200.so.

The product is the shared library (CUDA kernels for sm_100a behind the C ABI of
``include/gptoss_kernels.h`` plus the C++ host driver of ``include/gptoss_engine.h``).
This module is only the thin Python face of it that the tests and the bench use:
it loads the library, declares every prototype, and wraps device buffers.  There is
no Python or CPU implementation of any op here: if the library is missing or no
CUDA device answers, calls raise.

The directory name contains a hyphen, so import it with
``importlib.import_module("optimize_inference_gpt-oss_b200")``.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GPTOSS_B200_LIB") or os.path.join(_HERE, "libgptoss_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")

F32, BF16 = 0, 1
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA = 0, 1, 2, 3
EXACT, FMA, PDL, BULK_STAGE = 1, 2, 4, 8
CHAIN_SPLIT_EMBED_NORM = 0x100  # chain only: gather and first norm as two launches
MAX_TOPK, MAX_EXPERTS = 8, 256

# gptoss_chain_buffer_t
(BUF_EMBEDDING, BUF_GAIN_ATTN, BUF_GAIN_FFN, BUF_GAIN_OUT, BUF_QKV_BIAS, BUF_COS, BUF_SIN,
 BUF_ATTN_PROJ, BUF_QKV, BUF_ROUTER, BUF_MLP1, BUF_EXPERT, BUF_LOGITS, BUF_TOKENS, BUF_POS, BUF_X,
 BUF_NORMED, BUF_QKV_OUT, BUF_TOPK_W, BUF_TOPK_E, BUF_SWIGLU, BUF_NEXT, BUF_ROW_DONE, BUF_COUNT) = range(24)
# gptoss_chain_kernel_t
KERNEL_KINDS = ("embed", "norm", "rope", "add_norm", "router", "swiglu", "combine", "argmax")


class GptossError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(what)


class ChainConfig(C.Structure):
    _fields_ = [
        ("vocab", C.c_int), ("hidden", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int),
        ("inter", C.c_int), ("n_layers", C.c_int), ("head_dim", C.c_int), ("n_q_heads", C.c_int),
        ("n_kv_heads", C.c_int), ("max_pos", C.c_int), ("orig_ctx", C.c_float), ("theta", C.c_float),
        ("factor", C.c_float), ("beta_fast", C.c_float), ("beta_slow", C.c_float),
        ("swiglu_limit", C.c_float), ("act_dtype", C.c_int), ("flags", C.c_uint),
    ]

    @property
    def qkv_dim(self) -> int:
        return (self.n_q_heads + 2 * self.n_kv_heads) * self.head_dim


_p, _i, _l, _z, _f, _u = C.c_void_p, C.c_int, C.c_long, C.c_size_t, C.c_float, C.c_uint

# name -> (restype, argtypes); mirrors include/gptoss_kernels.h and include/gptoss_engine.h
PROTOTYPES = {
    "gptoss_version": (C.c_char_p, []),
    "gptoss_status_string": (C.c_char_p, [_i]),
    "gptoss_last_cuda_error": (_i, []),
    "gptoss_generic_launch_count": (_l, []),
    "gptoss_wait_giveups": (_l, []),
    "gptoss_bounds_enabled": (_i, []),
    "gptoss_bounds_violations": (_l, []),
    "gptoss_bounds_checked_spans": (_l, []),
    "gptoss_embed": (_i, [_p, _i, _p, _i, _i, _p, _p, _i, _i, _u]),
    "gptoss_embed_rmsnorm": (_i, [_p, _i, _p, _i, _i, _p, _p, _p, _p, _i, _i, _u]),
    "gptoss_add_rmsnorm": (_i, [_p, _i, _p, _p, _i, _p, _p, _i, _i, _u]),
    "gptoss_qkv_bias_rope": (_i, [_p, _i, _p, _i, _l, _p, _p, _i, _p, _p, _i, _i, _i, _i, _p, _i, _l, _u]),
    "gptoss_qkv_bias_rope_kv": (_i, [_p, _i, _p, _i, _l, _p, _p, _i, _p, _p, _i, _i, _i, _i, _p, _i, _l,
                                    _p, _p, _p, _i, _p, _i, _u]),
    "gptoss_router_topk": (_i, [_p, _i, _p, _i, _i, _i, _p, _p, _p, _p, _u]),
    "gptoss_swiglu": (_i, [_p, _p, _i, _p, _i, _z, _i, _f, _u]),
    "gptoss_moe_combine": (_i, [_p, _i, _p, _p, _i, _p, _p, _p, _i, _i, _p, _p, _p, _i, _u]),
    "gptoss_argmax": (_i, [_p, _i, _p, _i, _l, _l, _p, _p, _u]),
    "gptoss_moe_group": (_i, [_p, _p, _i, _i, _i, _p, _p, _p, _p, _u]),
    "gptoss_moe_gather": (_i, [_p, _i, _p, _i, _i, _p, _i, _p, _i, _u]),
    "gptoss_kv_cache_write": (_i, [_p, _i, _p, _i, _l, _i, _i, _i, _p, _p, _p, _i, _p, _i, _u]),
    "gptoss_argmax_keys_finish": (_i, [_p, _i, _p, _p, _u]),
    "gptoss_argmax_slices": (_i, [_i, _l, _i, _i]),
    "gptoss_argmax_noalloc": (_i, [_p, _i, _p, _i, _l, _l, _p]),
    "gptoss_device_count": (_i, [C.POINTER(_i)]),
    "gptoss_device_set": (_i, [_i]),
    "gptoss_device_name": (_i, [_i, C.c_char_p, _i]),
    "gptoss_device_alloc": (_i, [C.POINTER(_p), _z]),
    "gptoss_device_free": (_i, [_p]),
    "gptoss_device_memset": (_i, [_p, _i, _z, _p]),
    "gptoss_upload": (_i, [_p, _p, _z, _p]),
    "gptoss_download": (_i, [_p, _p, _z, _p]),
    "gptoss_host_alloc_pinned": (_i, [C.POINTER(_p), _z]),
    "gptoss_host_free_pinned": (_i, [_p]),
    "gptoss_stream_create": (_i, [C.POINTER(_p)]),
    "gptoss_stream_destroy": (_i, [_p]),
    "gptoss_stream_synchronize": (_i, [_p]),
    "gptoss_device_synchronize": (_i, []),
    "gptoss_event_create": (_i, [C.POINTER(_p)]),
    "gptoss_event_destroy": (_i, [_p]),
    "gptoss_event_record": (_i, [_p, _p]),
    "gptoss_event_synchronize": (_i, [_p]),
    "gptoss_event_elapsed_ms": (_i, [_p, _p, C.POINTER(_f)]),
    "gptoss_flush_l2": (_i, [_p, _z, _p]),
    "gptoss_graph_begin": (_i, [_p]),
    "gptoss_graph_end": (_i, [_p, C.POINTER(_p)]),
    "gptoss_graph_launch": (_i, [_p, _p]),
    "gptoss_graph_destroy": (_i, [_p]),
    "gptoss_build_rope_tables": (_i, [_i, _i, _f, _f, _f, _f, _f, _p, _p]),
    "gptoss_synth_normal": (_i, [_p, _i, _z, C.c_uint64, C.c_uint64, _f, _f, _i]),
    "gptoss_synth_uniform_int": (_i, [_p, _z, C.c_uint64, C.c_uint64, _i, _i]),
    "gptoss_chain_config_gpt_oss": (_i, [_i, _i, _i, C.POINTER(ChainConfig)]),
    "gptoss_chain_create": (_i, [C.POINTER(ChainConfig), _i, _i, C.POINTER(_p)]),
    "gptoss_chain_destroy": (_i, [_p]),
    "gptoss_chain_device_bytes": (_z, [_p]),
    "gptoss_chain_stream": (_p, [_p]),
    "gptoss_chain_buffer": (_i, [_p, _i, _i, C.POINTER(_p), C.POINTER(_z)]),
    "gptoss_chain_fill_synthetic": (_i, [_p, _i, C.c_uint64, _i]),
    "gptoss_chain_enqueue": (_i, [_p, _i, _i]),
    "gptoss_chain_step": (_i, [_p, _i, _p, _p, _p]),
    "gptoss_chain_run_wave": (_i, [_p, _p, _p, _i, _i, _p, C.POINTER(C.c_longlong), C.POINTER(_i)]),
    "gptoss_chain_run_wave_on_device": (_i, [_p, _p, _p, _i, _i, _p, C.POINTER(C.c_longlong), C.POINTER(_i)]),
    "gptoss_chain_profile": (_i, [_p, _i, _i, _i, C.POINTER(C.c_double), C.POINTER(_l)]),
    "gptoss_chain_kernel_bytes": (_z, [_p, _i, _i]),
    "gptoss_chain_launches_per_step": (_i, [_p, _i]),
}

_lib = None


def load() -> C.CDLL:
    """Loads libgptoss_b200.so (built by build.py).  Raises if it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise GptossError(-1, f"{LIB_PATH} is missing: run "
                                  f"`python optimize_inference_gpt-oss_b200/build.py` (needs nvcc); "
                                  f"there is no fallback implementation")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str = "") -> None:
    if status != OK:
        lib = load()
        msg = lib.gptoss_status_string(status).decode()
        if status == ERR_CUDA:
            msg += f" [cudaError {lib.gptoss_last_cuda_error()}]"
        raise GptossError(status, f"{what}: {msg}" if what else msg)


def device_count() -> int:
    n = _i(0)
    check(load().gptoss_device_count(C.byref(n)), "device_count")
    return n.value


def set_device(d: int) -> None:
    check(load().gptoss_device_set(d), "set_device")


def device_name(d: int = 0) -> str:
    buf = C.create_string_buffer(256)
    check(load().gptoss_device_name(d, buf, 256), "device_name")
    return buf.value.decode()


def synchronize() -> None:
    check(load().gptoss_device_synchronize(), "synchronize")


# ---- bf16 on the host (numpy has no bfloat16): raw uint16 bit patterns ------------

def to_bf16_bits(a) -> np.ndarray:
    """fp32 -> bf16 bits, round to nearest even, NaN kept quiet."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def from_bf16_bits(b) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(a) -> np.ndarray:
    """fp32 values rounded to the nearest bf16, still stored as fp32."""
    return from_bf16_bits(to_bf16_bits(a))


class DeviceBuffer:
    """A device allocation owned by the caller (the engine's gpu_alloc)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = _p()
        check(load().gptoss_device_alloc(C.byref(p), self.nbytes), "device_alloc")
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        b = cls(max(a.nbytes, 16))
        if a.nbytes:
            check(load().gptoss_upload(b.ptr, a.ctypes.data, a.nbytes, None), "upload")
            synchronize()
        return b

    @classmethod
    def filled(cls, nbytes: int, byte: int) -> "DeviceBuffer":
        b = cls(nbytes)
        check(load().gptoss_device_memset(b.ptr, byte, b.nbytes, None), "memset")
        synchronize()
        return b

    def numpy(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype)
        synchronize()
        if out.nbytes:
            check(load().gptoss_download(out.ctypes.data, self.ptr + offset, out.nbytes, None), "download")
            synchronize()
        return out

    def free(self) -> None:
        if getattr(self, "ptr", None):
            load().gptoss_device_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr(x):
    if x is None:
        return None
    if hasattr(x, "ptr"):  # a DeviceBuffer, or any view object that carries a device address
        return x.ptr
    return int(x)


# ---- the kernels (device pointers in, status checked) ----------------------------

def embed(T, table, table_dtype, V, ids, x, x_dtype, H, flags=0, stream=None):
    check(load().gptoss_embed(stream, T, _ptr(table), table_dtype, V, _ptr(ids), _ptr(x), x_dtype, H, flags), "embed")


def embed_rmsnorm(T, table, table_dtype, V, ids, x, weight, out, out_dtype, H, flags=0, stream=None):
    check(load().gptoss_embed_rmsnorm(stream, T, _ptr(table), table_dtype, V, _ptr(ids), _ptr(x), _ptr(weight),
                                      _ptr(out), out_dtype, H, flags), "embed_rmsnorm")


def add_rmsnorm(T, x, y, y_dtype, weight, out, out_dtype, H, flags=0, stream=None):
    check(load().gptoss_add_rmsnorm(stream, T, _ptr(x), _ptr(y), y_dtype, _ptr(weight), _ptr(out),
                                    out_dtype, H, flags), "add_rmsnorm")


def qkv_bias_rope(T, qkv_in, in_dtype, in_stride, bias, pos, pos_scalar, cos_tab, sin_tab, n_pos,
                  n_q, n_kv, head_dim, qkv_out, out_dtype, out_stride, flags=0, stream=None):
    check(load().gptoss_qkv_bias_rope(stream, T, _ptr(qkv_in), in_dtype, in_stride, _ptr(bias), _ptr(pos),
                                      pos_scalar, _ptr(cos_tab), _ptr(sin_tab), n_pos, n_q, n_kv,
                                      head_dim, _ptr(qkv_out), out_dtype, out_stride, flags), "qkv_bias_rope")


def qkv_bias_rope_kv(T, qkv_in, in_dtype, in_stride, bias, pos, pos_scalar, cos_tab, sin_tab, n_pos,
                     n_q, n_kv, head_dim, qkv_out, out_dtype, out_stride, kc, vq, vs, slots,
                     slot_of_row=None, slot_scalar=0, flags=0, stream=None):
    check(load().gptoss_qkv_bias_rope_kv(stream, T, _ptr(qkv_in), in_dtype, in_stride, _ptr(bias), _ptr(pos),
                                         pos_scalar, _ptr(cos_tab), _ptr(sin_tab), n_pos, n_q, n_kv,
                                         head_dim, _ptr(qkv_out), out_dtype, out_stride, _ptr(kc), _ptr(vq),
                                         _ptr(vs), slots, _ptr(slot_of_row), slot_scalar, flags),
          "qkv_bias_rope_kv")


def router_topk(T, logits, dtype, E, k, topk_w, topk_e, done=None, slot_of=None, flags=0, stream=None):
    check(load().gptoss_router_topk(stream, T, _ptr(logits), dtype, E, k, _ptr(topk_w), _ptr(topk_e),
                                    _ptr(done), _ptr(slot_of), flags), "router_topk")


def swiglu(Y, y_dtype, G, g_dtype, R, I, limit=7.0, flags=0, stream=None):
    check(load().gptoss_swiglu(stream, _ptr(Y), y_dtype, _ptr(G), g_dtype, R, I, limit, flags), "swiglu")


def moe_combine(T, x, Z, z_dtype, own_row, topk_w, topk_e, k, H, phys_of=None, norm_w=None, out=None,
                out_dtype=F32, flags=0, stream=None):
    check(load().gptoss_moe_combine(stream, T, _ptr(x), _ptr(Z), z_dtype, _ptr(own_row), _ptr(topk_w),
                                    _ptr(topk_e), k, H, _ptr(phys_of), _ptr(norm_w), _ptr(out), out_dtype,
                                    flags), "moe_combine")


def argmax(T, logits, dtype, V, row_stride, keys, out, flags=0, stream=None):
    check(load().gptoss_argmax(stream, T, _ptr(logits), dtype, V, row_stride, _ptr(keys), _ptr(out), flags), "argmax")


def moe_group(topk_e, n_pairs, e_begin, e_count, counts, offsets, row_pair, own_row, flags=0, stream=None):
    check(load().gptoss_moe_group(stream, _ptr(topk_e), n_pairs, e_begin, e_count, _ptr(counts), _ptr(offsets),
                                  _ptr(row_pair), _ptr(own_row), flags), "moe_group")


def moe_gather(R, t, dtype, n_tokens, row_pair, k, Xg, H, flags=0, stream=None):
    check(load().gptoss_moe_gather(stream, R, _ptr(t), dtype, n_tokens, _ptr(row_pair), k, _ptr(Xg), H, flags),
          "moe_gather")


def kv_cache_write(T, qkv, dtype, row_stride, n_q, n_kv, head_dim, kc, vq, vs, slots, slot_of_row=None,
                   slot_scalar=0, flags=0, stream=None):
    check(load().gptoss_kv_cache_write(stream, T, _ptr(qkv), dtype, row_stride, n_q, n_kv, head_dim, _ptr(kc),
                                       _ptr(vq), _ptr(vs), slots, _ptr(slot_of_row), slot_scalar, flags),
          "kv_cache_write")


def argmax_keys_finish(T, keys, out, flags=0, stream=None):
    check(load().gptoss_argmax_keys_finish(stream, T, _ptr(keys), _ptr(out), flags), "argmax_keys_finish")


def argmax_key_host(values: np.ndarray, cols: np.ndarray) -> np.ndarray:
    """The 64-bit key of gptoss_argmax_key.cuh computed on the host (for tests and for
    checking a producer): order-preserving value bits above the complemented column."""
    v = np.ascontiguousarray(values, np.float32)
    u = np.where(v == 0, np.uint32(0), v.view(np.uint32)).astype(np.uint32)
    neg = (u & np.uint32(0x80000000)) != 0
    u = np.where(neg, ~u, u | np.uint32(0x80000000)).astype(np.uint64)
    key = (u << np.uint64(32)) | (~np.ascontiguousarray(cols, np.uint32)).astype(np.uint64)
    return np.where(np.isnan(v), np.uint64(0), key)


ARGMAX_NOALLOC_MAX_ROWS = 16384


def argmax_noalloc(T, logits, dtype, V, row_stride, out, stream=None):
    """gptoss_argmax without caller scratch: the merge words sit in a fixed array inside the
    library, so at most ARGMAX_NOALLOC_MAX_ROWS rows per call and no overlapping calls per GPU."""
    check(load().gptoss_argmax_noalloc(stream, T, _ptr(logits), dtype, V, row_stride, _ptr(out)), "argmax_noalloc")


def build_rope_tables(n_pos, head_dim=64, theta=150000.0, factor=32.0, orig_ctx=4096.0,
                      beta_fast=32.0, beta_slow=1.0):
    """Host-side cos/sin tables [n_pos, head_dim/2] (the engine builds them on the host too)."""
    cs = np.empty((n_pos, head_dim // 2), np.float32)
    sn = np.empty((n_pos, head_dim // 2), np.float32)
    check(load().gptoss_build_rope_tables(n_pos, head_dim, theta, factor, orig_ctx, beta_fast, beta_slow,
                                          cs.ctypes.data, sn.ctypes.data), "build_rope_tables")
    return cs, sn


def synth_normal(count, dtype, seed, stream_id, mean=0.0, sd=1.0, threads=0) -> np.ndarray:
    out = np.empty(count, np.float32 if dtype == F32 else np.uint16)
    check(load().gptoss_synth_normal(out.ctypes.data, dtype, count, seed, stream_id, mean, sd, threads),
          "synth_normal")
    return out


def synth_uniform_int(count, seed, stream_id, lo, hi) -> np.ndarray:
    out = np.empty(count, np.int32)
    check(load().gptoss_synth_uniform_int(out.ctypes.data, count, seed, stream_id, lo, hi), "synth_uniform_int")
    return out


class PinnedArray:
    """A numpy view of page-locked host memory."""

    def __init__(self, shape, dtype):
        self.shape = tuple(np.atleast_1d(shape))
        self.dtype = np.dtype(dtype)
        n = int(np.prod(self.shape)) * self.dtype.itemsize
        p = _p()
        check(load().gptoss_host_alloc_pinned(C.byref(p), max(n, 16)), "host_alloc_pinned")
        self.ptr = p.value
        buf = (C.c_char * max(n, 16)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    def free(self):
        if getattr(self, "ptr", None):
            self.array = None
            load().gptoss_host_free_pinned(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Stream:
    """A stream of this library (gptoss_stream_create)."""

    def __init__(self):
        h = _p()
        check(load().gptoss_stream_create(C.byref(h)), "stream_create")
        self.h = h.value

    def synchronize(self):
        check(load().gptoss_stream_synchronize(self.h), "stream_synchronize")

    def close(self):
        if getattr(self, "h", None):
            load().gptoss_stream_destroy(self.h)
            self.h = None


class Graph:
    """Launches captured on a stream, replayable with one call (gptoss_graph_*).

        g = Graph(stream)
        with g:             # everything launched on `stream` by this thread is recorded
            pkg.swiglu(..., stream=stream)
        g.launch()
    """

    def __init__(self, stream):
        self.stream, self.h = stream, None

    def __enter__(self):
        check(load().gptoss_graph_begin(self.stream), "graph_begin")
        return self

    def __exit__(self, exc_type, exc, tb):
        h = _p()
        st = load().gptoss_graph_end(self.stream, C.byref(h))
        self.h = h.value
        if exc_type is None:
            check(st, "graph_end")
        return False

    def launch(self):
        check(load().gptoss_graph_launch(self.h, self.stream), "graph_launch")

    def close(self):
        if self.h:
            load().gptoss_graph_destroy(self.h)
            self.h = None


def chain_config(which: int, act_dtype: int = BF16, max_pos: int = 4096) -> ChainConfig:
    cfg = ChainConfig()
    check(load().gptoss_chain_config_gpt_oss(which, act_dtype, max_pos, C.byref(cfg)), "chain_config")
    return cfg


class Chain:
    """The C++ layer-chain driver (gptoss_chain_*) for one device."""

    def __init__(self, cfg: ChainConfig, max_tokens: int, n_standin_layers: int | None = None):
        self.cfg = cfg
        self.max_tokens = max_tokens
        h = _p()
        sets = cfg.n_layers if n_standin_layers is None else n_standin_layers
        check(load().gptoss_chain_create(C.byref(cfg), max_tokens, sets, C.byref(h)), "chain_create")
        self.h = h.value

    def close(self):
        if getattr(self, "h", None):
            load().gptoss_chain_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self):
        return load().gptoss_chain_stream(self.h)

    @property
    def device_bytes(self) -> int:
        return int(load().gptoss_chain_device_bytes(self.h))

    def buffer(self, which: int, layer: int = 0):
        p, n = _p(), _z()
        check(load().gptoss_chain_buffer(self.h, which, layer, C.byref(p), C.byref(n)), "chain_buffer")
        return p.value, n.value

    def upload(self, which: int, layer: int, a: np.ndarray):
        a = np.ascontiguousarray(a)
        p, n = self.buffer(which, layer)
        assert a.nbytes <= n, (which, a.nbytes, n)
        check(load().gptoss_upload(p, a.ctypes.data, a.nbytes, None), "upload")
        synchronize()

    def download(self, which: int, layer: int, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        p, n = self.buffer(which, layer)
        assert out.nbytes <= n
        synchronize()
        check(load().gptoss_download(out.ctypes.data, p, out.nbytes, None), "download")
        synchronize()
        return out

    def fill_synthetic(self, T: int, seed: int = 1, threads: int = 0):
        check(load().gptoss_chain_fill_synthetic(self.h, T, seed, threads), "chain_fill_synthetic")

    def enqueue(self, T: int, use_graph: bool = True):
        check(load().gptoss_chain_enqueue(self.h, T, 1 if use_graph else 0), "chain_enqueue")

    def step(self, tokens_host: np.ndarray, pos_host: np.ndarray, next_host: np.ndarray):
        T = tokens_host.size
        check(load().gptoss_chain_step(self.h, T, tokens_host.ctypes.data, pos_host.ctypes.data,
                                       next_host.ctypes.data), "chain_step")

    def run_wave(self, prompts, steps: int, on_device: bool = False):
        """Serves one wave (gptoss_chain_run_wave, or gptoss_chain_run_wave_on_device with the
        bookkeeping kept on the GPU).  prompts: a list of token lists.  Returns (generated
        [n, steps + 2] int32 closed with -1, the reference's generated-token count, steps
        actually run)."""
        offs = np.zeros(len(prompts) + 1, np.int32)
        offs[1:] = np.cumsum([len(p) for p in prompts])
        toks = np.ascontiguousarray(np.concatenate([np.asarray(p, np.int32) for p in prompts]) if prompts
                                    else np.zeros(0, np.int32))
        out = np.empty((len(prompts), steps + 2), np.int32)
        total, ran = C.c_longlong(0), _i(0)
        fn = load().gptoss_chain_run_wave_on_device if on_device else load().gptoss_chain_run_wave
        check(fn(self.h, toks.ctypes.data, offs.ctypes.data, len(prompts), steps,
                                           out.ctypes.data, C.byref(total), C.byref(ran)), "chain_run_wave")
        return out, int(total.value), int(ran.value)

    def profile(self, T: int, steps: int, mode: int = 0):
        """Per kernel kind: (summed device ms, launches).  mode 0: an event pair per launch;
        1: the same after an L2 flush; 2: one pair per kind around its back-to-back launches."""
        n = len(KERNEL_KINDS)
        ms = (C.c_double * n)()
        cnt = (_l * n)()
        check(load().gptoss_chain_profile(self.h, T, steps, mode, ms, cnt), "chain_profile")
        return {k: (ms[i], cnt[i]) for i, k in enumerate(KERNEL_KINDS)}

    def kernel_bytes(self, kind: str, T: int) -> int:
        return int(load().gptoss_chain_kernel_bytes(self.h, KERNEL_KINDS.index(kind), T))

    def launches_per_step(self, T: int) -> int:
        return int(load().gptoss_chain_launches_per_step(self.h, T))
