"""Helpers for the GPU parity tests: device buffers with canary guards, dtype plumbing,
and the tolerances the tests hold the kernels to."""
from __future__ import annotations

import numpy as np

# Tolerances (relative, per element, against max(|reference|, floor)):
#   fp32 mode  (GPTOSS_EXACT, fp32 tensors)      1e-5
#   bf16 mode  (bf16 activations, fast math)     2e-2
# The floor keeps elements that cancel to ~0 (RoPE's x1*c - x2*s, sums of signed
# terms) from being judged on noise: 1 % of the RMS of the reference tensor.
TOL_F32 = 1e-5
TOL_BF16 = 2e-2

GUARD = 256  # bytes of canary on each side of an output buffer
CANARY = 0x55


def floor_of(want) -> float:
    w = np.asarray(want, np.float64)
    return max(1e-30, 0.01 * float(np.sqrt(np.mean(w * w)))) if w.size else 1.0


def rel_err(got, want) -> float:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if got.size == 0:
        return 0.0
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor_of(want))))


def rel_err_unfloored(got, want) -> float:
    """max |got - want| / |want| over the elements whose reference is not zero: the plain
    relative error, with no floor under small references."""
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    nz = want != 0
    return float(np.max(np.abs(got[nz] - want[nz]) / np.abs(want[nz]))) if nz.any() else 0.0


def bf16_ulps_apart(a_bits, b_bits) -> int:
    """Largest distance, in representable bf16 values, between two arrays of bf16 bit patterns."""
    def ordered(u):
        u = np.asarray(u, np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7fff), u & 0x7fff)
    a, b = ordered(a_bits), ordered(b_bits)
    return int(np.max(np.abs(a - b))) if a.size else 0


def n_bit_diff(a, b) -> int:
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    v = {4: np.uint32, 2: np.uint16}[a.dtype.itemsize]
    return int(np.count_nonzero(a.view(v) != b.view(v)))


class Dev:
    """Uploads inputs / allocates guarded outputs on the current device."""

    def __init__(self, pkg):
        self.pkg = pkg
        self.keep = []

    def put(self, a, dtype=None):
        """numpy array -> device; dtype BF16 converts fp32 values to bf16 bits first."""
        pkg = self.pkg
        a = np.ascontiguousarray(a)
        if dtype == pkg.BF16 and a.dtype == np.float32:
            a = pkg.to_bf16_bits(a)
        b = pkg.DeviceBuffer.from_numpy(a)
        self.keep.append(b)
        return b

    def out(self, shape, dtype):
        """Guarded, canary-filled output buffer for `shape` elements of gptoss dtype or numpy dtype."""
        pkg = self.pkg
        np_dtype = {pkg.F32: np.float32, pkg.BF16: np.uint16}.get(dtype, dtype)
        n = int(np.prod(shape)) * np.dtype(np_dtype).itemsize
        pad = (-n) % 16
        b = pkg.DeviceBuffer.filled(GUARD + n + pad + GUARD, CANARY)
        self.keep.append(b)
        return Out(self.pkg, b, shape, np_dtype, n + pad)

    def put_inout(self, a):
        """Guarded buffer initialised with `a` (for tensors updated in place)."""
        a = np.ascontiguousarray(a)
        o = self.out(a.shape, a.dtype)
        pkg = self.pkg
        pkg.check(pkg.load().gptoss_upload(o.ptr, a.ctypes.data, a.nbytes, None))
        pkg.synchronize()
        return o


class Out:
    def __init__(self, pkg, buf, shape, np_dtype, padded):
        self.pkg, self.buf, self.shape, self.np_dtype, self.padded = pkg, buf, shape, np_dtype, padded
        self.ptr = buf.ptr + GUARD

    def get(self, as_f32=True):
        """Downloads the payload and checks that neither guard was touched."""
        raw = self.buf.numpy(np.uint8, self.buf.nbytes)
        n = int(np.prod(self.shape)) * np.dtype(self.np_dtype).itemsize
        assert (raw[:GUARD] == CANARY).all(), "write before the start of the output buffer"
        assert (raw[GUARD + n:] == CANARY).all(), "write past the end of the output buffer"
        a = raw[GUARD:GUARD + n].view(self.np_dtype).reshape(self.shape)
        if as_f32 and self.np_dtype == np.uint16:
            return self.pkg.from_bf16_bits(a).reshape(self.shape)
        return a.copy()


def widen(pkg, a, dtype):
    """The fp32 values a kernel sees for host data `a` stored as `dtype`."""
    a = np.ascontiguousarray(a, np.float32)
    return pkg.bf16_round(a) if dtype == pkg.BF16 else a
