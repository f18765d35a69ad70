"""The allocation-free argmax entry point (gptoss_argmax_noalloc) against the regular one.

Some hosts of the library cannot give a kernel scratch memory at call time (a serving
process whose pool owns the whole GPU; a decode loop that must never hit cudaMalloc), so
this entry point keeps its per-row merge words in a fixed array inside the library.  That
array is shared by every call and keeps the previous call's contents, which is what the
second call below is about: different data, same array, still the right answer.

The file name sorts last on purpose: a run that stops at the first failure has already run
every other test.  It needs nothing from them and passes alone in a fresh process too.
"""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(pkg, seed, T, V, dtype):
    vals = pkg.synth_normal(T * V, dtype, seed, 0, 0.0, 3.0).reshape(T, V)
    if dtype == pkg.F32:
        vals[1, 5], vals[1, V - 9] = 50.0, 50.0  # a tie across slices: the lower column wins
    return vals


@pytest.mark.parametrize("dtype_name,T,V", [("f32", 300, 50000), ("bf16", 96, 201088)])
def test_noalloc_argmax_equals_argmax_on_two_calls_in_a_row(gpu, orc, dtype_name, T, V):
    pkg = gpu
    dtype = pkg.F32 if dtype_name == "f32" else pkg.BF16
    # the shapes are chosen so that rows are cut into slices and the merge words are really used
    assert pkg.load().gptoss_argmax_slices(T, V, dtype, 1) > 1
    keys = pkg.DeviceBuffer.from_numpy(np.zeros(T, np.uint64))
    want_buf, got_buf = pkg.DeviceBuffer(T * 4), pkg.DeviceBuffer(T * 4)
    answers = []
    for call, seed in enumerate((101, 202)):
        logits = pkg.DeviceBuffer.from_numpy(_case(pkg, seed, T, V, dtype))
        pkg.argmax(T, logits, dtype, V, V, keys, want_buf)          # existing entry point, caller scratch
        pkg.argmax_noalloc(T, logits, dtype, V, V, got_buf)         # new entry point, built-in scratch
        want, got = want_buf.numpy(np.int32, T), got_buf.numpy(np.int32, T)
        assert np.array_equal(got, want), f"call {call}: indices are integers, they must match exactly"
        # both entry points share their kernels and the key merge, so the CPU oracle is asked too
        host = _case(pkg, seed, T, V, dtype)
        host = pkg.from_bf16_bits(host).reshape(T, V) if dtype == pkg.BF16 else host
        assert np.array_equal(got, orc.argmax_rows(host, threads=0)), f"call {call}: against the CPU oracle"
        answers.append(got)
        logits.free()
    assert not np.array_equal(answers[0], answers[1]), "the two calls must have seen different data"
    if dtype == pkg.F32:
        assert answers[0][1] == 5 and answers[1][1] == 5


def test_noalloc_argmax_takes_exactly_as_many_rows_as_its_scratch_holds(gpu, orc):
    """The largest batch the entry point accepts, with short rows: the last row's merge word is
    the last word of the built-in array."""
    pkg = gpu
    T, V = pkg.ARGMAX_NOALLOC_MAX_ROWS, 1024
    host = _case(pkg, 303, T, V, pkg.F32)
    logits, out = pkg.DeviceBuffer.from_numpy(host), pkg.DeviceBuffer(T * 4)
    for _ in range(2):
        pkg.argmax_noalloc(T, logits, pkg.F32, V, V, out)
        assert np.array_equal(out.numpy(np.int32, T), orc.argmax_rows(host, threads=0))
    logits.free()


def test_noalloc_argmax_refuses_more_rows_than_its_scratch_holds(gpu):
    pkg = gpu
    lib = pkg.load()
    T = pkg.ARGMAX_NOALLOC_MAX_ROWS + 1
    fake = 0x1000  # the size check comes before anything is touched or launched
    assert lib.gptoss_argmax_noalloc(None, T, fake, pkg.F32, 8, 8, fake) == pkg.ERR_UNSUPPORTED
    assert lib.gptoss_argmax_noalloc(None, 0, None, pkg.F32, 8, 8, None) == pkg.OK
    assert lib.gptoss_argmax_noalloc(None, 4, None, pkg.F32, 8, 8, fake) == pkg.ERR_BAD_ARG
