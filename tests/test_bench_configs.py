"""Host-side logic of bench.py: how each benchmark configuration resolves into what a rank
runs (no GPU, no CUDA library)."""
from __future__ import annotations

import argparse
import importlib.util
import os

import numpy as np
import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _args(**kw):
    base = dict(config=1, model=None, fp32=False, tokens_per_gpu=None, seed=1)
    base.update(kw)
    return argparse.Namespace(**base)


def test_bench_shard_range_is_the_package_split(bench):
    sharding = importlib.import_module("optimize_inference_gpt-oss_b200.sharding")
    for total, granule in ((16384, 1024), (4096, 1), (4097, 1), (3072, 1024)):
        for world in (1, 2, 3, 4, 8):
            for rank in range(world):
                assert bench.shard_range(total, world, rank, granule) == sharding.shard_range(total, world, rank, granule)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_prefill_configuration_shards_whole_sequences(bench, world):
    """Config 2: 16 sequences of 1024 positions over the ranks, contiguous, nothing lost, every
    rank's positions continue where the previous rank's stopped (t mod 1024)."""
    works = [bench.Work(_args(config=2), world, r) for r in range(world)]
    assert all(w.scaling == "strong" and w.total == 16384 for w in works)
    assert sum(w.T for w in works) == 16384 and all(w.T % 1024 == 0 for w in works)
    pos = np.concatenate([w.pos_array() for w in works])
    assert np.array_equal(pos, np.arange(16384) % 1024)
    assert works[0].T_max == max(w.T for w in works)
    assert works[0].describe()["total_tokens"] == 16384


def test_decode_configurations_are_weak_scaling(bench):
    for cfg, model, layers, experts in ((1, 20, 24, 32), (3, 120, 36, 128)):
        for world in (1, 8):
            w = bench.Work(_args(config=cfg), world, world - 1)
            assert (w.model, w.layers, w.experts, w.T, w.total, w.scaling) == (model, layers, experts, 4096, 4096 * world, "weak")
            p = w.pos_array()
            assert p.shape == (4096,) and p.min() >= 0 and p.max() < 4096
    w0 = bench.Work(_args(config=0), 1, 0)
    assert (w0.fp32, w0.layers, w0.T) == (True, 1, 64) and np.array_equal(w0.pos_array(), np.arange(64))
    # an explicit size overrides the configuration's and makes it per-GPU work
    w = bench.Work(_args(config=2, tokens_per_gpu=512), 4, 1)
    assert (w.T, w.total, w.scaling) == (512, 2048, "weak")


def test_bf16_rounding_of_the_cpu_arm_matches_the_oracle(bench, orc):
    r = np.random.default_rng(4)
    a = (r.standard_normal(100000) * 10.0 ** r.integers(-20, 20, 100000)).astype(np.float32)
    want = (orc.f32_to_bf16(a).astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(bench.bf16_values(a).view(np.uint32), want.view(np.uint32))
