"""The multi-GPU path without GPUs: two gloo ranks on the CPU.

The path shards with no exchange step, so what has to hold across ranks is bookkeeping:
every rank owns a contiguous range of whole sequences, the ranges tile the batch, a shard
computed alone equals the same rows computed inside the whole batch (rows are independent),
and the job's throughput is total tokens over the slowest rank's time."""
from __future__ import annotations

import importlib
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

PKG = "optimize_inference_gpt-oss_b200"


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = importlib.import_module(PKG + ".sharding")
        import oracle
        orc = oracle.Oracle()
        # prefill-shaped batch: 8 sequences of 16 positions, 32 experts, small hidden size
        T, seq, H, E = 128, 16, 256, 32
        rng = np.random.default_rng(7)  # same seed on every rank: everybody could build the whole batch
        x = rng.standard_normal((T, H)).astype(np.float32)
        d = rng.standard_normal((T, H)).astype(np.float32)
        g = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        scores = rng.standard_normal((T, E)).astype(np.float32)
        b, e = sh.shard_range(T, world, rank, granule=seq)
        assert b % seq == 0 and e % seq == 0
        x_s, n_s = orc.add_rmsnorm_rows(x[b:e], d[b:e], g)
        w_s, e_s = orc.router_rows(scores[b:e], 4)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), b=b, e=e, x=x_s, n=n_s, w=w_s, idx=e_s)
        # the bench's bookkeeping: slowest rank's time, total tokens
        t = sh.max_over_ranks(1.0 + rank, dist)
        total = sh.sum_over_ranks(e - b, dist)
        assert t == float(world) and total == T
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_tile_the_batch_and_agree_with_the_whole(tmp_path, orc):
    import torch.multiprocessing as mp
    world, port = 2, 29611 + os.getpid() % 200
    mp.start_processes(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    T, H, E = 128, 256, 32
    rng = np.random.default_rng(7)
    x = rng.standard_normal((T, H)).astype(np.float32)
    d = rng.standard_normal((T, H)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    scores = rng.standard_normal((T, E)).astype(np.float32)
    x_all, n_all = orc.add_rmsnorm_rows(x, d, g)
    w_all, e_all = orc.router_rows(scores, 4)
    covered = 0
    for r in range(world):
        z = np.load(tmp_path / f"rank{r}.npz")
        b, e = int(z["b"]), int(z["e"])
        assert b == covered
        covered = e
        assert np.array_equal(z["x"], x_all[b:e]) and np.array_equal(z["n"], n_all[b:e])
        assert np.array_equal(z["idx"], e_all[b:e]) and np.array_equal(z["w"], w_all[b:e])
    assert covered == T


def test_reference_arm_runs_on_rank_zero_only():
    """bench.py --impl reference under a 2-rank launch: rank 1 exits 0 without output."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "1"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_reference_arm_prints_the_contract_line():
    import json
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                        "--warmup", "1", "--tokens-per-gpu", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["steps"] == 2 and line["n_gpus"] == 1
