#!/usr/bin/env python
"""Benchmark of the fused-kernel layer chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one decode step of the gpt-oss-20b chain (embedding gather, first norm,
24 x [qkv bias + RoPE, residual add + RMSNorm, router top-4 + softmax, SwiGLU, expert
combine + residual + next norm], greedy argmax over the vocabulary) for 4096 tokens per
GPU in bf16-activation mode, with seeded synthetic tensors of the real shapes standing in
for the GEMM and attention outputs.  Rank 0 prints one JSON line:

  value       tokens/s over all GPUs, inputs resident in HBM, K CUDA-graph replays timed
              with CUDA events on the launching stream, max over ranks
  e2e         the same through the engine-step call (gptoss_chain_step): token ids and
              positions copied from pinned host memory and the picked tokens copied back
              inside the timed region every step (what the reference engine moves per
              step, gpu_engine.hpp:781-798), wall clock, max over ranks
  roofline    the dominant kernel: algorithmic bytes per launch / mean launch time (CUDA
              events on the launching stream around that kernel's launches of a step, one
              per layer, each on its own layer's tensors), against the measured HBM copy peak
  kernels     the same for every kernel kind
  cpu_baseline  the reference's CPU code (OpenMP over tokens, all host threads) on a
              bounded sample of the same workload; rank 0 at N = 1 only

--impl reference times only that CPU implementation, on the same config.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "optimize_inference_gpt-oss_b200"

FALLBACK_HBM_GBS = 6650.0  # an earlier measurement on this pool, used only without MEASURED_PEAKS.json


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", type=int, default=20, choices=[20, 120])
    ap.add_argument("--tokens-per-gpu", type=int, default=4096)
    ap.add_argument("--standin-sets", type=int, default=0, help="distinct per-layer input sets (0 = one per layer)")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="minimum CPU time of the baseline sample")
    ap.add_argument("--profile-steps", type=int, default=10)
    ap.add_argument("--ncu-steps", type=int, default=0,
                    help="profiler mode: build the chain, run this many steps kernel by kernel, exit (no timing)")
    ap.add_argument("--pdl", action="store_true",
                    help="launch the chain's kernels with programmatic stream serialization (GPTOSS_PDL); "
                         "measured neutral to slightly negative between these kernels, so off by default")
    ap.add_argument("--fp32", action="store_true",
                    help="fp32 mode instead of the headline's bf16-activation mode: fp32 tensors everywhere and the "
                         "CPU program's rounding sequence (GPTOSS_EXACT); twice the bytes")
    ap.add_argument("--split-embed-norm", action="store_true",
                    help="open the step with the reference's two launches (gather, then layer 0's norm) "
                         "instead of the fused one")
    ap.add_argument("--no-host-operands", action="store_true",
                    help="skip the extra e2e leg that re-sends every stand-in tensor from host memory each step")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (profiler mode: smaller footprint)")
    return ap.parse_args()


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


def ncu_traffic(kind: str):
    """DRAM bytes per launch from the committed ncu capture, if one has been taken."""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json"))).get(kind)
    except Exception:
        return None


# ---- clocks ------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
        self.marks = []

    def mark(self):
        self.marks.append(time.time())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "nvidia-smi not available"}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, pw, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in out.splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2])), pw.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "no samples"}
        # under load = the upper half of the samples by power draw (the sampler also sees idle gaps)
        order = np.argsort(pw)
        busy = [sm[i] for i in order[len(order) // 2:]]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": float(max(pw))}


def host_cores() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            pass
    return local_rank


# ---- the CPU implementation (cpu_baseline leg and --impl reference) ----------------------

class CpuChain:
    """The reference's CPU functions looped over a sample of tokens, OpenMP over tokens.

    rmsnorm, compute_cos_sin + apply_rotary_emb, topk + softmax and sample_argmax are the
    reference's own compiled functions when oracle/_ref/libgptoss_ref.so is present; the
    loops that exist only inline in forward() (embedding copy, bias add, SwiGLU, expert
    combine, residual adds) come from the restated oracle, as they do when it is absent."""

    def __init__(self, pkg, model: int, tokens: int, seed: int, sets: int = 2):
        import oracle
        if not os.path.exists(oracle.ORACLE_SO):
            oracle.build(ref=None)
        self.orc = oracle.Oracle()
        self.ref = oracle.Reference() if oracle.have_reference() else None
        self.kind = "reference" if self.ref is not None else "port"
        self.fn = self.ref if self.ref is not None else self.orc
        # every core this process may run on; passed explicitly to each call, because launchers
        # such as torchrun export OMP_NUM_THREADS=1
        self.threads = host_cores()
        c = pkg.chain_config(model, pkg.BF16, 4096)
        self.c, self.T, self.sets = c, tokens, sets
        T, K, H = tokens, c.top_k, c.hidden

        def normal(shape, sid, mean=0.0, sd=1.0):  # bf16 values widened exactly to fp32
            bits = pkg.synth_normal(int(np.prod(shape)), pkg.BF16, seed + 977, sid, mean, sd)
            return pkg.from_bf16_bits(bits).reshape(shape)

        self.vocab_rows = min(c.vocab, 8192)  # the gather only touches the sampled rows
        self.emb = normal((self.vocab_rows, H), 0, 0.0, 0.02)
        self.tokens = pkg.synth_uniform_int(T, seed, 1, 0, self.vocab_rows)
        self.pos = pkg.synth_uniform_int(T, seed, 2, 0, 4096)
        self.gain = (1 + 0.1 * normal((3, H), 3)).astype(np.float32)
        self.bias = normal((c.qkv_dim,), 4, 0.0, 0.02)
        self.proj = [normal((T, H), 10 + s) for s in range(sets)]
        self.qkv = [normal((T, c.qkv_dim), 20 + s) for s in range(sets)]
        self.router = [normal((T, c.n_experts), 30 + s) for s in range(sets)]
        self.mlp1 = [normal((K * T, 2 * c.inter), 40 + s, 0.0, 2.0) for s in range(sets)]
        self.expert = [normal((K * T, H), 50 + s) for s in range(sets)]
        self.logits = normal((T, c.vocab), 60, 0.0, 3.0)
        self.ident = np.arange(T * K, dtype=np.int32).reshape(T, K)

    def step(self):
        c, fn, orc, th = self.c, self.fn, self.orc, self.threads
        x = orc.embed_rows(self.emb, self.tokens, threads=th)
        fn.add_rmsnorm_rows(x, None, self.gain[0], threads=th)
        for l in range(c.n_layers):
            s = l % self.sets
            fn.bias_rope_rows(self.qkv[s], self.bias, self.pos, c.n_q_heads, c.n_kv_heads, c.head_dim, threads=th)
            x, _ = fn.add_rmsnorm_rows(x, self.proj[s], self.gain[1], threads=th)
            w, e = fn.router_rows(self.router[s], c.top_k, threads=th)
            orc.swiglu_rows(self.mlp1[s], c.swiglu_limit, threads=th)
            x = orc.combine_rows(x, self.expert[s], self.ident, w, e, c.n_experts, threads=th)
            fn.add_rmsnorm_rows(x, None, self.gain[2], threads=th)
        return fn.argmax_rows(self.logits, threads=th)

    def describe(self):
        return (f"{self.T} tokens through the whole {self.c.n_layers}-layer chain per pass, fp32 on the host, "
                f"OpenMP over tokens; rmsnorm/rope/top-k/softmax/argmax "
                f"{'are the reference functions compiled from run.cpp (-O3 -fopenmp)' if self.ref else 'from the restated oracle'}"
                f", SwiGLU/combine/bias/residual loops (inline in forward()) from the restated oracle")


def run_cpu(pkg, args, min_seconds: float, steps: int | None, warmup: int):
    """Times the CPU chain.  steps=None: repeat passes until min_seconds have gone by."""
    threads = host_cores()
    tokens = int(min(args.tokens_per_gpu, max(128, 8 * threads)))
    cpu = CpuChain(pkg, args.model, tokens, args.seed)
    for _ in range(max(1, warmup)):
        cpu.step()
    t0 = time.perf_counter()
    n = 0
    while True:
        cpu.step()
        n += 1
        el = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and el >= min_seconds):
            break
    return cpu, n, el


def reference_arm(pkg, args, rank: int):
    if rank != 0:
        return
    cpu, n, el = run_cpu(pkg, args, 0.0, args.steps, args.warmup)
    value = cpu.T * n / el
    line = {
        "impl": "reference", "metric": "layer_chain_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": n, "warmup": args.warmup, "ms_per_step": 1e3 * el / n,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, cpu.c),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cpu.threads, "kind": cpu.kind,
                         "sample": cpu.describe()},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, c):
    return {
        "workload": f"gpt-oss-{args.model}b decode chain: {c.n_layers} layers, {c.n_experts} experts top-{c.top_k}, "
                    f"hidden {c.hidden}, {'fp32 tensors, CPU rounding order' if getattr(args, 'fp32', False) else 'bf16 activations, fp32 residual'}, "
                    f"{args.tokens_per_gpu} tokens per GPU, "
                    f"positions uniform in [0,4096)",
        "tokens_per_gpu": args.tokens_per_gpu, "layers": c.n_layers, "experts": c.n_experts,
        "parallelism": f"dp{args.gpus} (token shards, no collective)",
        "l2": "inputs larger than L2: every layer reads its own seeded tensors, several GB per step",
    }


def host_operand_steps(pkg, chain, c, T, sets, tok, pos, nxt, barrier, sharding, dist, world, steps=3):
    """tokens/s when, besides the token ids, every tensor that stands in for a GEMM or attention
    output (5 per layer, and the logits) is copied from pinned host memory inside the timed
    region, every step.  One layer's worth of tensors is held on the host and sent once per
    layer, so the bytes moved are those of a full step (about 2.4 MB per token); the chain
    then computes on repeated data, which does not change its work.  PCIe-bound by construction:
    in the engine these tensors are produced on the device and never cross the bus."""
    lib = pkg.load()
    kinds = (pkg.BUF_ATTN_PROJ, pkg.BUF_QKV, pkg.BUF_ROUTER, pkg.BUF_MLP1, pkg.BUF_EXPERT)
    K = c.top_k
    rows = {pkg.BUF_ATTN_PROJ: T * c.hidden, pkg.BUF_QKV: T * c.qkv_dim, pkg.BUF_ROUTER: T * c.n_experts,
            pkg.BUF_MLP1: K * T * 2 * c.inter, pkg.BUF_EXPERT: K * T * c.hidden, pkg.BUF_LOGITS: T * c.vocab}
    try:
        host = {w: pkg.PinnedArray(n, np.uint16) for w, n in rows.items()}
    except pkg.GptossError:
        return None
    stream = chain.stream
    for w, h in host.items():  # real data: what the device holds for layer 0
        ptr, _ = chain.buffer(w, 0)
        pkg.check(lib.gptoss_download(h.ptr, ptr, h.array.nbytes, stream))
    pkg.synchronize()
    bytes_per_step = (sum(host[w].array.nbytes for w in kinds) * c.n_layers + host[pkg.BUF_LOGITS].array.nbytes
                      + 8 * T)

    def one_step():
        for layer in range(c.n_layers):
            for w in kinds:
                ptr, _ = chain.buffer(w, layer)
                pkg.check(lib.gptoss_upload(ptr, host[w].ptr, host[w].array.nbytes, stream))
        ptr, _ = chain.buffer(pkg.BUF_LOGITS, 0)
        pkg.check(lib.gptoss_upload(ptr, host[pkg.BUF_LOGITS].ptr, host[pkg.BUF_LOGITS].array.nbytes, stream))
        chain.step(tok.array, pos.array, nxt.array)

    one_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    el = time.perf_counter() - t0
    barrier()
    el = sharding.max_over_ranks(el, dist)
    for h in host.values():
        h.free()
    return {"value": world * T * steps / el, "unit": "tokens/s", "steps": steps,
            "h2d_bytes_per_step": int(bytes_per_step), "d2h_bytes_per_step": 4 * T,
            "ms_per_step": 1e3 * el / steps, "gbs_over_pcie": round(bytes_per_step / (el / steps) / 1e9, 1)}


# ---- our arm -------------------------------------------------------------------------------

def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # launched by hand without torchrun: start one process per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.abspath(__file__), *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))

    pkg = importlib.import_module(PKG)
    pkg.load()

    if args.impl == "reference":
        reference_arm(pkg, args, rank)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert pkg.device_count() > local_rank, "no CUDA device for this rank"
    pkg.set_device(local_rank)
    sharding = importlib.import_module(PKG + ".sharding")

    def barrier():
        pkg.synchronize()
        if dist is not None:
            dist.barrier()
        pkg.synchronize()

    T = args.tokens_per_gpu
    c = pkg.chain_config(args.model, pkg.F32 if args.fp32 else pkg.BF16, 4096)
    if args.vocab > 0:
        c.vocab = args.vocab
    if args.pdl:
        c.flags |= pkg.PDL
    if args.split_embed_norm:
        c.flags |= pkg.CHAIN_SPLIT_EMBED_NORM
    sets = args.standin_sets or c.n_layers
    t_setup = time.perf_counter()
    chain = pkg.Chain(c, T, sets)
    chain.fill_synthetic(T, seed=args.seed + 7919 * rank)
    # this rank's shard of the batch: its own token ids and positions
    tok = pkg.PinnedArray(T, np.int32)
    pos = pkg.PinnedArray(T, np.int32)
    nxt = pkg.PinnedArray(T, np.int32)
    tok.array[:] = pkg.synth_uniform_int(T, args.seed, 100 + rank, 0, c.vocab)
    pos.array[:] = pkg.synth_uniform_int(T, args.seed, 200 + rank, 0, 4096)
    chain.upload(pkg.BUF_TOKENS, 0, tok.array)
    chain.upload(pkg.BUF_POS, 0, pos.array)
    setup_s = time.perf_counter() - t_setup

    if args.ncu_steps > 0:  # launched under ncu: plain launches, nothing timed, nothing printed as a result
        for _ in range(args.ncu_steps):
            chain.enqueue(T, False)
        pkg.synchronize()
        print(json.dumps({"ncu_steps": args.ncu_steps, "launches_per_step": chain.launches_per_step(T),
                          "device_bytes": chain.device_bytes}), flush=True)
        chain.close()
        return

    lib = pkg.load()
    import ctypes as C
    ev = [C.c_void_p(), C.c_void_p()]
    for e in ev:
        pkg.check(lib.gptoss_event_create(C.byref(e)))
    stream = chain.stream

    # ---- value: K graph replays, inputs resident, CUDA events on the launching stream.  Clocks are
    # sampled during exactly this region; a region that saw a thermal or hardware slowdown is
    # measured a second time (once) and the second measurement is the one reported.
    def measure_value():
        sampler = ClockSampler(visible_gpu_index(local_rank)) if rank == 0 else None
        if sampler:
            time.sleep(0.3)  # nvidia-smi needs a moment before its first sample
        for _ in range(max(3, args.warmup)):
            chain.enqueue(T, True)
        barrier()
        pkg.check(lib.gptoss_event_record(ev[0], stream))
        for _ in range(args.steps):
            chain.enqueue(T, True)
        pkg.check(lib.gptoss_event_record(ev[1], stream))
        barrier()
        ms = C.c_float()
        pkg.check(lib.gptoss_event_elapsed_ms(ev[0], ev[1], C.byref(ms)))
        return sharding.max_over_ranks(ms.value, dist), (sampler.stop() if sampler else None)

    SLOW = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    ms_total, clocks = measure_value()
    slowed = 1.0 if (clocks and SLOW & set(clocks.get("reasons", []))) else 0.0
    if sharding.max_over_ranks(slowed, dist) > 0:  # rank 0 decides for everybody
        first = clocks
        ms_total, clocks = measure_value()
        if clocks is not None:
            clocks["remeasured_after"] = first
    ms_per_step = ms_total / args.steps
    value = world * T * args.steps / (ms_total * 1e-3)

    # ---- e2e: the engine-step call with host buffers, wall clock
    for _ in range(3):
        chain.step(tok.array, pos.array, nxt.array)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        chain.step(tok.array, pos.array, nxt.array)
    e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = sharding.max_over_ranks(e2e_s, dist)
    e2e_value = world * T * args.steps / e2e_s
    # ---- the same steps as one wave with the bookkeeping on the GPU: prompts in before, output rows
    # back after, no per-step round trip (one-token prompts, so every step feeds the picked token back)
    wave_steps = min(4 * args.steps, 1024, c.max_pos)  # a wave is long: its set-up and read-back are paid once
    w_tok = np.ascontiguousarray(tok.array, np.int32)
    w_off = np.arange(T + 1, dtype=np.int32)
    w_out = np.empty((T, wave_steps + 2), np.int32)
    w_total, w_ran = C.c_longlong(0), C.c_int(0)

    def wave(steps):
        pkg.check(lib.gptoss_chain_run_wave_on_device(chain.h, w_tok.ctypes.data, w_off.ctypes.data, T, steps,
                                                      w_out.ctypes.data, C.byref(w_total), C.byref(w_ran)))
        return int(w_ran.value)

    wave(min(3, wave_steps))
    barrier()
    t0 = time.perf_counter()
    wave_ran = wave(wave_steps)
    wave_s = sharding.max_over_ranks(time.perf_counter() - t0, dist)
    barrier()
    device_loop = {"value": world * T * wave_ran / wave_s, "unit": "tokens/s", "steps": wave_ran,
                   "ms_per_step": 1e3 * wave_s / max(1, wave_ran), "h2d_bytes": 8 * T + 4,
                   "d2h_bytes": 4 * T * (wave_steps + 2) + 4 * T,
                   "what": "gptoss_chain_run_wave_on_device: one wave of `steps` positions, token feedback and "
                           "finished-row handling by a kernel behind each step, host queues 16 steps at a time"}

    # ---- per-kernel device times: per kind, an event pair around its launches of a step
    prof = chain.profile(T, max(1, min(args.profile_steps, args.steps)), mode=2)

    # ---- the strictest reading of "end to end": every operand of every kernel comes from
    # host memory each step (done last: it overwrites the device-side stand-ins)
    host_operands = None if (args.no_host_operands or args.fp32) else host_operand_steps(pkg, chain, c, T, sets, tok, pos, nxt,
                                                                          barrier, sharding, dist, world)
    peak, peak_src = hbm_peak()
    kernels = {}
    chain_bytes = 0
    for kind, (kms, n) in prof.items():
        if n == 0:
            continue
        per_step = n // max(1, min(args.profile_steps, args.steps))
        b = chain.kernel_bytes(kind, T)
        us = 1e3 * kms / n
        gbs = b / (us * 1e-6) / 1e9
        kernels[kind] = {"launches_per_step": per_step, "us_per_launch": round(us, 3), "bytes_per_launch": b,
                         "achieved_gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
                         "pct_of_nominal_8tbs": round(gbs / 80.0, 1), "share_of_step": None}
        chain_bytes += b * per_step
    tot = sum(k["us_per_launch"] * k["launches_per_step"] for k in kernels.values())
    for k in kernels.values():
        k["share_of_step"] = round(k["us_per_launch"] * k["launches_per_step"] / tot, 4)
    top = max(kernels, key=lambda k: kernels[k]["share_of_step"])
    roofline = {"kernel": top, "bound": "hbm", "achieved": kernels[top]["achieved_gbs"], "peak": peak,
                "unit": "GB/s", "frac": kernels[top]["frac"], "traffic": ncu_traffic(top),
                "peak_source": peak_src,
                "chain": {"bytes_per_step": chain_bytes,
                          "achieved_gbs": round(chain_bytes / (ms_per_step * 1e-3) / 1e9, 1),
                          "frac": round(chain_bytes / (ms_per_step * 1e-3) / 1e9 / peak, 4),
                          "pct_of_nominal_8tbs": round(chain_bytes / (ms_per_step * 1e-3) / 1e9 / 80.0, 1)}}

    line = {
        "metric": "layer_chain_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32" if args.fp32 else "bf16", "data": "synthetic (seeded, host-generated)",
        "config": workload_config(args, c),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 8 * T, "d2h_bytes_per_step": 4 * T,
                "ms_per_step": 1e3 * e2e_s / args.steps,
                "what": "gptoss_chain_step: token ids + positions from pinned host memory in, picked tokens out, "
                        "stream synchronised every step; activations standing in for GEMM outputs stay on the device",
                "device_loop": device_loop, "all_operands_from_host": host_operands},
        "gpu_launches": chain.launches_per_step(T) * args.steps,
        "launches_per_step": chain.launches_per_step(T),
        "roofline": roofline, "kernels": kernels, "clocks": clocks,
        "device": pkg.device_name(local_rank), "device_bytes": chain.device_bytes, "setup_s": round(setup_s, 1),
    }

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, n, el = run_cpu(pkg, args, args.cpu_seconds, None, 1)
        line["cpu_baseline"] = {"value": cpu.T * n / el, "unit": "tokens/s", "cores": cpu.threads, "kind": cpu.kind,
                                "sample": f"{n} passes in {el:.1f} s; " + cpu.describe()}
        # the reference as it ships runs these ops serially per token: the same pass on one thread
        cpu.threads = 1
        t0 = time.perf_counter()
        cpu.step()
        line["cpu_baseline"]["one_thread"] = {"value": cpu.T / (time.perf_counter() - t0), "unit": "tokens/s",
                                              "cores": 1, "sample": "one pass"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    chain.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
