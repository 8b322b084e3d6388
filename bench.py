#!/usr/bin/env python
"""Benchmark of the continuous-batching decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads:
  paged_attn_decode      BASELINE configuration 1: paged-attention decode microbenchmark
                         (64 sequences, 32 q / 8 kv heads, head_dim 128, page 16, ctx U[128,4096]).
A "step" is one pass of the hot path over one synthetic batch.  `value` is timed on the device with
inputs resident in HBM; `e2e` goes through the C ABI with HOST buffers (copies inside the timed
region).  `--impl reference` times the CPU restatement of the reference's path (the reference itself
is Rust + MLX/Metal and cannot run on this box) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


# ------------------------------------------------------------------------------------------------
def config1_case(n_seqs=64, seed=0):
    from tests import helpers as H

    rng = np.random.default_rng(seed)
    ctx_lens = rng.integers(128, 4097, size=n_seqs)
    return H.make_paged_case(seed, ctx_lens, 32, 8, 128, 16)


def attn_alg_bytes(case):
    """Algorithmic bytes of one decode-attention pass: every cached K and V byte once (the GQA group
    shares it), q in, out back, block tables."""
    ctx = case["ctx_lens"].astype(np.int64)
    kv = int(ctx.sum()) * case["hkv"] * case["hd"] * 2 * 2
    return kv + 2 * case["q"].nbytes + 4 * int(((ctx + case["page"] - 1) // case["page"]).sum())


def run_paged_attn(args, rank, world, local_rank, barrier, reduce_max):
    from mlx_llm_b200 import _lib, kernels

    ctx = _lib.Context(local_rank)
    case = config1_case()
    kp, vp = ctx.buf(case["kpool"]), ctx.buf(case["vpool"])
    bt, cl, q = ctx.buf(case["block_tables"]), ctx.buf(case["ctx_lens"]), ctx.buf(case["q"])
    o = ctx.empty(case["q"].shape, np.uint16)
    n = case["ctx_lens"].size
    call = lambda: kernels.paged_attn_decode(ctx, q, kp, vp, bt, cl, n, 32, 8, 128, 16, case["scale"], o, case["max_blocks"],
                                             args.chunk_tokens)
    for _ in range(max(args.warmup, 3)):
        call()
    ctx.sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ctx.launch_count()
    barrier()
    t_dev = 0.0
    for _ in range(args.steps):
        ctx.flush_l2()
        ctx.timer_start()
        call()
        t_dev += ctx.timer_stop_ms()
    ctx.sync()
    barrier()
    launches = ctx.launch_count() - l0
    t_dev = reduce_max(t_dev)
    # e2e: host q in, host out back, through the host-buffer entry point
    import ctypes as C
    hq = C.c_void_p(); ho = C.c_void_p()
    lib = _lib.load()
    _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(case["q"].nbytes), C.byref(hq)))
    _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(case["q"].nbytes), C.byref(ho)))
    C.memmove(hq, case["q"].ctypes.data, case["q"].nbytes)
    e2e_call = lambda: kernels.paged_attn_decode_host(ctx, hq.value, kp, vp, bt, cl, n, 32, 8, 128, 16, case["scale"], ho.value,
                                                      case["max_blocks"], args.chunk_tokens)
    for _ in range(3):
        e2e_call()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ctx.flush_l2()
        e2e_call()
    ctx.sync()
    t_e2e = reduce_max((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop()
    barrier()

    alg = attn_alg_bytes(case)
    peaks = measured_peaks()
    ms = t_dev / args.steps
    gbs = alg / (ms * 1e-3) / 1e9
    toks = n * world / (ms * 1e-3)
    out = dict(
        metric="paged-attention decode tokens/s (one token per sequence per step)", value=toks, unit="tok/s", n_gpus=world,
        steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
        dtype="bf16", data="synthetic",
        config=dict(workload="paged_attn_decode (BASELINE configuration 1): 64 seqs, 32q/8kv heads, hd 128, page 16, ctx U[128,4096]",
                    l2="flushed between timed iterations", parallelism=f"replica x{world}", chunk_tokens=args.chunk_tokens),
        roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"], traffic=None,
                      peak_source=peaks["source"], algorithmic_bytes=alg, kernel="paged_attn_decode_kernel<128> (+worklist, merge)"),
        e2e=dict(value=n * world / (t_e2e / args.steps * 1e-3), unit="tok/s", h2d_bytes_per_step=case["q"].nbytes,
                 d2h_bytes_per_step=case["q"].nbytes),
        gpu_launches=int(launches), clocks=clocks,
    )
    if rank == 0:
        out["cpu_baseline"] = cpu_baseline_paged_attn(case)
    return out


def cpu_baseline_paged_attn(case, sample=16):
    """Oracle paged attention (f32 accumulate, OpenMP over (sequence, kv head)) on the first `sample`
    sequences of the same batch."""
    from oracle import oracle as orc

    sub = dict(case)
    n = min(sample, case["ctx_lens"].size)
    orc.paged_attention(case["q"][:1], case["kpool"], case["vpool"], case["block_tables"][:1], None, case["ctx_lens"][:1],
                        case["scale"], fast_decode=True)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 5.0:
        orc.paged_attention(case["q"][:n], case["kpool"], case["vpool"], case["block_tables"][:n], None, case["ctx_lens"][:n],
                            case["scale"], fast_decode=True)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return dict(value=n / dt, unit="tok/s", cores=os.cpu_count(), kind="port",
                sample=f"first {n} of {case['ctx_lens'].size} sequences of the same batch, {reps} repetitions")


def run_reference(args, rank, world):
    """CPU restatement of the reference path on this box's host cores (rank 0 only)."""
    if rank != 0:
        return None
    case = config1_case()
    from oracle import oracle as orc

    n = 16
    f = lambda: orc.paged_attention(case["q"][:n], case["kpool"], case["vpool"], case["block_tables"][:n], None,
                                    case["ctx_lens"][:n], case["scale"], fast_decode=True)
    for _ in range(max(1, min(args.warmup, 3))):
        f()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        f()
    dt = (time.perf_counter() - t0) / args.steps
    v = n / dt
    sample = f"each step = first {n} of 64 sequences of the configuration-1 batch"
    return dict(impl="reference", metric="paged-attention decode tokens/s (one token per sequence per step)", value=v, unit="tok/s",
                n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload="paged_attn_decode (BASELINE configuration 1)", parallelism="cpu"),
                cpu_baseline=dict(value=v, unit="tok/s", cores=os.cpu_count(), kind="port", sample=sample),
                e2e=dict(value=v, unit="tok/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="paged_attn_decode")
    ap.add_argument("--chunk-tokens", dest="chunk_tokens", type=int, default=0)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0

    barrier = lambda: None
    reduce_max = lambda x: x
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

        def barrier():
            dist.barrier()
            torch.cuda.synchronize()

        def reduce_max(x):
            t = torch.tensor([float(x)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

    out = run_paged_attn(args, rank, world, local_rank, barrier, reduce_max)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
