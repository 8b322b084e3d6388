#!/usr/bin/env python
"""Benchmark of the continuous-batching decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads:
  llama3_8b_q4_continuous  (default) BASELINE configuration 3: Llama-3-8B-architecture, Q4 group-64
                           projections, bf16 embeddings / head / norms, 2048 synthetic requests, up to
                           256 concurrent sequences, page 16, 512-token prefill chunks packed with the
                           decode tokens of every live sequence in one ragged batch, greedy.  One
                           independent replica per GPU, requests sharded id mod N, no collective.
  paged_attn_decode        BASELINE configuration 1: paged-attention decode microbenchmark
                           (64 sequences, 32 q / 8 kv heads, head_dim 128, page 16, ctx U[128,4096]).
  qmm                      BASELINE configuration 2: MLX group-64 Q4 / Q8 dequant GEMV / GEMM on the four
                           Llama-3-8B projection shapes at 1, 8, 32, 128 and 256 tokens.
  decode_only              decode iterations without prefill (the weight-streaming regime).
  qwen3_32b_q8_tp          BASELINE configuration 4: one Qwen3-32B-architecture Q8 model over N ranks.
A "step" is one iteration of the serving loop (one ragged forward over one batch).  The engine is
first rolled to its steady state (`ramp` iterations, untimed, all requests available at t = 0), then W
warm-up and K timed iterations follow.  `value` = generated tokens / device time of the K forwards
(CUDA events on the launching stream); `e2e` = the same K iterations by wall clock through the C ABI,
host scheduling and the per-step host<->device copies included.  `--impl reference` times the CPU
restatement of the reference's path (the reference itself is Rust + MLX/Metal and cannot run on this
box) on a bounded sample of the same workload.
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


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernels, from the ncu captures summarised under
# profiles/ (each summary gives the capturing command).
NCU_TRAFFIC = {
    "gemm_gate_up": dict(kernel="gemm_tc_pair_kernel<4,0>", bytes_per_launch=94.1e6, summary="gemm_tc_pair_kernel_q4_2layer_step.md",
                         note="gate+up projection launch (N 28672, K 4096) at ~570 tokens in the 2-layer capture; algorithmic 66.1 MB of packed "
                              "weights + activations/outputs that mostly stay in L2"),
    "paged_attn_decode_config1": dict(kernel="paged_attn_decode_kernel<128>", bytes_per_launch=572.7e6, summary="paged_attn_decode_kernel_config1.md",
                                      note="the configuration-1 batch (algorithmic 565.0 MB)"),
    "gemm_stream_gate_up": dict(kernel="gemm_stream_kernel<4,1,0>", bytes_per_launch=66.2e6, summary="gemm_stream_kernel_decode_only_step.md",
                                note="gate+up projection (28672 x 4096, Q4) at 8 tokens in a decode-only iteration; algorithmic 66.1 MB"),
}


def ncu_traffic(key):
    """Returns (bytes per launch, note) for a dominant kernel, or (None, reason)."""
    e = NCU_TRAFFIC.get(key)
    if not e:
        return None, "no ncu capture recorded for this kernel"
    return float(e["bytes_per_launch"]), f"{e['kernel']}: {e['note']} (summary: profiles/{e['summary']})"


def host_threads():
    """Threads the CPU legs really use: every core this process may run on, set explicitly."""
    from oracle import oracle as orc

    return orc.use_host_cores()


# ------------------------------------------------------------------------------------------------
# BASELINE configuration 3: Llama-3-8B-architecture Q4 continuous batching
def continuous_setup(args, rank, world, local_rank):
    from mlx_llm_b200 import _lib, engine as eng, workloads as wl
    from mlx_llm_b200.replica import replica_requests

    if args.workload == "qwen3_32b_q8_tp":
        return tp_setup(args, rank, world, local_rank)
    shape = dict(wl.LLAMA3_8B if args.layers <= 0 else dict(wl.LLAMA3_8B, num_layers=args.layers))
    ctx = _lib.Context(local_rank)
    cfg = eng.model_config(**shape, quant_bits=4, quant_group=64)
    model = eng.CausalLm.synthetic(ctx, cfg, seed=0)
    # weak scaling: the job is N x `requests` requests, replica r serves the r-th block of them, and every block is
    # the same seeded draw, so that all replicas do identical work and the per-GPU figures are comparable across N
    prompts, outs, arrival = replica_requests(args.requests, rank, world, 50.0, seed=0, vocab=shape["vocab_size"],
                                              poisson=args.arrivals == "poisson")
    reqs = [eng.BatchRequest(p, int(o), arrival_s=float(a)) for p, o, a in zip(prompts, outs, arrival)]
    ccfg = eng.ContinuousConfig(max_batch=args.max_batch, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=args.chunk,
                                max_pages=args.max_pages, max_blocks_per_seq=(8192 + 512) // 16 + 2)
    return ctx, model, reqs, ccfg, shape


def tp_setup(args, rank, world, local_rank):
    """BASELINE configuration 4: ONE Qwen3-32B-architecture Q8 model split over the N ranks by KV heads; every rank
    runs the same schedule on the same 512 requests.  The pool takes what is left of HBM after the weights."""
    from mlx_llm_b200 import _lib, engine as eng, workloads as wl

    shape = dict(wl.QWEN3_32B if args.layers <= 0 else dict(wl.QWEN3_32B, num_layers=args.layers))
    ctx = _lib.Context(local_rank)
    uid = None
    if world > 1:
        import torch
        import torch.distributed as dist

        t = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            t.copy_(torch.frombuffer(bytearray(eng.TpGroup.unique_id()), dtype=torch.uint8))
        dist.broadcast(t, 0)
        uid = bytes(t.cpu().numpy().tobytes())
    tp = eng.TpGroup(ctx, uid, rank, world)
    tp.reduce_path = "none" if world == 1 else "nccl"
    if world > 1 and args.tp_reduce in ("peer", "peer-push"):
        def gather(blob):
            mine = torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda()
            every = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            return [bytes(e.cpu().numpy().tobytes()) for e in every]

        if tp.enable_peer(args.chunk + 512, shape["hidden_size"], gather):
            tp.reduce_path = "peer memory"
            if args.tp_reduce == "peer-push":
                tp.peer_set_push(True)
                tp.reduce_path = "peer memory, pushed"
    cfg = eng.model_config(**shape, quant_bits=8, quant_group=64)
    model = eng.CausalLm.synthetic(ctx, cfg, seed=0, tp=tp)
    model._tp = tp  # the model points at its group: keep it alive
    prompts, outs, arrival = wl.long_context_requests(n=args.requests if args.requests != 2048 else 512, seed=0, vocab=shape["vocab_size"])
    reqs = [eng.BatchRequest(p, int(o), arrival_s=0.0) for p, o in zip(prompts, outs)]
    page_bytes = shape["num_layers"] * 2 * (shape["num_kv_heads"] // world) * 16 * shape["head_dim"] * 2
    free, _ = ctx.mem_info()
    max_pages = args.max_pages if args.max_pages != 49152 else int((free - (12 << 30)) // page_bytes)
    ccfg = eng.ContinuousConfig(max_batch=512, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=args.chunk,
                                max_pages=max_pages, max_blocks_per_seq=(32768 + 256 + args.chunk) // 16 + 2)
    return ctx, model, reqs, ccfg, shape


def run_continuous(args, rank, world, local_rank, barrier, reduce_max, reduce_sum):
    from mlx_llm_b200 import engine as eng, workloads as wl

    ctx, model, reqs, ccfg, shape = continuous_setup(args, rank, world, local_rank)
    engine = eng.ContinuousEngine(model, reqs, ccfg)
    done, st = engine.step(args.ramp)                 # untimed roll to the steady state
    warm = max(args.warmup, 3)
    done, st = engine.step(warm)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    s0 = st
    if args.profiler_range:
        ctx.profiler_range(True)
    t0 = time.perf_counter()
    seg_ms, prev, left = [], s0, args.steps   # exactly K iterations, read out in four consecutive parts
    for part in range(4):
        k = left // (4 - part)
        left -= k
        if k == 0:
            continue
        done, s1 = engine.step(k)
        if s1["steps"] > prev["steps"]:
            seg_ms.append((s1["device_ms"] - prev["device_ms"]) / (s1["steps"] - prev["steps"]))
        prev = s1
    ctx.sync()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if args.profiler_range:
        ctx.profiler_range(False)
    barrier()
    clocks = sampler.stop()
    steps = s1["steps"] - s0["steps"]
    gen = s1["decode_tokens"] - s0["decode_tokens"]
    pre = s1["prefill_tokens"] - s0["prefill_tokens"]
    dev_ms = s1["device_ms"] - s0["device_ms"]
    launches = s1["kernel_launches"] - s0["kernel_launches"]
    h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) / max(steps, 1)
    d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) / max(steps, 1)
    # per-kernel-class durations over further iterations of the same steady state (CUDA events
    # between the classes on the launching stream)
    eng.profile_enable(ctx, True)
    p0 = engine.step(0)[1]
    done, p1 = engine.step(args.profile_steps)
    prof = eng.profile_read(ctx)
    eng.profile_enable(ctx, False)
    prof_steps = max(p1["steps"] - p0["steps"], 1)
    tp_mode = args.workload == "qwen3_32b_q8_tp"
    # replicas: tokens add up over ranks; tensor parallelism: every rank produced the SAME tokens, count them once
    all_gen, all_dev, all_wall = (gen if tp_mode else reduce_sum(gen)), reduce_max(dev_ms), reduce_max(wall_ms)
    peaks = measured_peaks()
    traffic, traffic_note = (None, None) if tp_mode else ncu_traffic("gemm_gate_up")
    gemm_ms = prof["ms"]["gemm"]
    tfl = prof["gemm_flops"] / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    total_prof_ms = sum(prof["ms"].values())
    dec_ms = prof["ms"]["attn_decode"]
    out = dict(
        metric="continuous-batch decode tok/s, Qwen3-32B-arch Q8, tensor-parallel" if tp_mode else "continuous-batch decode tok/s, Llama-3-8B-arch Q4",
        value=all_gen / (all_dev * 1e-3), unit="tok/s", n_gpus=world,
        steps=int(steps), warmup=warm, ms_per_step=all_dev / max(steps, 1),
        ms_per_step_by_quarter=[round(x, 4) for x in seg_ms], higher_is_better=True, scaling="strong" if tp_mode else "weak",
        vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="qwen3_32b_q8_tp (BASELINE configuration 4)" if tp_mode else "llama3_8b_q4_continuous (BASELINE configuration 3)",
                    layers=shape["num_layers"], requests=len(reqs) if tp_mode else args.requests,
                    arrivals="all at time 0" if tp_mode else args.arrivals, max_batch=ccfg.max_batch, page=16, prefill_chunk=args.chunk,
                    ramp_steps=args.ramp, max_pages=int(ccfg.max_pages), peak_concurrent=int(s1.get("peak_concurrent", 0)),
                    parallelism=(f"tensor-parallel x{world} over KV heads; o_proj / down_proj partial sums (f32) reduced by: "
                                 + {"peer memory": "one kernel over peer memory (loads from every rank, sum + residual add, stores to every rank)",
                                    "peer memory, pushed": "projection epilogues storing each column range into its owner's memory + one kernel (sum + residual add, stores to every rank)",
                                    "nccl": "NCCL all-reduce + residual-add kernel", "none": "nothing (one rank)"}[getattr(model._tp, "reduce_path", "none")]
                                 if tp_mode
                                 else f"replica x{world}: {world} x {args.requests} requests, one block of {args.requests} per replica, no collective"),
                    l2="per-step working set (weights + KV) exceeds L2",
                    prefill_tokens_per_step=pre / max(steps, 1), generated_tokens_per_step=gen / max(steps, 1)),
        roofline=dict(bound="tensor", achieved=tfl, peak=peaks["bf16_tflops_sustained"], unit="TFLOP/s",
                      frac=tfl / peaks["bf16_tflops_sustained"], traffic=traffic, traffic_note=traffic_note, peak_source=peaks["source"] + " (sustained)",
                      kernel=("projection GEMMs (Q8 dequant fused) + bf16 lm_head" if tp_mode else "projection GEMMs (Q4 dequant fused) + bf16 lm_head"), launches_per_step=prof["launches"]["gemm"] / prof_steps,
                      ms_per_step=gemm_ms / prof_steps, share_of_step=gemm_ms / total_prof_ms if total_prof_ms else None,
                      algorithmic_flops_per_step=prof["gemm_flops"] / prof_steps),
        roofline_paged_attn_decode=dict(bound="hbm", achieved=(prof["attn_decode_bytes"] / (dec_ms * 1e-3) / 1e9) if dec_ms > 0 else None,
                                        peak=peaks["hbm_gbs"], unit="GB/s",
                                        frac=(prof["attn_decode_bytes"] / (dec_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if dec_ms > 0 else None,
                                        ms_per_step=dec_ms / prof_steps, algorithmic_bytes_per_step=prof["attn_decode_bytes"] / prof_steps),
        class_ms_per_step={k: v / prof_steps for k, v in prof["ms"].items()},
        e2e=dict(value=all_gen / (all_wall * 1e-3), unit="tok/s", h2d_bytes_per_step=int(h2d), d2h_bytes_per_step=int(d2h)),
        gpu_launches=int(launches), clocks=clocks,
    )
    engine.free()
    model.free()
    return out


def cpu_baseline_continuous(args, seconds=20.0):
    """The CPU restatement of the reference's loop (whole-prompt prefill at admission, batched decode)
    on a bounded sample of the same workload: the same Q4 Llama-3-8B-shape model cut to `cpu_layers`
    layers, `cpu_requests` requests with prompts clipped to 64 tokens and 8 new tokens each."""
    from mlx_llm_b200 import workloads as wl
    from oracle import oracle as orc

    threads = host_threads()
    shape = dict(wl.LLAMA3_8B, num_layers=args.cpu_layers)
    m = orc.Model(layers=shape["num_layers"], hidden=shape["hidden_size"], heads=shape["num_heads"], kv_heads=shape["num_kv_heads"],
                  head_dim=shape["head_dim"], inter=shape["intermediate_size"], vocab=shape["vocab_size"], eps=1e-5, theta=500000.0,
                  rope_kind=1, rope_factor=8.0, rope_low=1.0, rope_high=4.0, rope_orig=8192.0, qk_norm=0, quant_bits=4, group=64, f32_mode=0)
    m.fill_synthetic(0)
    prompts, outs, _ = wl.serving_requests(n=args.cpu_requests, seed=0, vocab=shape["vocab_size"], poisson=False)
    prompts = [p[:64] for p in prompts]
    t0 = time.perf_counter()
    res = m.generate_continuous(prompts, [8] * len(prompts), max_batch=len(prompts), throughput=True)
    dt = time.perf_counter() - t0
    gen = sum(len(t) for t in res["tokens"])
    # scale the layer cut back to the full depth (the per-layer work is identical; embeddings and the
    # head are counted once)
    full = dt * 32.0 / args.cpu_layers
    m.free()
    return dict(value=gen / full, unit="tok/s", cores=threads, kind="port",
                sample=f"{len(prompts)} requests, prompts clipped to 64 tokens, 8 new tokens each, {args.cpu_layers} of 32 layers timed "
                       f"({dt:.1f} s) and scaled to 32 layers", measured_seconds=dt)


# ------------------------------------------------------------------------------------------------
# BASELINE configuration 1: paged-attention decode microbenchmark
def config1_case(n_seqs=64, seed=0):
    from tests import helpers as H

    rng = np.random.default_rng(seed)
    ctx_lens = rng.integers(128, 4097, size=n_seqs)
    return H.make_paged_case(seed, ctx_lens, 32, 8, 128, 16)


def attn_alg_bytes(case):
    """Every cached K and V byte once (the GQA group shares it), q in, out back, block tables."""
    ctx = case["ctx_lens"].astype(np.int64)
    kv = int(ctx.sum()) * case["hkv"] * case["hd"] * 2 * 2
    return kv + 2 * case["q"].nbytes + 4 * int(((ctx + case["page"] - 1) // case["page"]).sum())


def run_paged_attn(args, rank, world, local_rank, barrier, reduce_max, reduce_sum):
    import ctypes as C

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
    if args.profiler_range:
        ctx.profiler_range(True)
    for _ in range(args.steps):
        ctx.flush_l2()
        ctx.timer_start()
        call()
        t_dev += ctx.timer_stop_ms()
    ctx.sync()
    if args.profiler_range:
        ctx.profiler_range(False)
    barrier()
    launches = ctx.launch_count() - l0
    t_dev = reduce_max(t_dev)
    # The same K iterations back to back without the flush: every iteration streams 565 MB out of a 1.1 GB pool, more than
    # four times L2, so nothing of it survives from one iteration to the next; the difference to the flushed figure is what
    # the write-backs of the flush buffer's dirty lines cost the kernel that follows it.
    ctx.timer_start()
    for _ in range(args.steps):
        call()
    t_unflushed = reduce_max(ctx.timer_stop_ms())
    hq, ho = C.c_void_p(), C.c_void_p()
    lib = _lib.load()
    _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(case["q"].nbytes), C.byref(hq)))
    _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(case["q"].nbytes), C.byref(ho)))
    C.memmove(hq, case["q"].ctypes.data, case["q"].nbytes)
    e2e_call = lambda: kernels.paged_attn_decode_host(ctx, hq.value, kp, vp, bt, cl, n, 32, 8, 128, 16, case["scale"], ho.value,
                                                      case["max_blocks"], args.chunk_tokens)
    for _ in range(3):
        e2e_call()
    barrier()
    t_e2e = 0.0
    for _ in range(args.steps):
        ctx.flush_l2()
        ctx.sync()
        t0 = time.perf_counter()
        e2e_call()
        t_e2e += (time.perf_counter() - t0) * 1e3
    t_e2e = reduce_max(t_e2e)
    clocks = sampler.stop()
    barrier()
    alg, peaks = attn_alg_bytes(case), measured_peaks()
    ms = t_dev / args.steps
    gbs = alg / (ms * 1e-3) / 1e9
    out = dict(
        metric="paged-attention decode tokens/s (one token per sequence per step)", value=n * world / (ms * 1e-3), unit="tok/s",
        n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="paged_attn_decode (BASELINE configuration 1): 64 seqs, 32q/8kv heads, hd 128, page 16, ctx U[128,4096]",
                    l2="flushed between timed iterations", parallelism=f"replica x{world}", chunk_tokens=args.chunk_tokens or 512),
        roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"],
                      traffic=ncu_traffic("paged_attn_decode_config1")[0], traffic_note=ncu_traffic("paged_attn_decode_config1")[1],
                      peak_source=peaks["source"], algorithmic_bytes=alg, kernel="paged_attn_decode_kernel<128> (work list and merge inside: one launch)",
                      unflushed=dict(ms_per_step=t_unflushed / args.steps, achieved=alg / (t_unflushed / args.steps * 1e-3) / 1e9,
                                     frac=alg / (t_unflushed / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                     note="the same iterations back to back, no flush: the inputs (565 MB of a 1.1 GB pool per iteration) exceed L2")),
        e2e=dict(value=n * world / (t_e2e / args.steps * 1e-3), unit="tok/s", h2d_bytes_per_step=case["q"].nbytes,
                 d2h_bytes_per_step=case["q"].nbytes),
        gpu_launches=int(launches), clocks=clocks,
    )
    if rank == 0 and world == 1 and args.cpu_baseline:
        out["cpu_baseline"] = cpu_baseline_paged_attn(case)
    return out


# ------------------------------------------------------------------------------------------------
# BASELINE configuration 2: group-64 affine Q4 / Q8 dequant GEMV / GEMM (QuantizedLinear::forward, quant.rs:56-70)
QMM_SHAPES = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]   # out x in
QMM_TOKENS = [1, 8, 32, 128, 256]


def qmm_case(n, k, bits, seed=0):
    rng = np.random.default_rng(seed + 7 * bits + n + k)
    packed = rng.integers(0, 2**32, size=(n, k * bits // 32), dtype=np.uint32)
    from tests import helpers as H

    scales = H.f32_to_bf16_np(np.abs(rng.standard_normal((n, k // 64)).astype(np.float32) * 0.02) / 7.5)
    biases = H.f32_to_bf16_np(-8.0 * H.bf16_to_f32_np(scales) + rng.standard_normal((n, k // 64)).astype(np.float32) * 1e-3)
    x = H.f32_to_bf16_np(rng.standard_normal((max(QMM_TOKENS), k)).astype(np.float32))
    return packed, scales, biases, x


def qmm_alg_bytes(n, k, bits, m):
    return n * k * bits // 8 + n * (k // 64) * 4 + m * k * 2 + m * n * 2


def run_qmm(args, rank, world, local_rank, barrier, reduce_max, reduce_sum):
    """One step = one pass over all 40 (shape, bits, tokens) cases, L2 flushed before every call, each call timed with
    CUDA events on the launching stream.  The headline value is the weight-streaming rate of the small-token cases
    (algorithmic bytes of all cases with <= 32 tokens / their summed time); every case is listed under `cases` with its
    own GB/s (HBM bound) and TFLOP/s (tensor bound)."""
    import ctypes as C

    from mlx_llm_b200 import _lib, kernels

    ctx = _lib.Context(local_rank)
    lib = _lib.load()
    peaks = measured_peaks()
    cases = []
    only = [tuple(int(v) for v in item.split("x")) for item in args.qmm_only.split(",") if item]   # e.g. "14336x4096x4x1"
    for bits in (4, 8):
        for n, k in QMM_SHAPES:
            if only and not any(o[:3] == (n, k, bits) for o in only):
                continue
            packed, scales, biases, x = qmm_case(n, k, bits)
            dev = dict(p=ctx.buf(packed), s=ctx.buf(scales), b=ctx.buf(biases), x=ctx.buf(x), y=ctx.empty((max(QMM_TOKENS), n), np.uint16))
            hx, hy = C.c_void_p(), C.c_void_p()
            _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(x.nbytes), C.byref(hx)))
            _lib.check(lib.b2_host_alloc_pinned(C.c_size_t(max(QMM_TOKENS) * n * 2), C.byref(hy)))
            C.memmove(hx, x.ctypes.data, x.nbytes)
            for m in QMM_TOKENS:
                if only and (n, k, bits, m) not in only:
                    continue
                cases.append(dict(n=n, k=k, bits=bits, m=m, dev=dev, hx=hx, hy=hy, ms=0.0, e2e_ms=0.0))
    run = lambda c: kernels.qmm(ctx, c["dev"]["x"], c["dev"]["p"], c["dev"]["s"], c["dev"]["b"], c["m"], c["n"], c["k"], c["bits"], c["dev"]["y"], None)
    run_host = lambda c: kernels.qmm_host(ctx, c["hx"].value, c["dev"]["p"], c["dev"]["s"], c["dev"]["b"], c["m"], c["n"], c["k"], c["bits"], c["hy"].value)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        for c in cases:
            run(c)
            run_host(c)
    ctx.sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = ctx.launch_count()
    barrier()
    if args.profiler_range:
        ctx.profiler_range(True)
    for _ in range(args.steps):
        for c in cases:
            ctx.flush_l2()
            ctx.timer_start()
            run(c)
            c["ms"] += ctx.timer_stop_ms()
    ctx.sync()
    if args.profiler_range:
        ctx.profiler_range(False)
    launches = ctx.launch_count() - l0
    barrier()
    for _ in range(args.steps):
        for c in cases:
            ctx.flush_l2()
            ctx.sync()
            t0 = time.perf_counter()
            run_host(c)
            c["e2e_ms"] += (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    barrier()
    rows, small_bytes, small_ms, small_e2e, small_tok, dom = [], 0.0, 0.0, 0.0, 0, None
    for c in cases:
        ms, e2e = c["ms"] / args.steps, c["e2e_ms"] / args.steps
        alg = qmm_alg_bytes(c["n"], c["k"], c["bits"], c["m"])
        gbs, tfl = alg / (ms * 1e-3) / 1e9, 2.0 * c["m"] * c["n"] * c["k"] / (ms * 1e-3) / 1e12
        row = dict(out=c["n"], inp=c["k"], bits=c["bits"], tokens=c["m"], us=round(ms * 1e3, 2), gbs=round(gbs, 1), tflops=round(tfl, 2),
                   frac_hbm=round(gbs / peaks["hbm_gbs"], 4), frac_tensor=round(tfl / peaks["bf16_tflops"], 4), e2e_us=round(e2e * 1e3, 2),
                   algorithmic_bytes=alg)
        rows.append(row)
        if c["m"] <= 32:
            small_bytes += alg
            small_ms += ms
            small_e2e += e2e
            small_tok += c["m"]
        if (c["n"], c["k"], c["bits"], c["m"]) == (14336, 4096, 4, 1) or dom is None:
            dom = row
    total_ms = reduce_max(sum(c["ms"] for c in cases) / args.steps)
    gbs = small_bytes / (reduce_max(small_ms) * 1e-3) / 1e9
    traffic, note = ncu_traffic("gemm_stream_gate_up")
    out = dict(
        metric="Q4/Q8 group-64 dequant GEMV weight-streaming GB/s (cases with <= 32 tokens)", value=gbs * world, unit="GB/s", n_gpus=world,
        steps=args.steps, warmup=warm, ms_per_step=total_ms, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload="qmm (BASELINE configuration 2): out x in 4096x4096, 1024x4096, 14336x4096, 4096x14336; Q4 and Q8; 1, 8, 32, 128, 256 tokens",
                    l2="flushed before every call", parallelism=f"replica x{world}"),
        roofline=dict(bound="hbm", achieved=dom["gbs"], peak=peaks["hbm_gbs"], unit="GB/s", frac=dom["gbs"] / peaks["hbm_gbs"], traffic=traffic,
                      traffic_note=note, peak_source=peaks["source"], kernel="gemm_stream_kernel, Q4 14336x4096 at 1 token",
                      algorithmic_bytes=dom["algorithmic_bytes"], us_per_launch=dom["us"]),
        cases=rows,
        e2e=dict(value=small_bytes / (reduce_max(small_e2e) * 1e-3) / 1e9 * world, unit="GB/s",
                 h2d_bytes_per_step=int(sum(c["m"] * c["k"] * 2 for c in cases)), d2h_bytes_per_step=int(sum(c["m"] * c["n"] * 2 for c in cases))),
        gpu_launches=int(launches), clocks=clocks,
    )
    if rank == 0 and world == 1 and args.cpu_baseline:
        out["cpu_baseline"] = cpu_baseline_qmm()
    return out


def cpu_baseline_qmm(seconds=10.0):
    """Oracle quantized matmul (dequantize on the fly, f32 accumulate, OpenMP over output rows) on the cases with
    <= 32 tokens of two shapes, repeated for about ten seconds."""
    from oracle import oracle as orc

    threads = host_threads()
    todo = [(n, k, bits, m) for bits in (4, 8) for n, k in QMM_SHAPES[:2] for m in QMM_TOKENS[:3]]
    data = {(n, k, bits): qmm_case(n, k, bits) for n, k, bits, _ in todo}
    t0, reps, nbytes = time.perf_counter(), 0, 0
    while time.perf_counter() - t0 < seconds:
        for n, k, bits, m in todo:
            packed, scales, biases, x = data[(n, k, bits)]
            orc.qmm(x[:m], packed, scales, biases, 64, bits)
            nbytes += qmm_alg_bytes(n, k, bits, m)
        reps += 1
    dt = time.perf_counter() - t0
    return dict(value=nbytes / dt / 1e9, unit="GB/s", cores=threads, kind="port",
                sample=f"Q4 and Q8, shapes 4096x4096 and 1024x4096, 1 / 8 / 32 tokens, {reps} passes in {dt:.1f} s")


def run_reference_qmm(args, world, threads):
    r = [cpu_baseline_qmm(seconds=4.0) for _ in range(max(1, min(args.steps, 3)))]
    v = float(np.mean([x["value"] for x in r]))
    return dict(impl="reference", metric="Q4/Q8 group-64 dequant GEMV weight-streaming GB/s (cases with <= 32 tokens)", value=v, unit="GB/s",
                n_gpus=world, steps=len(r), warmup=0, ms_per_step=4000.0, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                data="synthetic", config=dict(workload="qmm (BASELINE configuration 2)", parallelism="host cores (OpenMP)",
                                              note="CPU restatement of the reference path; the reference itself (Rust + MLX/Metal) is unavailable on this box"),
                cpu_baseline=dict(value=v, unit="GB/s", cores=threads, kind="port", sample=r[0]["sample"]),
                e2e=dict(value=v, unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)


# ------------------------------------------------------------------------------------------------
# Decode-only iterations (no prefill in the batch): the weight-streaming regime of low-concurrency serving
def run_decode_only(args, rank, world, local_rank, barrier, reduce_max, reduce_sum):
    from mlx_llm_b200 import _lib, engine as eng, workloads as wl

    shape = dict(wl.LLAMA3_8B if args.layers <= 0 else dict(wl.LLAMA3_8B, num_layers=args.layers))
    ctx = _lib.Context(local_rank)
    model = eng.CausalLm.synthetic(ctx, eng.model_config(**shape, quant_bits=4, quant_group=64), seed=0)
    B = args.max_batch if args.max_batch != 256 else 8
    rng = np.random.default_rng(rank)
    warm = max(args.warmup, 3)
    reqs = [eng.BatchRequest(rng.integers(0, 1000, size=32, dtype=np.int32), args.steps + warm + args.profile_steps + 64) for _ in range(B)]
    ccfg = eng.ContinuousConfig(max_batch=B, block_size=16, exactness=eng.THROUGHPUT, prefill_chunk_tokens=args.chunk, max_pages=4096,
                                max_blocks_per_seq=256)
    engine = eng.ContinuousEngine(model, reqs, ccfg)
    done, st = engine.step(8)          # the prompts (one chunk) and a few decode iterations, untimed
    done, st = engine.step(warm)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    if args.profiler_range:
        ctx.profiler_range(True)
    t0 = time.perf_counter()
    done, s1 = engine.step(args.steps)
    ctx.sync()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if args.profiler_range:
        ctx.profiler_range(False)
    barrier()
    clocks = sampler.stop()
    steps = s1["steps"] - st["steps"]
    gen = s1["decode_tokens"] - st["decode_tokens"]
    dev_ms = s1["device_ms"] - st["device_ms"]
    eng.profile_enable(ctx, True)
    p0 = engine.step(0)[1]
    done, p1 = engine.step(args.profile_steps)
    prof = eng.profile_read(ctx)
    eng.profile_enable(ctx, False)
    prof_steps = max(p1["steps"] - p0["steps"], 1)
    all_gen, all_dev, all_wall = reduce_sum(gen), reduce_max(dev_ms), reduce_max(wall_ms)
    peaks = measured_peaks()
    weight_bytes = wl.step_weight_bytes(shape, 4)
    gemm_ms = prof["ms"]["gemm"] / prof_steps
    gbs = weight_bytes / (gemm_ms * 1e-3) / 1e9 if gemm_ms > 0 else 0.0
    out = dict(
        metric="decode-only tok/s, Llama-3-8B-arch Q4", value=all_gen / (all_dev * 1e-3), unit="tok/s", n_gpus=world, steps=int(steps),
        warmup=warm, ms_per_step=all_dev / max(steps, 1), higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=f"llama3_8b_q4 decode-only iterations, {B} sequences per replica", layers=shape["num_layers"], page=16,
                    parallelism=f"replica x{world}", l2="every iteration streams 5 GB of weights, far beyond L2",
                    generated_tokens_per_step=gen / max(steps, 1)),
        roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"], traffic=None,
                      peak_source=peaks["source"], kernel="gemm_stream_kernel (projection weights once per iteration) + bf16 lm_head",
                      algorithmic_bytes_per_step=weight_bytes, ms_per_step=gemm_ms, launches_per_step=prof["launches"]["gemm"] / prof_steps),
        class_ms_per_step={k: v / prof_steps for k, v in prof["ms"].items()},
        e2e=dict(value=all_gen / (all_wall * 1e-3), unit="tok/s", h2d_bytes_per_step=int((s1["h2d_bytes"] - st["h2d_bytes"]) / max(steps, 1)),
                 d2h_bytes_per_step=int((s1["d2h_bytes"] - st["d2h_bytes"]) / max(steps, 1))),
        gpu_launches=int(s1["kernel_launches"] - st["kernel_launches"]), clocks=clocks,
    )
    engine.free()
    model.free()
    return out


def cpu_baseline_paged_attn(case, sample=16, seconds=5.0):
    """Oracle paged attention (f32 accumulate, OpenMP over (sequence, kv head)) on the first `sample`
    sequences of the same batch."""
    from oracle import oracle as orc

    threads = host_threads()
    n = min(sample, case["ctx_lens"].size)
    f = lambda k: orc.paged_attention(case["q"][:k], case["kpool"], case["vpool"], case["block_tables"][:k], None, case["ctx_lens"][:k],
                                      case["scale"], fast_decode=True)
    f(1)
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < seconds:
        f(n)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return dict(value=n / dt, unit="tok/s", cores=threads, kind="port",
                sample=f"first {n} of {case['ctx_lens'].size} sequences of the same batch, {reps} repetitions")


# ------------------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """`--impl reference`: the CPU restatement of the reference path on this box's host cores (rank 0
    only).  Every step is one bounded sample of the same workload."""
    if rank != 0:
        return None
    threads = host_threads()
    if args.workload == "qmm":
        return run_reference_qmm(args, world, threads)
    if args.workload == "paged_attn_decode":
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
        v, metric = n / dt, "paged-attention decode tokens/s (one token per sequence per step)"
        sample = f"each step = first {n} of 64 sequences of the configuration-1 batch"
        wl_name = "paged_attn_decode (BASELINE configuration 1)"
    else:
        steps = max(1, min(args.steps, 3))
        runs = [cpu_baseline_continuous(args) for _ in range(steps)]
        v = float(np.mean([r["value"] for r in runs]))
        dt = float(np.mean([r["measured_seconds"] for r in runs]))
        metric, sample = "continuous-batch decode tok/s, Llama-3-8B-arch Q4", runs[0]["sample"] + f"; {steps} such samples"
        wl_name = "llama3_8b_q4_continuous (BASELINE configuration 3)"
        if args.workload == "decode_only":
            metric, wl_name = "decode-only tok/s, Llama-3-8B-arch Q4", "llama3_8b_q4 decode-only iterations (CPU: the same bounded loop)"
        elif args.workload == "qwen3_32b_q8_tp":
            metric, wl_name = ("continuous-batch decode tok/s, Qwen3-32B-arch Q8, tensor-parallel",
                               "qwen3_32b_q8_tp (BASELINE configuration 4; CPU: the bounded Llama-3-8B-shape sample, the 32B model is not run on CPU)")
        args.steps = steps
    return dict(impl="reference", metric=metric, value=v, unit="tok/s", n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload=wl_name, parallelism="host cores (OpenMP)",
                            note="CPU restatement of the reference path; the reference itself (Rust + MLX/Metal) is unavailable on this box"),
                cpu_baseline=dict(value=v, unit="tok/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=v, unit="tok/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3_8b_q4_continuous", choices=["llama3_8b_q4_continuous", "paged_attn_decode", "qwen3_32b_q8_tp", "decode_only", "qmm"])
    ap.add_argument("--chunk-tokens", dest="chunk_tokens", type=int, default=0, help="paged_attn_decode: split-K chunk")
    ap.add_argument("--requests", type=int, default=2048)
    ap.add_argument("--arrivals", default="saturated", choices=["saturated", "poisson"])
    ap.add_argument("--max-batch", dest="max_batch", type=int, default=256)
    ap.add_argument("--chunk", type=int, default=512, help="prefill chunk tokens per step")
    ap.add_argument("--max-pages", dest="max_pages", type=int, default=49152, help="KV pool pages (2 MiB each for the 8B shape)")
    ap.add_argument("--ramp", type=int, default=400, help="untimed iterations that roll the engine to its steady state")
    ap.add_argument("--profile-steps", dest="profile_steps", type=int, default=20)
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (0 = the full 32); not a valid bench line")
    ap.add_argument("--cpu-layers", dest="cpu_layers", type=int, default=2)
    ap.add_argument("--cpu-requests", dest="cpu_requests", type=int, default=4)
    ap.add_argument("--tp-reduce", dest="tp_reduce", default="peer", choices=["peer", "peer-push", "nccl"],
                    help="qwen3_32b_q8_tp: the reduction after o_proj / down_proj (peer falls back to nccl when a region cannot be mapped)")
    ap.add_argument("--profiler-range", dest="profiler_range", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for `ncu --profile-from-start off`)")
    ap.add_argument("--qmm-only", dest="qmm_only", default="", help="qmm: comma-separated OUTxINxBITSxTOKENS cases to run (profiling); not a valid bench line")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0

    from mlx_llm_b200.replica import ReplicaGroup

    group = ReplicaGroup()
    barrier, reduce_max, reduce_sum = group.barrier, group.reduce_max, group.reduce_sum

    if args.workload == "paged_attn_decode":
        out = run_paged_attn(args, rank, world, local_rank, barrier, reduce_max, reduce_sum)
    elif args.workload == "qmm":
        out = run_qmm(args, rank, world, local_rank, barrier, reduce_max, reduce_sum)
    elif args.workload == "decode_only":
        out = run_decode_only(args, rank, world, local_rank, barrier, reduce_max, reduce_sum)
    else:
        out = run_continuous(args, rank, world, local_rank, barrier, reduce_max, reduce_sum)
        if rank == 0 and world == 1 and args.cpu_baseline:   # a reported baseline, timed at N = 1 only
            out["cpu_baseline"] = cpu_baseline_continuous(args)
    if rank == 0:
        print(json.dumps(out), flush=True)
    group.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
