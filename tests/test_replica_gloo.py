"""Host logic of the N-replica path on CPU: two gloo ranks shard one request list, each "serves" its shard
with a deterministic stand-in for the step loop, and the whole-job figures are aggregated the way bench.py
does it (sum of units over ranks / max of the ranks' times).  No GPU, no data-path collective."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from mlx_llm_b200 import replica

    g = replica.ReplicaGroup(backend="gloo")
    prompts, outs, arrival = replica.weak_scaled_requests(8, world, 50.0, seed=0, vocab=1000, max_prompt=64)
    mine = replica.shard_indices(len(prompts), g.rank, world)
    # stand-in for the serving loop: every request "generates" its output budget; rank r takes (r + 1) ms per token
    tokens = int(sum(int(outs[i]) for i in mine))
    ms = tokens * (g.rank + 1.0)
    g.barrier()
    rate, units, slowest = replica.whole_job_rate(g, tokens, ms)
    total_prompt = g.reduce_sum(sum(len(prompts[i]) for i in mine))
    q.put((g.rank, mine, tokens, ms, rate, units, slowest, total_prompt, int(sum(len(p) for p in prompts)), int(outs.sum())))
    g.close()


def test_two_ranks_shard_and_aggregate():
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, idx0, tok0, ms0, rate0, units0, slow0, pr0, all_prompt, all_out), (r1, idx1, tok1, ms1, rate1, units1, slow1, pr1, _, _) = res
    # disjoint cover, id mod world
    assert idx0 == list(range(0, 16, 2)) and idx1 == list(range(1, 16, 2))
    # both ranks hold the same aggregates: sum of units, max of times
    assert units0 == units1 == tok0 + tok1 == all_out
    assert slow0 == slow1 == max(ms0, ms1)
    assert rate0 == rate1 == pytest.approx((tok0 + tok1) / (max(ms0, ms1) * 1e-3))
    assert pr0 == pr1 == all_prompt


def test_single_replica_needs_no_process_group():
    sys.path.insert(0, ROOT)
    from mlx_llm_b200 import replica

    g = replica.ReplicaGroup(rank=0, world=1, local_rank=0)
    g.barrier()
    assert g.reduce_max(3.5) == 3.5 and g.reduce_sum(2) == 2.0
    rate, units, ms = replica.whole_job_rate(g, 100, 50.0)
    assert rate == pytest.approx(2000.0) and units == 100 and ms == 50.0
    assert replica.shard(list("abcdefg"), 1, 3) == ["b", "e"]
    with pytest.raises(ValueError):
        replica.shard_indices(4, 2, 2)
    # weak scaling: N replicas see N times the requests at N times the rate; replica 0's own shard keeps
    # the single-replica statistics (same count, arrival gaps N times shorter in the merged stream)
    p1, o1, a1 = replica.weak_scaled_requests(32, 1, 50.0, seed=0, vocab=100, max_prompt=32)
    p4, o4, a4 = replica.weak_scaled_requests(32, 4, 50.0, seed=0, vocab=100, max_prompt=32)
    assert len(p1) == 32 and len(p4) == 128
    assert np.all(np.diff(a4) >= 0) and a4[-1] / 128 < a1[-1] / 32 * 0.6
    # the benchmark's weak scaling: every replica gets the same seeded block, whatever N
    blocks = [replica.replica_requests(16, r, 4, 50.0, seed=0, vocab=100, max_prompt=32) for r in range(4)]
    one = replica.replica_requests(16, 0, 1, 50.0, seed=0, vocab=100, max_prompt=32)
    for pr, out, arr in blocks:
        assert all(np.array_equal(a, b) for a, b in zip(pr, one[0])) and np.array_equal(out, one[1]) and np.array_equal(arr, one[2])
    with pytest.raises(ValueError):
        replica.replica_requests(16, 4, 4, 50.0)
    g.close()


def test_cpu_legs_take_every_core_they_may_use():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the timed CPU legs must not inherit it."""
    import subprocess

    code = ("import os, sys; sys.path.insert(0, %r); from oracle import oracle as orc; "
            "print(orc.threads(), orc.use_host_cores(), len(os.sched_getaffinity(0)))" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, OMP_NUM_THREADS="1"), capture_output=True, text=True, check=True)
    before, after, cores = (int(x) for x in out.stdout.split())
    assert before == 1 and after == cores


def _tp_worker(rank, world, port, q, die_at, how):
    """A rank of a lock-step group on CPU: every step is announce -> all-reduce (stand-in for the forward's reductions)."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    import datetime

    import torch
    import torch.distributed as dist

    from mlx_llm_b200 import replica

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.TCPStore("127.0.0.1", port + 1, world, rank == 0, timeout=datetime.timedelta(seconds=20))
    watch = replica.StepWatch(store, rank, world, timeout_s=1.5)
    done, err = 0, None
    try:
        for step in range(8):
            if rank == 1 and step == die_at:
                if how == "leave":
                    watch.leave()
                break                                  # "crash": simply stops announcing
            watch.ready(step)                          # nothing that waits on a peer is launched before this returns
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            assert float(t[0]) == sum(range(1, world + 1))
            done += 1
    except replica.RankLost as e:
        err = str(e)
    q.put((rank, done, err))
    # no destroy_process_group: a lost peer would make it wait


@pytest.mark.parametrize("how", ["crash", "leave"])
def test_lost_rank_is_detected_between_steps(how):
    import time

    import torch.multiprocessing as mp

    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    t0 = time.time()
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, q, 3, how)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict((r, (done, err)) for r, done, err in (q.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
    assert res[1] == (3, None)                          # the rank that goes away did three steps
    for r in (0, 2):                                    # the survivors did the same three, then stopped with a typed error,
        done, err = res[r]                              # never entering the fourth step's collective
        assert done == 3 and err is not None and "rank 1" in err and "step 3" in err, res
    assert ("left the group" in res[0][1]) == (how == "leave")
    assert time.time() - t0 < 60
