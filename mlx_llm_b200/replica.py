"""Replica data-parallelism: one process per GPU, independent request shards, no data-path collective.

The continuous-batching path shards by REQUEST: every replica serves its own requests with its own weights,
page pool and scheduler, exactly as N independent instances of the reference's `generate_continuous`
(src/decode/continuous.rs:117-229) would.  A request list is cut id mod N (shard_indices); the benchmark gives
every replica the same seeded block of requests (replica_requests) so that per-GPU work does not depend on N.  The only cross-rank traffic is
measurement: a barrier on both sides of a timed region and a max / sum of a few scalars.  The process
group is NCCL when the ranks own GPUs and gloo otherwise (CPU tests of this host logic).
"""
import os

import numpy as np


def shard_indices(n_items, rank, world):
    """Indices of the items replica `rank` owns (item id mod world)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return list(range(rank, n_items, world))


def shard(items, rank, world):
    return [items[i] for i in shard_indices(len(items), rank, world)]


class ReplicaGroup:
    """Rank bookkeeping plus the three collectives the measurement needs.  With world == 1 nothing is
    initialised and every call is the identity."""

    def __init__(self, backend=None, rank=None, world=None, local_rank=None, device_sync=None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
        self.device_sync = device_sync or (lambda: None)
        self.backend = None
        self._dist = None
        self._device = None
        if self.world > 1:
            import torch
            import torch.distributed as dist

            self.backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            if self.backend == "nccl":
                torch.cuda.set_device(self.local_rank)
                self._device = torch.device("cuda", self.local_rank)
                self.device_sync = torch.cuda.synchronize
                if not dist.is_initialized():
                    dist.init_process_group("nccl", device_id=self._device)
            else:
                self._device = torch.device("cpu")
                if not dist.is_initialized():
                    dist.init_process_group(self.backend, rank=self.rank, world_size=self.world)
            self._dist = dist
            self._torch = torch

    def barrier(self):
        """All ranks arrive, then each waits for its own device to drain."""
        if self._dist is not None:
            self._dist.barrier()
        self.device_sync()

    def _reduce(self, x, op):
        if self._dist is None:
            return float(x)
        t = self._torch.tensor([float(x)], device=self._device, dtype=self._torch.float64)
        self._dist.all_reduce(t, op=op)
        return float(t.item())

    def reduce_max(self, x):
        return self._reduce(x, None if self._dist is None else self._dist.ReduceOp.MAX)

    def reduce_sum(self, x):
        return self._reduce(x, None if self._dist is None else self._dist.ReduceOp.SUM)

    def close(self):
        if self._dist is not None and self._dist.is_initialized():
            self._dist.barrier()
            self._dist.destroy_process_group()
            self._dist = None


def whole_job_rate(group, units_this_rank, device_ms_this_rank):
    """Units all ranks processed divided by the slowest rank's device time (units per second)."""
    units = group.reduce_sum(units_this_rank)
    ms = group.reduce_max(device_ms_this_rank)
    return units / (ms * 1e-3) if ms > 0 else 0.0, units, ms


def weak_scaled_requests(requests_per_replica, world, rate_per_replica, **kw):
    """The N-replica workload: N times the requests at N times the arrival rate, so that each replica sees
    the single-GPU workload's statistics.  Returns (prompts, max_new, arrival_s) of ALL replicas."""
    from . import workloads as wl

    return wl.serving_requests(n=requests_per_replica * world, rate=rate_per_replica * world, **kw)


def replica_requests(requests_per_replica, rank, world, rate_per_replica, **kw):
    """Weak scaling with identical work per replica: the N-replica job is N blocks of `requests_per_replica`
    requests, replica r serves block r, and every block is the same seeded draw (same prompts, output budgets and
    arrival times).  Each replica therefore repeats the single-GPU workload exactly, and tokens per iteration do
    not drift with N.  Returns (prompts, max_new, arrival_s) of replica `rank`."""
    from . import workloads as wl

    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return wl.serving_requests(n=requests_per_replica, rate=rate_per_replica, **kw)


class RankLost(RuntimeError):
    """A rank of the group did not announce the step the others are about to launch."""


class StepWatch:
    """Host-side failure detection for ranks that step in lock-step (the tensor-parallel group: every rank launches the
    same forward, whose reductions wait on every other rank).  Before each step a rank announces it in a key-value
    store and looks for every peer's announcement; a peer that has left, crashed or hung on the host is then found
    within `timeout_s` BEFORE anything that would wait for it is launched, and the survivors stop with RankLost between
    steps, with no kernel or collective in flight.  (On the device every such wait is bounded as well -- see
    b2_ctx_set_wait_limit_ms -- but the host check keeps the group from ever entering it.)  The reference has no
    counterpart: it is a single-device program whose only failure path is cooperative cancel
    (src/decode/continuous.rs:138-140, :198-214).

    `store` is a torch.distributed store (TCPStore, FileStore, or the default store of an initialised process group)."""

    def __init__(self, store, rank, world, timeout_s=5.0, poll_s=0.01):
        self.store, self.rank, self.world, self.timeout_s, self.poll_s = store, rank, world, timeout_s, poll_s

    def announce(self, step):
        self.store.set(f"b2/step/{self.rank}", str(int(step)))

    def leave(self):
        """An orderly exit between steps: peers see it at once instead of after the timeout."""
        self.store.set(f"b2/step/{self.rank}", "-1")

    def _peer_step(self, r):
        import datetime

        key = f"b2/step/{r}"
        try:
            self.store.wait([key], datetime.timedelta(seconds=self.poll_s))
        except Exception:  # the key does not exist yet
            return None
        return int(self.store.get(key).decode())

    def ready(self, step):
        """Announce `step`, then return once every peer has announced it too; raise RankLost otherwise."""
        import time

        self.announce(step)
        deadline = time.monotonic() + self.timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                s = self._peer_step(r)
                if s is not None and s < 0:
                    raise RankLost(f"rank {r} left the group before step {step}")
                if s is not None and s >= step:
                    break
                if time.monotonic() > deadline:
                    raise RankLost(f"rank {r} did not announce step {step} within {self.timeout_s} s (last seen: {s})")
                time.sleep(self.poll_s)
