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
