"""Batch-sharded replicas: one process per GPU, no collective on the data path.

tfjs has no distributed runtime; its Engine is a per-process singleton with one
active backend (tfjs-core/src/engine.ts:168-186), so several GPUs means several
processes (or Node workers), each with its own backend instance bound to one
device, each taking a contiguous slice of the batch; results are gathered on the
host.  This module holds that host logic: rank discovery from the torchrun
environment, the batch split, and the host-side barrier / max / gather used for
timing and for collecting outputs.  The process group is gloo (CPU): nothing
crosses NVLink and NCCL is not involved.
"""
import os

import numpy as np


def shard_range(total, world, rank):
    """Contiguous ceil(total / world) slices; trailing ranks may get fewer (or no)
    units."""
    per = -(-total // world)
    lo = min(rank * per, total)
    return lo, min(lo + per, total)


def bind_to_gpu_cpus(device_ordinal):
    """Pins this process to the CPU cores that share a NUMA node with its GPU, before any
    pinned host memory is allocated, so that a replica's staging buffers and its
    host-to-device copies stay on the GPU's own socket (with eight replicas on a
    two-socket host, half of them would otherwise cross the inter-socket link).  Uses
    NVML's read-only affinity query; returns the chosen cores, or None when NVML or the
    query is unavailable or none of those cores is usable by this process (a container
    confined to one socket)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(int(device_ordinal))
        allowed = os.sched_getaffinity(0)
        words = (max(allowed) // 64) + 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        near = set(i * 64 + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1)
        cores = sorted(near & allowed)
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None


def sharded_execute(engine, build_model, feeds, output, group, replay=False):
    """One model call on a batch split over the group's replicas, the way the path is
    meant to span GPUs: rank r takes the contiguous ceil(B / world) slice
    `shard_range(B, world, r)` of every input (axis 0), builds the model for that many
    units (`build_model(units) -> (model_json, weight_bytes)`; every replica holds its own
    copy of the weights), executes it on its own backend, reads the result back and rank 0
    concatenates the slices in rank order (None on the other ranks).  No device-to-device
    traffic: each Engine has one backend, and tensors move between backends through the
    host (tfjs-core/src/engine.ts:424-439)."""
    from .graph_model import GraphModel
    total = int(next(iter(feeds.values())).shape[0])
    lo, hi = shard_range(total, group.world, group.rank)
    if hi == lo:
        return group.gather_to_root(np.zeros((0,), np.float32))
    model_json, weights = build_model(hi - lo)
    gm = GraphModel(model_json, weights, engine, replay=replay)
    ins = {}
    try:
        for name, v in feeds.items():
            part = np.ascontiguousarray(v[lo:hi])
            ins[name] = engine.make_tensor(part, list(part.shape),
                                           "int32" if part.dtype == np.int32 else "float32")
        y = gm.execute(ins, [output])[0]
        local = y.arraySync()
        y.dispose()
    finally:
        for t in ins.values():
            t.dispose()
        gm.dispose()
    return group.gather_to_root(local)


class ReplicaGroup(object):
    def __init__(self, rank=None, world=None):
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        self._dist = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            import torch.distributed as dist
            if not dist.is_initialized():
                dist.init_process_group("gloo", rank=self.rank, world_size=self.world)
            self._dist = dist

    def barrier(self):
        if self._dist is not None:
            self._dist.barrier()

    def max_over_ranks(self, value):
        if self._dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX)
        return float(t[0])

    def sum_over_ranks(self, value):
        if self._dist is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64)
        self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM)
        return float(t[0])

    def gather_to_root(self, array):
        """Concatenates per-rank host arrays along axis 0 on rank 0 (None elsewhere)."""
        if self._dist is None:
            return np.asarray(array)
        parts = [None] * self.world if self.rank == 0 else None
        self._dist.gather_object(np.asarray(array), parts, dst=0)
        if self.rank != 0:
            return None
        return np.concatenate([p for p in parts if p.shape[0] > 0], axis=0)

    def close(self):
        if self._dist is not None and self._dist.is_initialized():
            self._dist.barrier()
            self._dist.destroy_process_group()
            self._dist = None
