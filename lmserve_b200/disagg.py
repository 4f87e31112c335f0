"""Host-side plumbing of the multi-GPU cases: rank roles for disaggregated serving, the
descriptor exchange, and the barrier / max-over-ranks used for timing.

There is no collective on the data path.  Under tensor parallelism every rank owns
``num_kv_heads / tp`` heads (``runtime/worker/llm_worker/models/__init__.py:34-37``) and
LMServe sends the same block ids to every rank
(``runtime/src/llm_engine/worker.rs:235-252,434-453``), so cache writes, copy-on-write and
swap are rank-local.  Prefill -> decode transfer is point-to-point, rank i of the prefill
group to rank i of the decode group (``worker.rs:502-515``).  ``torch.distributed`` is used
only to exchange descriptors and to time.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


def kv_heads_per_rank(num_kv_heads: int, tp_size: int) -> int:
    """KV heads a rank owns under tensor parallelism (``models/__init__.py:34-37``)."""
    if tp_size <= 0 or num_kv_heads % tp_size:
        raise ValueError(f"{num_kv_heads} KV heads do not split over {tp_size} ranks")
    return num_kv_heads // tp_size


def transfer_role(rank: int, world: int) -> Tuple[str, Optional[int]]:
    """("prefill", peer) for the first half of the ranks, ("decode", peer) for the second;
    ("none", None) when the world cannot be halved."""
    if world < 2 or world % 2 or not (0 <= rank < world):
        return "none", None
    half = world // 2
    return ("prefill", rank + half) if rank < half else ("decode", rank - half)


def build_push_pairs(block_ids: Sequence[int], remote_block_ids: Sequence[int]) -> np.ndarray:
    """(local src, remote dst) table of a push.  As in ``kv_worker.py:386-387`` surplus
    remote blocks are dropped; fewer remote than local blocks is an error."""
    remote = list(remote_block_ids)[:len(block_ids)]
    if len(remote) != len(block_ids):
        raise ValueError(f"{len(block_ids)} blocks to push but only {len(remote)} reserved on the peer")
    if len(set(remote)) != len(remote):
        raise ValueError("reserved destination blocks must be distinct")
    return np.stack([np.asarray(block_ids, dtype=np.int64).reshape(-1),
                     np.asarray(remote, dtype=np.int64).reshape(-1)], axis=1).reshape(-1, 2)


class Comm:
    """Process-group helper: barrier, max over ranks, object all-gather.  A single process
    needs no group and every method degenerates."""

    def __init__(self, world: int, device: torch.device, rank: Optional[int] = None,
                 backend: Optional[str] = None):
        self.world = world
        self.device = device
        self.dist = None
        if world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            backend = backend or ("nccl" if device.type == "cuda" else "gloo")
            kw = {}
            if rank is not None:
                kw.update(rank=rank, world_size=world)
            if backend == "nccl":
                kw["device_id"] = device
            dist.init_process_group(backend, **kw)
            self.dist = dist

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()

    def max(self, x: float) -> float:
        if self.dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather_objects(self, obj) -> List:
        if self.dist is None:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def close(self) -> None:
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None
