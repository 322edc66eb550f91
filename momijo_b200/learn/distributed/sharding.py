"""Sharding helpers and ``ZeroStage1`` (legacy/src/momijo/learn/distributed/sharding.mojo:41-240).

``partition_1d(total, world, rank)`` is balanced: the first ``total % world`` ranks get one extra
element, offset ``rank*base + min(rank, rem)`` (sharding.mojo:69-85). ``ZeroStage1`` shards the
optimizer state; ``ShardedDataParallel`` (``momijo_b200.parallel.zero``) is the stage 1-3 engine
on flat buffers with the fused peer-memory kernels.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import List

import torch

from . import collective as C


@dataclass
class ShardRange:
    start: int = 0
    end: int = 0

    def size(self) -> int:
        return max(0, self.end - self.start)

    def contains(self, i: int) -> bool:
        return self.start <= i < self.end

    def length(self) -> int:
        return self.end - self.start

    def clamp_index(self, idx: int) -> int:
        """``idx`` moved into [start, end] (the end itself is allowed)."""
        return min(max(idx, self.start), self.end)

    def __str__(self):
        return f"[{self.start},{self.end})"


def partition_1d(total: int, world: int, rank: int) -> ShardRange:
    if world <= 0 or not (0 <= rank < world) or total < 0:
        return ShardRange(0, 0)
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return ShardRange(start, start + base + (1 if rank < rem else 0))


class ZeroStage1:
    """Optimizer-state sharding over a flat parameter list."""

    def __init__(self, world_size: int | None = None, rank: int | None = None, optimizer=None):
        self.world_size = C.get_world_size() if world_size is None else world_size
        self.rank = C.get_rank() if rank is None else rank
        self.optimizer = optimizer

    def shard_range(self, total: int) -> ShardRange:
        return partition_1d(total, self.world_size, self.rank)

    def shard_index(self, length: int) -> ShardRange:
        return partition_1d(length, self.world_size, self.rank)

    def shard_list_i32(self, xs: List[int]) -> List[int]:
        r = self.shard_index(len(xs))
        return [int(v) for v in xs[r.start:r.end]]

    def shard_list(self, xs: List):
        r = self.shard_range(len(xs))
        return list(xs[r.start:r.end])

    def allgather_list(self, local: List[float], total_len: int) -> List[float]:
        """Every rank contributes its shard; returns the full list."""
        buf = torch.zeros(total_len, dtype=torch.float64)
        r = self.shard_range(total_len)
        buf[r.start:r.end] = torch.tensor(local, dtype=torch.float64)
        if C.is_distributed():
            buf = C.allreduce(buf)  # disjoint shards: the sum is the concatenation
        C.barrier()
        return buf.tolist()

    def allgather_list_i32(self, local: List[int], total_len: int) -> List[int]:
        return [int(v) for v in self.allgather_list([float(v) for v in local], total_len)]

    def reduce_scatter_list(self, full: List[float]) -> List[float]:
        t = torch.tensor(full, dtype=torch.float64)
        if C.is_distributed():
            t = C.allreduce(t)
        r = self.shard_range(len(full))
        return t[r.start:r.end].tolist()

    def step_sharded(self, *args, **kw):
        if self.optimizer is not None:
            return self.optimizer.step(*args, **kw)

    def zero_grad_sharded(self):
        if self.optimizer is not None and hasattr(self.optimizer, "zero_grad"):
            self.optimizer.zero_grad()

    def state_dict(self) -> str:
        return json.dumps({"world_size": self.world_size, "rank": self.rank}, separators=(",", ":"))

    def load_state_dict(self, s: str) -> bool:
        try:
            d = json.loads(s)
            self.world_size, self.rank = int(d["world_size"]), int(d["rank"])
            return True
        except Exception:
            return False

    # tensor adapters
    def shard_tensor(self, t: torch.Tensor) -> torch.Tensor:
        r = self.shard_range(t.numel())
        return t.reshape(-1)[r.start:r.end]

    def allgather_tensor(self, shard: torch.Tensor, total_len: int) -> torch.Tensor:
        buf = torch.zeros(total_len, dtype=shard.dtype, device=shard.device)
        r = self.shard_range(total_len)
        buf[r.start:r.end] = shard
        return C.allreduce(buf) if C.is_distributed() else buf

    def reduce_scatter_tensor(self, grads_full: torch.Tensor) -> torch.Tensor:
        """Sum ``grads_full`` over ranks and keep this rank's shard."""
        flat = grads_full.reshape(-1)
        total = C.allreduce(flat.clone()) if C.is_distributed() else flat
        r = self.shard_range(flat.numel())
        return total[r.start:r.end]

    # names of the reference's 1-D adapters (legacy/src/momijo/learn/distributed/sharding.mojo:225-240)
    shard_tensor_f64 = shard_tensor
    allgather_tensor_f64 = allgather_tensor
    reduce_scatter_tensor_f64 = reduce_scatter_tensor


def shard_tensor_f64(zero: ZeroStage1, t: torch.Tensor) -> torch.Tensor:
    return zero.shard_tensor(t)


def allgather_tensor_f64(zero: ZeroStage1, shard: torch.Tensor, total_len: int) -> torch.Tensor:
    return zero.allgather_tensor(shard, total_len)


def reduce_scatter_tensor_f64(zero: ZeroStage1, grads_full: torch.Tensor) -> torch.Tensor:
    return zero.reduce_scatter_tensor(grads_full)
