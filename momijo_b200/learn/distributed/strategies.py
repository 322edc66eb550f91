"""``DataParallel`` and ``DistributedDataParallel``
(legacy/src/momijo/learn/distributed/strategies.mojo:51-234).

Method names follow the reference: ``broadcast_parameters``, ``allreduce_gradients``,
``allreduce_tensor``, ``allreduce_tensor_keep``, ``step_and_sync``. Gradients are reduced in
flat buckets; on an NCCL group with a peer-memory communicator the reduction is this library's
two-shot all-reduce kernel over NVLink, otherwise torch.distributed (gloo on CPU).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from . import collective as C


class DataParallel:
    """Single-process helper: split dim 0 into ``min(chunks, n_devices)`` slices (the last takes
    the remainder), run, concatenate (strategies.mojo:97-143)."""

    def __init__(self, model, devices: Optional[List[int]] = None, chunks: Optional[int] = None):
        self._model = model
        self._devices = list(devices) if devices else [0]
        self._chunks = chunks or len(self._devices)

    # accessors in the reference's call form (strategies.mojo:61-78)
    def world_size(self) -> int:
        return max(1, len(self._devices))

    def devices(self) -> List[int]:
        return list(self._devices)

    def chunks(self) -> int:
        return self._chunks

    def set_chunks(self, chunks: int) -> None:
        self._chunks = max(1, int(chunks))

    def model(self):
        return self._model

    def scatter_tensor(self, x: torch.Tensor):
        k = max(1, min(self._chunks, len(self._devices)))
        n = x.shape[0]
        base = n // k
        out, s = [], 0
        for i in range(k):
            e = n if i == k - 1 else s + base
            out.append(x[s:e])
            s = e
        return out

    def gather_tensor(self, outs):
        return torch.cat(list(outs), 0)

    def scatter(self, x):
        return x

    def gather(self, x):
        return x

    def forward(self, x):
        return self.gather_tensor([self._model(c) for c in self.scatter_tensor(x) if c.shape[0]])

    __call__ = forward


class DistributedDataParallel(nn.Module):
    def __init__(self, model: nn.Module, world_size: Optional[int] = None, rank: Optional[int] = None,
                 bucket_mb: float = 64.0, comm=None):
        super().__init__()
        self.module = model
        self._world_size = C.get_world_size() if world_size is None else world_size
        self._rank = C.get_rank() if rank is None else rank
        self.bucket_elems = int(bucket_mb * (1 << 20) / 4)
        self.comm = comm

    # accessors in the reference's call form (strategies.mojo:165-173)
    def model(self):
        return self.module

    def world_size(self) -> int:
        return self._world_size

    def rank(self) -> int:
        return self._rank

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def broadcast_parameters(self, src: int = 0):
        if C.is_distributed():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                C.broadcast(t.data, src)
        C.barrier()

    def _buckets(self):
        cur, n = [], 0
        for p in self.module.parameters():
            if p.grad is None:
                continue
            cur.append(p)
            n += p.numel()
            if n >= self.bucket_elems:
                yield cur
                cur, n = [], 0
        if cur:
            yield cur

    def allreduce_gradients(self, average: bool = True):
        """Bucketed gradient all-reduce."""
        if not C.is_distributed():
            return
        for bucket in self._buckets():
            flat = torch.cat([p.grad.reshape(-1) for p in bucket])
            if self.comm is not None and flat.is_cuda:
                self._peer_allreduce(flat, average)
            else:
                C.allreduce(flat, C.ReduceOp.AVG if average else C.ReduceOp.SUM)
            off = 0
            for p in bucket:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()

    def _peer_allreduce(self, flat, average):
        comm = self.comm
        n = flat.numel()
        unit = 8 * comm.world
        padded = (n + unit - 1) // unit * unit
        if not hasattr(self, "_stage") or self._stage.numel() < padded:
            self._stage = comm.alloc(padded, torch.bfloat16)
        st = self._stage[:padded]
        st[:n].copy_(flat)
        if padded > n:
            st[n:].zero_()
        comm.all_reduce_(st, 1.0 / comm.world if average else 1.0)
        flat.copy_(st[:n])

    def allreduce_tensor(self, t: torch.Tensor):
        return C.allreduce(t, C.ReduceOp.SUM)

    def allreduce_tensor_keep(self, t: torch.Tensor, average: bool = True):
        out = C.allreduce(t.clone(), C.ReduceOp.SUM)
        return out / self._world_size if average else out

    def step_and_sync(self, optimizer, grad_blob=None, found_inf: bool = False, average: bool = True):
        """all-reduce -> skip the step on ``found_inf`` -> ``zero_grad`` (strategies.mojo:218-229)."""
        if grad_blob is not None:
            C.allreduce(grad_blob, C.ReduceOp.AVG if average else C.ReduceOp.SUM)
        else:
            self.allreduce_gradients(average)
        if not found_inf:
            optimizer.step()
        if hasattr(optimizer, "zero_grad"):
            optimizer.zero_grad()
