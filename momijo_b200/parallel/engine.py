"""Optimizer engines for models whose parameters are not all plain data-parallel replicas.

``HybridEngine`` splits a module's parameters into

* *sharded-local* parameters, of which every rank owns a different slice outright (tensor-parallel
  weight shards, expert-parallel expert weights, the layers of one pipeline stage): updated by the
  fused AdamW kernel on a local flat buffer, no gradient exchange;
* *replicated-in-group* parameters that every rank of a tensor-parallel group holds in full but sees
  only part of the gradient of (norm weights under sequence parallelism): their gradients are summed
  over the group with the peer all-reduce kernel (or torch.distributed) before the local update;
* optionally *data-parallel* parameters (the dense part of an expert-parallel model), which go through
  ``ShardedDataParallel``: gradient reduce-scatter fused with the sharded AdamW, then the parameter
  all-gather.

The reference's wrappers stop at one level (``DDP.wrap`` legacy/src/momijo/learn/distributed/ddp.mojo:52-105,
``ZeroStage1`` legacy/src/momijo/learn/distributed/sharding.mojo:121-184); this composes them the way a
TP x PP x EP job needs.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .zero import AdamWConfig, ShardedDataParallel


def mark_replicated(params: Iterable[nn.Parameter]) -> None:
    for p in params:
        p.tp_replicated = True


class HybridEngine(nn.Module):
    def __init__(self, module: nn.Module, optim: Optional[AdamWConfig] = None, *, dp_comm=None,
                 dp_params: Optional[List[nn.Parameter]] = None, rep_comm=None, rep_group=None,
                 local_grad_scale: float = 1.0, local_grad_dtype: Optional[torch.dtype] = None):
        """``dp_params`` (with ``dp_comm``): parameters updated through the sharded data-parallel path;
        everything else is local. ``rep_comm`` / ``rep_group``: where to sum the gradients of parameters
        flagged ``tp_replicated`` (a ``PeerComm`` of the tensor-parallel group, or a process group).
        ``local_grad_dtype=torch.float32``: accumulate the local parameters' gradients in fp32 (pipeline
        schedules add many micro-batch gradients before one update)."""
        super().__init__()
        self.module = module
        self.optim = optim or AdamWConfig()
        dp_ids = {id(p) for p in (dp_params or [])}
        local = [p for p in module.parameters() if p.requires_grad and id(p) not in dp_ids]
        self.local = ShardedDataParallel(module, self.optim, stage=3, comm=None, params=local,
                                         grad_scale=local_grad_scale, grad_dtype=local_grad_dtype) if local else None
        self.dp = ShardedDataParallel(module, self.optim, stage=3, comm=dp_comm, params=list(dp_params)) \
            if dp_params else None
        self.rep_comm, self.rep_group = rep_comm, rep_group
        self._rep = [p for p in local if getattr(p, "tp_replicated", False)]
        self._rep_buf = None
        if self._rep and self.local is not None and (rep_comm is not None or rep_group is not None):
            self.local.pre_update_hook = self._sync_replicated

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def _sync_replicated(self, _sdp):
        n = sum(p.numel() for p in self._rep)
        if self.rep_comm is not None:
            W = self.rep_comm.world
            if W == 1:
                return
            if self._rep_buf is None:
                pad = (n + 8 * W - 1) // (8 * W) * (8 * W)
                self._rep_buf = self.rep_comm.alloc(pad, torch.bfloat16)
            buf = self._rep_buf
            off = 0
            # one gather of the (small, scattered) replicated gradients into the symmetric buffer
            torch.cat([p.main_grad.reshape(-1) for p in self._rep], out=buf[:n]) if all(
                p.main_grad.dtype == buf.dtype for p in self._rep) else buf[:n].copy_(
                torch.cat([p.main_grad.reshape(-1).to(buf.dtype) for p in self._rep]))
            self.rep_comm.all_reduce_(buf)
        else:
            buf = torch.cat([p.main_grad.reshape(-1) for p in self._rep])
            dist.all_reduce(buf, group=self.rep_group)
        off = 0
        for p in self._rep:
            p.main_grad.copy_(buf[off:off + p.numel()].view_as(p.main_grad))
            off += p.numel()

    def zero_grad(self):
        for e in (self.local, self.dp):
            if e is not None:
                e.zero_grad()

    def step(self, lr: Optional[float] = None):
        if self.dp is not None:
            self.dp.step(lr)
        if self.local is not None:
            self.local.step(lr)

    # ---- checkpoint / resume ----
    def save_checkpoint(self, base: str, extra: Optional[dict] = None) -> None:
        """Optimizer state of both parts in the MNP layout: the local part as ``<base>.local<global rank>``
        (every process owns different local parameters), the data-parallel part as ``<base>.dp`` with one blob
        per rank of its group. Every process calls it."""
        g = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if self.local is not None:
            self.local.save_checkpoint(f"{base}.local{g}", extra)
        if self.dp is not None:
            self.dp.save_checkpoint(f"{base}.dp", extra)

    def load_checkpoint(self, base: str) -> dict:
        """Restore what ``save_checkpoint`` wrote. The local part needs the layout it was written with (same
        tensor / expert / pipeline split, same global ranks); the data-parallel part may come from a group of
        another size."""
        g = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        extra = {}
        if self.local is not None:
            extra = self.local.load_checkpoint(f"{base}.local{g}")
        if self.dp is not None:
            extra = self.dp.load_checkpoint(f"{base}.dp") or extra
        return extra
