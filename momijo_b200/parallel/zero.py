"""Sharded data parallelism (ZeRO stages 1-3) over flat buffers.

``ShardedDataParallel`` wraps a module, re-homes its parameters into one flat bf16 buffer and
keeps fp32 master weights and AdamW moments only for the local shard (``partition_1d`` layout,
legacy/src/momijo/learn/distributed/sharding.mojo:69-85). One optimizer step is

  gradient reduce-scatter  +  1/world scaling  +  AdamW on the local shard  +  bf16 write-back

executed by ONE kernel per step over NVLink peer memory (``csrc/comm.cu``), followed by the
parameter all-gather (a peer-copy kernel, or fused into the consuming GEMM). With one rank the
same code path degenerates to the fused AdamW kernel on the whole buffer.

API parity: ``step_sharded`` / ``zero_grad_sharded`` / ``state_dict`` follow ``ZeroStage1``
(legacy/src/momijo/learn/distributed/sharding.mojo:164-184); stage 1 is kept as a mode.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .flat import FlatParams


@dataclass
class AdamWConfig:
    lr: float = 1e-3
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0


class ShardedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, optim: Optional[AdamWConfig] = None, stage: int = 3,
                 comm=None, grad_clip: Optional[float] = None, params=None, grad_scale: float = 1.0):
        """``params``: restrict the wrapper to these parameters of ``module`` (default: all of them).
        ``grad_scale``: constant applied to the gradients of a single-rank wrapper (a rank that owns
        its shard outright but whose loss is a per-rank mean needs 1/world here)."""
        super().__init__()
        self.module = module
        self.optim = optim or AdamWConfig()
        self.stage = stage
        self.comm = comm  # parallel.peer.PeerComm or None (single rank)
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.grad_clip = grad_clip
        alloc = comm.alloc if comm is not None else None
        self.flat = FlatParams(module, self.world, self.rank, alloc=alloc, params=params)
        self.grad_scale = grad_scale
        self.pre_update_hook = None  # called after gradients are final in the flat buffer, before the update
        dev = self.flat.param.device
        n = self.flat.layout.shard
        a, b = self.flat.layout.shard_range(self.rank)
        self.master = self.flat.param[a:b].float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    # ---- ZeroStage1-style names ----
    def zero_grad_sharded(self):
        self.flat.mark_fresh()

    zero_grad = zero_grad_sharded

    def step_sharded(self, lr: Optional[float] = None):
        return self.step(lr)

    def step(self, lr: Optional[float] = None):
        """Reduce gradients across ranks, update the local shard, republish bf16 parameters."""
        o = self.optim
        lr = o.lr if lr is None else lr
        self.flat.zero_untouched()
        if self.pre_update_hook is not None:
            self.pre_update_hook(self)
        self.step_count += 1
        if self.world == 1:
            grad_scale = self.grad_scale
            gs_dev = None
            if self.grad_clip is not None:
                ops.sq_norm(self.flat.grad, out=self.gnorm_sq)
                gs_dev = torch.clamp(self.grad_clip / (self.gnorm_sq.sqrt() + 1e-6), max=1.0)
            ops.adamw_flat(self.flat.grad, self.master, self.m, self.v, self.flat.param, lr=lr,
                           beta1=o.betas[0], beta2=o.betas[1], eps=o.eps,
                           weight_decay=o.weight_decay, step=self.step_count,
                           grad_scale=grad_scale, grad_scale_dev=gs_dev)
        else:
            self.comm.reduce_scatter_adamw(self, lr)
            self.comm.all_gather_params(self)
        self.flat.mark_fresh()

    def state_dict_sharded(self) -> str:
        """Same JSON shape as ``ZeroStage1.state_dict``."""
        return json.dumps({"world_size": self.world, "rank": self.rank})
