"""Data-parallel wrapper over flat gradient storage.

``DistributedDataParallel`` keeps parameters and gradients in two flat bf16 buffers (``FlatParams``);
``sync_gradients`` averages the gradient buffer over the ranks: with a peer communicator by this
library's two-shot all-reduce kernel over NVLink peer memory, otherwise through torch.distributed
(gloo on CPU). Every rank then applies the same optimizer step to the full buffers. Reference shape:
``DDP.wrap`` / ``allreduce_grads_mean`` (legacy/src/momijo/learn/distributed/ddp.mojo:52-105) and
``DistributedDataParallel.step_and_sync`` (legacy/src/momijo/learn/distributed/strategies.mojo:218-229),
which skips the update when an inf was found.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from .flat import FlatParams
from .zero import AdamWConfig


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, optim: Optional[AdamWConfig] = None, comm=None, group=None,
                 dtype: torch.dtype = None):
        super().__init__()
        self.module, self.comm, self.group = module, comm, group
        self.optim = optim or AdamWConfig()
        if comm is not None:
            self.world, self.rank = comm.world, comm.rank
        elif dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        p0 = next(module.parameters())
        dtype = dtype or (torch.bfloat16 if p0.is_cuda else p0.dtype)
        alloc = comm.alloc if comm is not None else None
        # total padded to 8 * world elements: the all-reduce kernel works on 16-byte vectors per rank
        self.flat = FlatParams(module, self.world, self.rank, alloc=alloc, dtype=dtype)
        n = self.flat.layout.total
        dev = self.flat.param.device
        self.master = self.flat.param.float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def sync_gradients(self):
        """Average gradients over the data-parallel group (in place in the flat buffer)."""
        self.flat.zero_untouched()
        if self.world == 1:
            return
        if self.comm is not None and self.flat.grad.dtype == torch.bfloat16:
            self.comm.all_reduce_(self.flat.grad, scale=1.0 / self.world)
        else:
            dist.all_reduce(self.flat.grad, group=self.group)
            self.flat.grad.div_(self.world)

    def step(self, lr: Optional[float] = None, found_inf: bool = False):
        self.sync_gradients()
        if found_inf:  # same protocol as GradScaler.step: skip the update, keep the state
            self.flat.mark_fresh()
            return False
        o = self.optim
        self.step_count += 1
        ops.adamw_flat(self.flat.grad, self.master, self.m, self.v, self.flat.param, lr=o.lr if lr is None else lr,
                       beta1=o.betas[0], beta2=o.betas[1], eps=o.eps, weight_decay=o.weight_decay,
                       step=self.step_count)
        self.flat.mark_fresh()
        return True

    step_and_sync = step

    def zero_grad(self):
        self.flat.mark_fresh()
