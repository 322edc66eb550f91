"""Flat parameter / gradient storage shared by the data-parallel and sharded wrappers.

All parameters of a module are re-homed as views into one contiguous bf16 buffer (optionally
allocated in peer-visible symmetric memory), with a second buffer of the same layout for
gradients. Each parameter gets a ``main_grad`` view; the backward kernels store or accumulate
into it directly (``_mg_fresh`` marks "first write of this step overwrites").

The layout aligns every parameter to ``align`` elements and the total to ``align * world`` so
that shard boundaries (``partition_1d`` semantics, legacy/src/momijo/learn/distributed/
sharding.mojo:69-85, with equal shards because of the padding) never split a 16-byte vector.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.nn as nn


class FlatLayout:
    def __init__(self, params: List[nn.Parameter], world: int = 1, align: int = 128):
        self.params = params
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        unit = align * world
        self.total = (off + unit - 1) // unit * unit
        self.world = world
        self.shard = self.total // world

    def shard_range(self, rank: int):
        return rank * self.shard, (rank + 1) * self.shard


class FlatParams:
    """Owns the flat parameter and gradient buffers of a module."""

    def __init__(self, module: nn.Module, world: int = 1, rank: int = 0,
                 alloc: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None, params: Optional[List[nn.Parameter]] = None,
                 grad_dtype: Optional[torch.dtype] = None):
        """``grad_dtype``: element type of the gradient buffer (default: the parameter type). fp32 keeps
        the sum over many micro-batches exact to fp32 rounding: the weight-gradient GEMMs accumulate into it
        directly, the few non-GEMM gradients are folded in by a conversion."""
        source = list(params) if params is not None else list(module.parameters())
        seen, params = set(), []
        for p in source:
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                params.append(p)
        if not params:
            raise ValueError("module has no trainable parameters")
        device = torch.device(device) if device is not None else params[0].device
        self.layout = FlatLayout(params, world)
        self.world, self.rank = world, rank
        self.dtype = dtype
        if alloc is None:
            alloc = lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev)
        self.param = alloc(self.layout.total, dtype, device)
        self.grad_dtype = grad_dtype or dtype
        self.grad = alloc(self.layout.total, self.grad_dtype, device)
        with torch.no_grad():
            for p, off in zip(params, self.layout.offsets):
                view = self.param[off:off + p.numel()].view(p.shape)
                view.copy_(p.detach().to(dtype))
                p.data = view
                p.main_grad = self.grad[off:off + p.numel()].view(p.shape)
                p._mg_fresh = True
        self.params = params

    def mark_fresh(self):
        """Start of a step: the first gradient written to each parameter overwrites."""
        for p in self.params:
            p._mg_fresh = True

    def zero_untouched(self):
        """Fold gradients that arrived through autograd's ``.grad`` into the flat buffer;
        parameters that received no gradient this step contribute zeros."""
        for p in self.params:
            if p.grad is not None:
                g = p.grad.to(p.main_grad.dtype)
                if p._mg_fresh:
                    p.main_grad.copy_(g)
                else:
                    p.main_grad.add_(g)
                p.grad = None
                p._mg_fresh = False
            if p._mg_fresh:
                p.main_grad.zero_()
                p._mg_fresh = False

    def local_shard(self, buf: torch.Tensor) -> torch.Tensor:
        a, b = self.layout.shard_range(self.rank)
        return buf[a:b]
