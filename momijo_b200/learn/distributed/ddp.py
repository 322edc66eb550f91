"""``ProcessGroup``, ``init_process_group(backend, rank, world_size)`` and ``DDPLinear``
(legacy/src/momijo/learn/distributed/ddp.mojo:18-65)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..nn.layers import Linear
from ..nn.module import Module
from . import collective as C


@dataclass
class ProcessGroup:
    backend: str = "single"
    rank: int = 0
    world_size: int = 1
    comm: object = field(default=None, repr=False)  # PeerComm for nccl groups with peer memory

    def peer(self):
        """Lazily create the peer-memory communicator (symmetric heap + signal pads)."""
        if self.comm is None and self.backend == "nccl" and self.world_size > 1:
            from ...parallel.peer import PeerComm

            self.comm = PeerComm.from_default_group()
        return self.comm


def init_process_group(backend: str = "single", rank: int = 0, world_size: int = 1, **kw) -> ProcessGroup:
    print(f"[ddp:init] backend={backend} rank={rank} world_size={world_size}")
    C.init_process_group(backend, world_size, rank, **kw)
    return ProcessGroup(backend, rank, world_size)


def destroy_process_group(pg: ProcessGroup | None = None):
    C.destroy_process_group()


class DDPLinear(Module):
    """One ``Linear`` whose gradients are averaged over the group after backward."""

    def __init__(self, in_features, out_features, bias=True, pg: ProcessGroup | None = None, **kw):
        super().__init__()
        self.linear = Linear(in_features, out_features, bias, **kw)
        self.pg = pg or ProcessGroup()

    def forward(self, x):
        return self.linear(x)

    @staticmethod
    def from_module(module: Linear, pg: ProcessGroup | None = None) -> "DDPLinear":
        """Wrap an existing ``Linear`` (shares its parameters)."""
        d = DDPLinear(module.in_features, module.out_features, module.bias, pg)
        d.linear = module
        return d

    def replace_module(self, module: Linear) -> None:
        self.linear = module

    @property
    def module(self) -> Linear:
        return self.linear

    def sync_gradients(self):
        for p in self.linear.parameters():
            if p.grad is not None:
                C.allreduce(p.grad, C.ReduceOp.AVG)
