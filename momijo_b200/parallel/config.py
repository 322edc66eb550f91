"""``ParallelConfig``: how the ranks of a job are split over data, tensor, pipeline and expert
parallelism, and the process groups that go with it. The reference has no such object (its option
structs are per component, e.g. legacy/src/momijo/learn/data/dataloader.mojo:54-76); the field
style follows them."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch.distributed as dist


@dataclass
class ParallelConfig:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    zero_stage: int = 0
    micro_batches: int = 1
    sequence_parallel: bool = True
    use_peer_kernels: bool = True

    def world(self) -> int:
        return self.dp * self.tp * self.pp

    def validate(self, world_size: int):
        if self.world() != world_size:
            raise ValueError(f"dp*tp*pp = {self.world()} does not match world size {world_size}")
        if self.ep > 1 and (self.dp * self.tp) % self.ep:
            raise ValueError("ep must divide dp*tp")
        return self

    # rank layout: tp fastest, then dp, then pp (tp groups are contiguous: same NVSwitch island)
    def coords(self, rank: int):
        tp_r = rank % self.tp
        dp_r = (rank // self.tp) % self.dp
        pp_r = rank // (self.tp * self.dp)
        return {"tp": tp_r, "dp": dp_r, "pp": pp_r}

    def tp_ranks(self, rank: int):
        base = rank - rank % self.tp
        return list(range(base, base + self.tp))

    def dp_ranks(self, rank: int):
        c = self.coords(rank)
        return [c["pp"] * self.tp * self.dp + d * self.tp + c["tp"] for d in range(self.dp)]

    def pp_ranks(self, rank: int):
        c = self.coords(rank)
        return [p * self.tp * self.dp + c["dp"] * self.tp + c["tp"] for p in range(self.pp)]

    def build_groups(self):
        """Create the tp / dp / pp process groups (collective: every rank creates all groups)."""
        world = dist.get_world_size()
        rank = dist.get_rank()
        self.validate(world)
        groups = {}
        for kind, fn in (("tp", self.tp_ranks), ("dp", self.dp_ranks), ("pp", self.pp_ranks)):
            seen = set()
            for r in range(world):
                ranks = tuple(fn(r))
                if ranks in seen:
                    continue
                seen.add(ranks)
                g = dist.new_group(list(ranks))
                if rank in ranks:
                    groups[kind] = g
        return groups
