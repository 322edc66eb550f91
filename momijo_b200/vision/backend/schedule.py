"""Launch parameters for the tiled CPU kernels of the reference
(legacy/src/momijo/vision/backend/schedule.mojo:15-32: ``tile_h``, ``tile_w``, ``vec``). On the GPU the
same record carries the block size and the cap on the grid; the pixel kernels use grid-stride loops, so
any positive values are valid."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Schedule:
    tile_h: int = 32
    tile_w: int = 128
    vec: int = 8
    block: int = 256
    max_blocks: int = 148 * 16

    def tile_h_(self):
        return self.tile_h

    def tile_w_(self):
        return self.tile_w

    def vec_(self):
        return self.vec


def default_schedule() -> Schedule:
    return Schedule()
