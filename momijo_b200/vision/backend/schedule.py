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


def auto_schedule(img_h: int, img_w: int) -> Schedule:
    """The reference's heuristic is a constant 64 x 64 tile with 16-wide vectors
    (legacy/src/momijo/vision/backend/schedule.mojo:28-33); the CUDA fields keep their defaults, except that
    the grid cap shrinks for images with fewer pixels than a full grid would cover."""
    px = max(1, int(img_h) * int(img_w))
    return Schedule(64, 64, 16, 256, max(1, min(148 * 16, (px + 255) // 256)))
