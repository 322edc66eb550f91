"""Host model of the signal-pad protocol used by the peer-memory kernels, for interleaving tests.

Device protocol (``csrc/comm.cu`` ``block_barrier``, ``signal_kernel`` / ``wait_kernel``): every rank owns
an array of int32 slots; a barrier with base ``b`` and epoch ``e`` has rank ``r`` store ``e`` into slot
``b + r`` of every rank (release) and then wait until its own slots ``b + 0 .. b + W-1`` all hold a value
``>= e`` (acquire). Epochs of one base only grow, so a slot is never reset and a late reader can never
mistake an old value for a new one; a rank that runs ahead can at most be one barrier ahead of the
slowest rank, because its next barrier cannot complete without the slowest rank's store.

``simulate`` runs W ranks through a sequence of barriers under an arbitrary interleaving of their
individual stores and polls and checks the two safety properties on every step: nobody leaves barrier
``e`` before everybody entered it, and nobody is ever more than one barrier ahead.
"""
from __future__ import annotations

import random
from typing import List, Optional


class Rank:
    def __init__(self, r: int, world: int, n_barriers: int):
        self.r, self.world, self.n = r, world, n_barriers
        self.epoch = 1          # barrier being executed (1-based)
        self.phase = 0          # 0 .. W-1: store to peer `phase`; W .. 2W-1: poll own slot `phase - W`
        self.done = 0           # barriers completed
        self.entered = 0        # barriers entered (first store issued)

    def finished(self) -> bool:
        return self.done >= self.n


def simulate(world: int, n_barriers: int, seed: int = 0, schedule: Optional[List[int]] = None,
             skip_store: Optional[tuple] = None, max_steps: int = 1_000_000):
    """Returns ``(ok, steps, stuck_ranks)``. ``skip_store=(rank, epoch, peer)`` drops one store (a lost
    signal): the run must then end with ranks stuck, never with a safety violation."""
    rng = random.Random(seed)
    slots = [[0] * world for _ in range(world)]   # slots[owner][writer]
    ranks = [Rank(r, world, n_barriers) for r in range(world)]
    steps = 0
    idle_rounds = 0
    while not all(x.finished() for x in ranks) and steps < max_steps:
        live = [x for x in ranks if not x.finished()]
        x = ranks[schedule[steps % len(schedule)]] if schedule else rng.choice(live)
        if x.finished():
            steps += 1
            continue
        progressed = True
        if x.phase < world:
            if x.phase == 0:
                x.entered = x.epoch
            peer = x.phase
            if skip_store != (x.r, x.epoch, peer):
                assert slots[peer][x.r] < x.epoch, "epochs must grow"
                slots[peer][x.r] = x.epoch
            x.phase += 1
        else:
            src = x.phase - world
            if slots[x.r][src] >= x.epoch:
                x.phase += 1
                if x.phase == 2 * world:
                    # safety 1: everyone has entered this barrier
                    assert all(y.entered >= x.epoch for y in ranks), "left a barrier nobody else entered"
                    x.done = x.epoch
                    x.epoch += 1
                    x.phase = 0
            else:
                progressed = False
        # safety 2: nobody more than one barrier ahead
        lo = min(y.done for y in ranks)
        assert all(y.done - lo <= 1 for y in ranks), "a rank ran more than one barrier ahead"
        steps += 1
        idle_rounds = 0 if progressed else idle_rounds + 1
        if idle_rounds > 50 * world * world:
            break
    stuck = [x.r for x in ranks if not x.finished()]
    return len(stuck) == 0, steps, stuck
