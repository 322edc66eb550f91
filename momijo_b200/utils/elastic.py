"""Failure detection and restart on the host.

The reference cannot lose a rank because it never has more than one (``init_process_group`` asserts
``world_size == 1``, legacy/src/momijo/learn/distributed/collective.mojo:74-78); what it has is local
error swallowing. A multi-GPU job needs three things, all of which live on the host here:

* ``Heartbeat``: every rank writes a timestamp into the job's key-value store (the TCP store that
  torch.distributed already runs) from a daemon thread; ``FailureDetector.dead_ranks()`` lists the
  ranks whose last beat is older than the deadline. Device-side waits are bounded separately (they
  return an error status that ``_C.check_status`` turns into ``DeviceTimeout``).
* ``guarded_step``: runs one training step and converts a device timeout, a collective timeout or a
  peer's death into one ``RankFailure`` exception, so that the training loop has a single thing to catch.
* ``run_elastic``: the restart loop. On ``RankFailure`` every surviving rank leaves the step, the caller's
  ``rebuild`` callback tears down and re-creates the process group (possibly with fewer ranks), the
  last checkpoint is reloaded (``load_resharded`` re-partitions flat optimizer state for the new world
  size with the same ``partition_1d`` rule the sharded optimizer uses) and training continues.

Nothing here touches a GPU; faults are injected in tests by raising on the host, by a rank process that
exits between steps, or by a store that drops keys.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, Iterable, List, Optional

import torch


class RankFailure(RuntimeError):
    """A peer died, a collective timed out or a device-side wait ran out."""

    def __init__(self, msg: str, dead: Optional[List[int]] = None):
        super().__init__(msg)
        self.dead = list(dead or [])


class DictStore:
    """In-process stand-in for the TCP store (tests, single-process runs)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()
        self.drop: Callable[[str], bool] = lambda key: False   # fault injection: drop matching writes

    def set(self, key: str, value):
        if self.drop(key):
            return
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys: Iterable[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, interval_s: float = 0.5, prefix: str = "mmj/hb", clock=time.time):
        self.store, self.rank, self.interval, self.prefix, self.clock = store, rank, interval_s, prefix, clock
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self):
        self.store.set(self.key(self.rank), repr(self.clock()))

    def start(self):
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, name="mmj-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)


class FailureDetector:
    def __init__(self, store, world: int, deadline_s: float = 3.0, prefix: str = "mmj/hb", clock=time.time):
        self.store, self.world, self.deadline, self.prefix, self.clock = store, world, deadline_s, prefix, clock

    def last_beat(self, rank: int) -> Optional[float]:
        key = f"{self.prefix}/{rank}"
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return float(self.store.get(key).decode())
        except Exception:
            return None

    def dead_ranks(self) -> List[int]:
        now = self.clock()
        out = []
        for r in range(self.world):
            t = self.last_beat(r)
            if t is None or now - t > self.deadline:
                out.append(r)
        return out

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(f"no heartbeat from ranks {dead} within {self.deadline} s", dead)


def guarded_step(step_fn: Callable[[], object], detector: Optional[FailureDetector] = None,
                 check_device: bool = True):
    """Run ``step_fn``; any of the three failure channels surfaces as ``RankFailure``."""
    if detector is not None:
        detector.check()
    try:
        out = step_fn()
        if check_device and torch.cuda.is_available():
            from .. import _C
            _C.check_status()
        return out
    except RankFailure:
        raise
    except Exception as e:  # DeviceTimeout, DistBackendError / collective timeout, injected faults
        name = type(e).__name__
        msg = str(e).lower()
        # what a vanished peer looks like from a collective: a timeout, or the transport's own words for a
        # closed connection (gloo: "Connection reset by peer", "Connection closed by peer", "Read error")
        lost = ("timeout", "timed out", "connection reset", "connection closed", "broken pipe", "read error",
                "write error", "socket closed")
        if name in ("DeviceTimeout", "DistBackendError", "DistNetworkError", "InjectedFault") or \
                any(w in msg for w in lost):
            dead = detector.dead_ranks() if detector is not None else []
            raise RankFailure(f"{name}: {e}", dead) from e
        raise


class InjectedFault(RuntimeError):
    """Raised by tests in place of a real failure."""


def partition_1d(n: int, world: int, rank: int):
    """Contiguous near-equal split, remainder to the lowest ranks
    (legacy/src/momijo/learn/distributed/sharding.mojo:69-85)."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def reshard_flat(shards: List[torch.Tensor], new_world: int) -> List[torch.Tensor]:
    """Concatenate the per-rank shards of a flat state tensor and cut it again for ``new_world`` ranks."""
    full = torch.cat([s.reshape(-1) for s in shards])
    return [full[slice(*partition_1d(full.numel(), new_world, r))].clone() for r in range(new_world)]


def run_elastic(make_state: Callable[[int, int], object], train_step: Callable[[object, int], object],
                save: Callable[[object, int], None], load: Callable[[object], int],
                rebuild: Callable[[RankFailure], tuple], total_steps: int, rank: int, world: int,
                detector_factory: Optional[Callable[[int], FailureDetector]] = None, save_every: int = 1,
                max_restarts: int = 3):
    """Training loop with restart. ``make_state(rank, world)`` builds model + optimizer; ``load(state)``
    restores the last checkpoint and returns the step to resume from (0 if none); ``rebuild(failure)``
    re-creates the communication layer and returns the new ``(rank, world)``. Returns the final state and
    the number of restarts taken."""
    restarts = 0
    state = make_state(rank, world)
    step = load(state)
    detector = detector_factory(world) if detector_factory else None
    while step < total_steps:
        try:
            guarded_step(lambda: train_step(state, step), detector, check_device=False)
            step += 1
            if step % save_every == 0:
                save(state, step)
        except RankFailure as f:
            restarts += 1
            if restarts > max_restarts:
                raise
            rank, world = rebuild(f)
            state = make_state(rank, world)
            step = load(state)
            detector = detector_factory(world) if detector_factory else None
    return state, restarts
