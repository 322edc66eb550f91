"""Wall-clock profilers (legacy/src/momijo/learn/utils/profiling.mojo:50-468). The classes never
read a clock themselves: the caller passes monotonic ``t_ns``. ``cuda_clock_ns`` is a clock
source that returns device-timed nanoseconds (CUDA events), so ``TrainingLoopProfiler`` can be
fed device time."""
from __future__ import annotations

import time


def host_clock_ns() -> int:
    return time.monotonic_ns()


class CudaClock:
    """Device-time clock: ``now_ns()`` records an event and returns ns since construction."""

    def __init__(self):
        import torch

        self.torch = torch
        self.t0 = torch.cuda.Event(enable_timing=True)
        self.t0.record()

    def now_ns(self) -> int:
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        e.synchronize()
        return int(self.t0.elapsed_time(e) * 1e6)


class Timer:
    def __init__(self):
        self.start_ns, self.elapsed_ns, self.running = 0, 0, False

    def start(self, t_ns: int):
        self.start_ns, self.running = t_ns, True

    def stop(self, t_ns: int) -> int:
        if self.running:
            self.elapsed_ns += t_ns - self.start_ns
            self.running = False
        return self.elapsed_ns

    def reset(self):
        self.__init__()

    def elapsed_ms(self) -> float:
        return self.elapsed_ns / 1e6


class LapStats:
    def __init__(self):
        self.count, self.total, self.min, self.max = 0, 0, None, None

    def add(self, dt_ns: int):
        self.count += 1
        self.total += dt_ns
        self.min = dt_ns if self.min is None else min(self.min, dt_ns)
        self.max = dt_ns if self.max is None else max(self.max, dt_ns)

    def mean(self) -> float:
        return self.total / self.count if self.count else 0.0

    def merge(self, o):
        if o.count:
            self.count += o.count
            self.total += o.total
            self.min = o.min if self.min is None else min(self.min, o.min)
            self.max = o.max if self.max is None else max(self.max, o.max)
        return self


class ScopedTimer:
    def __init__(self, stats: LapStats, t_ns: int):
        self.stats, self.t0 = stats, t_ns

    def close(self, t_ns: int):
        self.stats.add(t_ns - self.t0)


class LabelProfiler:
    def __init__(self):
        self.stats, self._open = {}, {}

    def begin(self, label: str, t_ns: int):
        self._open[label] = t_ns

    def end(self, label: str, t_ns: int):
        t0 = self._open.pop(label, None)
        if t0 is not None:
            self.stats.setdefault(label, LapStats()).add(t_ns - t0)

    def get(self, label: str) -> LapStats:
        return self.stats.setdefault(label, LapStats())

    def table(self) -> str:
        rows = ["Label | Count | Total(ms) | Mean(ms) | Min(ms) | Max(ms)"]
        for k, s in self.stats.items():
            rows.append(f"{k} | {s.count} | {s.total / 1e6:.3f} | {s.mean() / 1e6:.3f} | "
                        f"{(s.min or 0) / 1e6:.3f} | {(s.max or 0) / 1e6:.3f}")
        return "\n".join(rows)


class ScopedSection:
    def __init__(self, prof: LabelProfiler, label: str, t_ns: int):
        self.prof, self.label = prof, label
        prof.begin(label, t_ns)

    def close(self, t_ns: int):
        self.prof.end(self.label, t_ns)


class SMA:
    """Simple moving average over a fixed window."""

    def __init__(self, window: int = 10):
        self.window, self.buf, self.sum = max(1, window), [], 0.0

    def add(self, x: float) -> float:
        self.buf.append(x)
        self.sum += x
        if len(self.buf) > self.window:
            self.sum -= self.buf.pop(0)
        return self.value()

    def value(self) -> float:
        return self.sum / len(self.buf) if self.buf else 0.0


class TrainingLoopProfiler(LabelProfiler):
    LABELS = ("data", "forward", "backward", "step", "misc")

    def begin_data(self, t): self.begin("data", t)
    def end_data(self, t): self.end("data", t)
    def begin_forward(self, t): self.begin("forward", t)
    def end_forward(self, t): self.end("forward", t)
    def begin_backward(self, t): self.begin("backward", t)
    def end_backward(self, t): self.end("backward", t)
    def begin_step(self, t): self.begin("step", t)
    def end_step(self, t): self.end("step", t)
    def begin_misc(self, t): self.begin("misc", t)
    def end_misc(self, t): self.end("misc", t)

    def summary(self) -> dict:
        return {k: self.get(k).mean() / 1e6 for k in self.LABELS}


# unit conversions of the reference (legacy/src/momijo/learn/utils/profiling.mojo:31-46)
def ns_to_s(ns: int) -> float:
    return float(ns) / 1_000_000_000.0


def ns_to_ms(ns: int) -> float:
    return float(ns) / 1_000_000.0


def s_to_ns(seconds: float) -> int:
    """Negative durations clamp to 0; the result saturates at 2**64 - 1."""
    s = max(float(seconds), 0.0)
    return min(int(s * 1_000_000_000.0), (1 << 64) - 1)
