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
    """Stopwatch over caller-supplied timestamps in nanoseconds; results are seconds
    (legacy/src/momijo/learn/utils/profiling.mojo:50-107)."""

    def __init__(self):
        self.running, self.start_ns, self.accum_ns = False, 0, 0

    def reset(self, t_ns: int = 0, keep_running: bool = False):
        self.accum_ns = 0
        if keep_running and self.running:
            self.start_ns = t_ns
        else:
            self.running, self.start_ns = False, 0

    def start(self, t_ns: int):
        if not self.running:
            self.running, self.start_ns = True, t_ns

    def stop(self, t_ns: int) -> float:
        """Seconds of the segment that just ended (0 if the timer was not running)."""
        if not self.running:
            return 0.0
        seg = t_ns - self.start_ns
        self.accum_ns += seg
        self.running = False
        return ns_to_s(seg)

    def lap(self, t_ns: int) -> float:
        return ns_to_s(t_ns - self.start_ns) if self.running else 0.0

    def _total_ns(self, t_ns):
        return self.accum_ns + ((t_ns - self.start_ns) if self.running and t_ns is not None else 0)

    def elapsed(self, t_ns: int = None) -> float:
        return ns_to_s(self._total_ns(t_ns))

    def elapsed_ms(self, t_ns: int = None) -> float:
        return ns_to_ms(self._total_ns(t_ns))

    def measure(self, t_start_ns: int, t_end_ns: int) -> float:
        self.running, self.accum_ns = False, 0
        self.start(t_start_ns)
        return self.stop(t_end_ns)

    @property
    def elapsed_ns(self) -> int:
        return self.accum_ns


class LapStats:
    """count / total / min / max of lap durations in nanoseconds (profiling.mojo:138-198)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.count, self.total_ns, self.min_ns, self.max_ns = 0, 0, 0, 0

    def add_lap(self, lap_ns: int):
        self.count += 1
        self.total_ns += lap_ns
        self.min_ns = lap_ns if self.count == 1 else min(self.min_ns, lap_ns)
        self.max_ns = lap_ns if self.count == 1 else max(self.max_ns, lap_ns)

    add = add_lap

    def mean_ns(self) -> float:
        return self.total_ns / self.count if self.count else 0.0

    mean = mean_ns

    def mean_ms(self) -> float:
        return self.mean_ns() / 1e6

    def mean_s(self) -> float:
        return self.mean_ns() / 1e9

    def total_s(self) -> float:
        return ns_to_s(self.total_ns)

    def min_s(self) -> float:
        return ns_to_s(self.min_ns)

    def max_s(self) -> float:
        return ns_to_s(self.max_ns)

    def merge(self, o):
        if o.count:
            self.min_ns = o.min_ns if not self.count else min(self.min_ns, o.min_ns)
            self.max_ns = o.max_ns if not self.count else max(self.max_ns, o.max_ns)
            self.count += o.count
            self.total_ns += o.total_ns
        return self

    def __str__(self):
        return (f"LapStats(count={self.count}, total_s={self.total_s()}, mean_s={self.mean_s()}, "
                f"min_s={self.min_s()}, max_s={self.max_s()})")


class ScopedTimer:
    """Starts a timer on construction; ``stop`` ends the segment (profiling.mojo:110-135). Given a ``LapStats`` instead
    of a ``Timer`` it records the lap there."""

    def __init__(self, target, t_ns: int):
        self.target, self.t0, self.active = target, t_ns, True
        if isinstance(target, Timer):
            target.start(t_ns)

    def stop(self, t_ns: int) -> float:
        if not self.active:
            return 0.0
        self.active = False
        if isinstance(self.target, Timer):
            return self.target.stop(t_ns)
        self.target.add_lap(t_ns - self.t0)
        return ns_to_s(t_ns - self.t0)

    close = stop


class LabelProfiler:
    """Lap statistics per label, labels kept in first-seen order (profiling.mojo:201-265)."""

    def __init__(self):
        self.stats, self._open = {}, {}

    def clear(self):
        self.stats, self._open = {}, {}

    def add_lap_ns(self, label: str, lap_ns: int):
        self.stats.setdefault(label, LapStats()).add_lap(lap_ns)

    def add_lap_s(self, label: str, lap_s: float):
        self.add_lap_ns(label, s_to_ns(lap_s))

    def begin(self, label: str, t_ns: int):
        self._open[label] = t_ns

    def end(self, label: str, t_ns: int):
        t0 = self._open.pop(label, None)
        if t0 is not None:
            self.add_lap_ns(label, t_ns - t0)

    def get(self, label: str) -> LapStats:
        return self.stats.setdefault(label, LapStats())

    def summary(self):
        return [f" - {k}: count={s.count}, total_s={s.total_s()}, mean_s={s.mean_s()}, min_s={s.min_s()}, "
                f"max_s={s.max_s()}" for k, s in self.stats.items()]

    def table(self) -> str:
        rows = ["Label | Count | Total(ms) | Mean(ms) | Min(ms) | Max(ms)"]
        for k, s in self.stats.items():
            rows.append(f"{k} | {s.count} | {s.total_ns / 1e6:.3f} | {s.mean_ms():.3f} | "
                        f"{s.min_ns / 1e6:.3f} | {s.max_ns / 1e6:.3f}")
        return "\n".join(rows)

    def __str__(self):
        return "LabelProfiler:\n" + "".join(line + "\n" for line in self.summary())


class ScopedSection:
    def __init__(self, prof: LabelProfiler, label: str, t_ns: int):
        self.prof, self.label, self.t0, self.active = prof, label, t_ns, True

    def end(self, t_ns: int):
        if self.active:
            self.active = False
            self.prof.add_lap_ns(self.label, t_ns - self.t0)

    close = end


class SMA:
    """Simple moving average of the last ``capacity`` durations in nanoseconds (profiling.mojo:296-348)."""

    def __init__(self, capacity: int = 10):
        self.window = self.capacity = max(1, capacity)
        self.reset()

    def reset(self):
        self.buf, self.sum = [], 0.0

    def add(self, x: float) -> float:
        self.buf.append(x)
        self.sum += x
        if len(self.buf) > self.capacity:
            self.sum -= self.buf.pop(0)
        return self.value()

    def value(self) -> float:
        return self.sum / len(self.buf) if self.buf else 0.0

    def mean_s(self) -> float:
        return self.value() / 1e9

    def mean_ms(self) -> float:
        return self.value() / 1e6


class TrainingLoopProfiler(LabelProfiler):
    """The five phases of a step, each with lap statistics and a moving average (profiling.mojo:352-470). ``end``
    closes the phase that ``begin`` opened; a label may still be given."""
    LABELS = ("data", "forward", "backward", "step", "misc")

    def __init__(self, window: int = 50):
        super().__init__()
        self.window = window
        self.clear()

    def clear(self):
        self.stats = {k: LapStats() for k in self.LABELS}
        self.smas = {k: SMA(self.window) for k in self.LABELS}
        self._open, self._active = {}, None

    def begin(self, label: str, t_ns: int):
        self._active = label
        self._open[label] = t_ns

    def end(self, label_or_t, t_ns: int = None):
        label, t = (self._active, label_or_t) if t_ns is None else (label_or_t, t_ns)
        t0 = self._open.pop(label, None)
        if t0 is not None:
            self.add_lap_ns(label, t - t0)
            self.smas.setdefault(label, SMA(self.window)).add(t - t0)
        if label == self._active:
            self._active = None

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
        return {k: self.get(k).mean_ms() for k in self.LABELS}

    def summary_lines(self):
        return [f" - {k}: count={s.count}, total_s={s.total_s()}, mean_s={s.mean_s()}, sma_s={self.smas[k].mean_s()}"
                for k, s in self.stats.items()]

    def __str__(self):
        return "TrainingLoopProfiler:\n" + "".join(line + "\n" for line in self.summary_lines())


# unit conversions of the reference (legacy/src/momijo/learn/utils/profiling.mojo:31-46)
def ns_to_s(ns: int) -> float:
    return float(ns) / 1_000_000_000.0


def ns_to_ms(ns: int) -> float:
    return float(ns) / 1_000_000.0


def s_to_ns(seconds: float) -> int:
    """Negative durations clamp to 0; the result saturates at 2**64 - 1."""
    s = max(float(seconds), 0.0)
    return min(int(s * 1_000_000_000.0), (1 << 64) - 1)
