"""Mergeable streaming statistics (Welford + Chan's parallel merge), the cross-rank reduction
primitive for metrics (legacy/src/momijo/learn/metrics/streaming.mojo:38-168)."""
from __future__ import annotations

import math


class StreamingMetric:
    def __init__(self):
        self.count, self.mean, self.m2 = 0, 0.0, 0.0
        self.min, self.max = math.inf, -math.inf

    def update(self, x: float):
        self.count += 1
        d = x - self.mean
        self.mean += d / self.count
        self.m2 += d * (x - self.mean)
        self.min, self.max = min(self.min, x), max(self.max, x)
        return self

    def update_many(self, xs):
        for x in xs:
            self.update(float(x))
        return self

    def merge(self, other: "StreamingMetric"):
        if other.count == 0:
            return self
        if self.count == 0:
            self.__dict__.update(other.__dict__)
            return self
        n = self.count + other.count
        d = other.mean - self.mean
        self.m2 = self.m2 + other.m2 + d * d * self.count * other.count / n
        self.mean = self.mean + d * other.count / n
        self.count = n
        self.min, self.max = min(self.min, other.min), max(self.max, other.max)
        return self

    def variance(self, unbiased: bool = False) -> float:
        if self.count < (2 if unbiased else 1):
            return 0.0
        return self.m2 / (self.count - 1 if unbiased else self.count)

    def std(self, unbiased: bool = False) -> float:
        return math.sqrt(self.variance(unbiased))

    def total(self) -> float:
        return self.mean * self.count

    def to_tuple(self):
        return (self.count, self.mean, self.m2, self.min, self.max)

    @staticmethod
    def from_tuple(t):
        s = StreamingMetric()
        s.count, s.mean, s.m2, s.min, s.max = int(t[0]), float(t[1]), float(t[2]), float(t[3]), float(t[4])
        return s

    def all_reduce(self, group=None):
        """Merge the statistics of every rank (no-op without an initialised process group)."""
        import torch
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            return self
        objs = [None] * dist.get_world_size(group)
        dist.all_gather_object(objs, self.to_tuple(), group=group)
        merged = StreamingMetric()
        for t in objs:
            merged.merge(StreamingMetric.from_tuple(t))
        self.__dict__.update(merged.__dict__)
        return self


class WeightedStreamingMetric:
    def __init__(self):
        self.wsum, self.mean, self.m2 = 0.0, 0.0, 0.0

    def update(self, x: float, w: float = 1.0):
        if w <= 0:
            return self
        self.wsum += w
        d = x - self.mean
        self.mean += d * w / self.wsum
        self.m2 += w * d * (x - self.mean)
        return self

    def merge(self, o):
        if o.wsum == 0:
            return self
        if self.wsum == 0:
            self.__dict__.update(o.__dict__)
            return self
        w = self.wsum + o.wsum
        d = o.mean - self.mean
        self.m2 += o.m2 + d * d * self.wsum * o.wsum / w
        self.mean += d * o.wsum / w
        self.wsum = w
        return self

    def variance(self):
        return self.m2 / self.wsum if self.wsum > 0 else 0.0


class ConfusionMatrixBinary:
    def __init__(self):
        self.tp = self.fp = self.tn = self.fn = 0

    def update(self, pred: int, target: int):
        if pred and target:
            self.tp += 1
        elif pred and not target:
            self.fp += 1
        elif not pred and target:
            self.fn += 1
        else:
            self.tn += 1
        return self

    def merge(self, o):
        self.tp += o.tp; self.fp += o.fp; self.tn += o.tn; self.fn += o.fn
        return self

    def precision(self):
        return self.tp / (self.tp + self.fp) if (self.tp + self.fp) else 0.0

    def recall(self):
        return self.tp / (self.tp + self.fn) if (self.tp + self.fn) else 0.0

    def f1(self):
        p, r = self.precision(), self.recall()
        return 2 * p * r / (p + r) if (p + r) else 0.0

    def accuracy(self):
        n = self.tp + self.fp + self.tn + self.fn
        return (self.tp + self.tn) / n if n else 0.0
