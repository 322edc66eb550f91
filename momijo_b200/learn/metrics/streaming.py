"""Mergeable streaming statistics (Welford + Chan's parallel merge), the cross-rank reduction
primitive for metrics (legacy/src/momijo/learn/metrics/streaming.mojo:38-440). Every statistic is read
through a method (``count()``, ``mean()``, ``min()`` ...) as in the reference; ``compute()`` is the
primary one (the mean, or accuracy for the confusion matrix). ``std`` is the square root of the variance."""
from __future__ import annotations

import math


class StreamingMetric:
    def __init__(self):
        self.reset()

    def reset(self):
        self._count, self._sum, self._mean, self._m2 = 0, 0.0, 0.0, 0.0
        self._min, self._max = math.inf, -math.inf

    def update(self, x: float):
        x = float(x)
        self._count += 1
        self._sum += x
        d = x - self._mean
        self._mean += d / self._count
        self._m2 += d * (x - self._mean)
        self._min, self._max = min(self._min, x), max(self._max, x)
        return self

    def update_batch(self, values) -> int:
        for x in values:
            self.update(x)
        return len(values)

    def update_many(self, xs):
        self.update_batch(list(xs))
        return self

    def merge(self, other: "StreamingMetric"):
        if other._count == 0:
            return self
        if self._count == 0:
            self.__dict__.update(other.__dict__)
            return self
        n = self._count + other._count
        d = other._mean - self._mean
        self._m2 = self._m2 + other._m2 + d * d * self._count * other._count / n
        self._mean = self._mean + d * other._count / n
        self._count, self._sum = n, self._sum + other._sum
        self._min, self._max = min(self._min, other._min), max(self._max, other._max)
        return self

    def count(self) -> int:
        return self._count

    def sum(self) -> float:
        return self._sum

    total = sum

    def mean(self) -> float:
        return self._mean if self._count else 0.0

    def variance(self, unbiased: bool = True) -> float:
        if self._count < (2 if unbiased else 1):
            return 0.0
        return self._m2 / (self._count - 1 if unbiased else self._count)

    def std(self, unbiased: bool = True) -> float:
        return math.sqrt(self.variance(unbiased))

    def min(self) -> float:
        return self._min if self._count else 0.0

    def max(self) -> float:
        return self._max if self._count else 0.0

    def compute(self) -> float:
        return self.mean()

    def to_tuple(self):
        return (self._count, self._mean, self._m2, self._min, self._max, self._sum)

    @staticmethod
    def from_tuple(t):
        s = StreamingMetric()
        s._count, s._mean, s._m2, s._min, s._max = int(t[0]), float(t[1]), float(t[2]), float(t[3]), float(t[4])
        s._sum = float(t[5]) if len(t) > 5 else s._mean * s._count
        return s

    def all_reduce(self, group=None):
        """Merge the statistics of every rank (no-op without an initialised process group)."""
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
    """Weighted mean / variance; non-positive weights are skipped (streaming.mojo:179-312)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self._w_sum, self._mean, self._m2 = 0.0, 0.0, 0.0
        self._min, self._max = math.inf, -math.inf

    def update(self, x: float, w: float = 1.0):
        if w <= 0:
            return self
        x = float(x)
        self._w_sum += w
        d = x - self._mean
        self._mean += d * w / self._w_sum
        self._m2 += w * d * (x - self._mean)
        self._min, self._max = min(self._min, x), max(self._max, x)
        return self

    def update_batch(self, values, weights) -> int:
        k = min(len(values), len(weights))
        for i in range(k):
            self.update(values[i], weights[i])
        return k

    def merge(self, o):
        if o._w_sum == 0:
            return self
        if self._w_sum == 0:
            self.__dict__.update(o.__dict__)
            return self
        w = self._w_sum + o._w_sum
        d = o._mean - self._mean
        self._m2 += o._m2 + d * d * self._w_sum * o._w_sum / w
        self._mean += d * o._w_sum / w
        self._w_sum = w
        self._min, self._max = min(self._min, o._min), max(self._max, o._max)
        return self

    def weight_sum(self) -> float:
        return self._w_sum

    def mean(self) -> float:
        return self._mean if self._w_sum > 0 else 0.0

    def variance(self) -> float:
        return self._m2 / self._w_sum if self._w_sum > 0 else 0.0

    def std(self) -> float:
        return math.sqrt(self.variance())

    def min(self) -> float:
        return self._min if self._w_sum > 0 else 0.0

    def max(self) -> float:
        return self._max if self._w_sum > 0 else 0.0

    def compute(self) -> float:
        return self.mean()


class ConfusionMatrixBinary:
    """Binary confusion counts from scores (thresholded) or labels (streaming.mojo:314-440)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self._tp = self._fp = self._tn = self._fn = 0

    def update(self, score: float, target: int, threshold: float = 0.5):
        return self.update_label(1 if score >= threshold else 0, target)

    def update_label(self, pred_label: int, target: int):
        p, t = pred_label != 0, target != 0
        if p and t:
            self._tp += 1
        elif p and not t:
            self._fp += 1
        elif not p and not t:
            self._tn += 1
        else:
            self._fn += 1
        return self

    def update_batch_scores(self, scores, targets, threshold: float = 0.5) -> int:
        k = min(len(scores), len(targets))
        for i in range(k):
            self.update(scores[i], targets[i], threshold)
        return k

    def update_batch_labels(self, preds, targets) -> int:
        k = min(len(preds), len(targets))
        for i in range(k):
            self.update_label(preds[i], targets[i])
        return k

    def merge(self, o):
        self._tp += o._tp; self._fp += o._fp; self._tn += o._tn; self._fn += o._fn
        return self

    def tp(self) -> int: return self._tp
    def fp(self) -> int: return self._fp
    def tn(self) -> int: return self._tn
    def fn(self) -> int: return self._fn

    def support_pos(self) -> int:
        return self._tp + self._fn

    def support_neg(self) -> int:
        return self._tn + self._fp

    def total(self) -> int:
        return self._tp + self._fp + self._tn + self._fn

    @staticmethod
    def _ratio(a, b) -> float:
        return a / b if b else 0.0

    def accuracy(self) -> float:
        return self._ratio(self._tp + self._tn, self.total())

    def precision(self) -> float:
        return self._ratio(self._tp, self._tp + self._fp)

    def recall(self) -> float:
        return self._ratio(self._tp, self._tp + self._fn)

    def specificity(self) -> float:
        return self._ratio(self._tn, self._tn + self._fp)

    def f1(self) -> float:
        p, r = self.precision(), self.recall()
        return 2 * p * r / (p + r) if (p + r) else 0.0

    def balanced_accuracy(self) -> float:
        return (self.recall() + self.specificity()) / 2.0

    def compute(self) -> float:
        return self.accuracy()
