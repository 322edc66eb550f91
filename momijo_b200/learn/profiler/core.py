"""Op-count profiler: ``Profiler.record(key, est_ops, shapes)`` + ``table()``
(legacy/src/momijo/learn/profiler/core.mojo:12-111). ``attach(model)`` feeds it automatically
from forward hooks with analytic FLOPs, and ``roofline()`` turns measured times into fractions of
the measured peaks."""
from __future__ import annotations

from dataclasses import dataclass

from .estimators import est_ops_linear, est_ops_relu


@dataclass
class ProfRow:
    key: str
    calls: int
    est_ops: float
    shapes: str


class Profiler:
    def __init__(self, record_shapes: bool = True):
        self.record_shapes = record_shapes
        self.rows = {}
        self._handles = []

    def record(self, key: str, est_ops: float, shapes: str = ""):
        r = self.rows.get(key)
        if r is None:
            self.rows[key] = ProfRow(key, 1, float(est_ops), shapes if self.record_shapes else "")
        else:
            r.calls += 1
            r.est_ops += float(est_ops)

    def table(self, sort_by_ops: bool = True, row_limit: int = 5) -> str:
        rows = list(self.rows.values())
        if sort_by_ops:
            rows.sort(key=lambda r: -r.est_ops)
        rows = rows[:row_limit] if row_limit > 0 else rows
        w = max([len(r.key) for r in rows] + [3])
        out = [f"{'Key'.ljust(w)} | Calls | EstOps(×1e6) | Shapes"]
        for r in rows:
            out.append(f"{r.key.ljust(w)} | {r.calls:5d} | {r.est_ops / 1e6:12.3f} | {r.shapes}")
        return "\n".join(out)

    def total_ops(self) -> float:
        return sum(r.est_ops for r in self.rows.values())

    def attach(self, model):
        """Register forward hooks on Linear / activation layers of ``model``."""
        from ..nn.layers import Linear, ReLU

        for name, m in model.named_modules():
            if isinstance(m, Linear):
                def hook(mod, inp, out, _n=name):
                    x = inp[0]
                    n = x.numel() // x.shape[-1]
                    self.record(_n or "linear", est_ops_linear(n, mod.in_features, mod.out_features),
                                f"{list(x.shape)}x{list(mod.weight.shape)}")
                self._handles.append(m.register_forward_hook(hook))
            elif isinstance(m, ReLU):
                def hook2(mod, inp, out, _n=name):
                    x = inp[0]
                    self.record(_n or "relu", est_ops_relu(x.shape[0], x.numel() // max(x.shape[0], 1)),
                                f"{list(x.shape)}")
                self._handles.append(m.register_forward_hook(hook2))
        return self

    def detach(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    @staticmethod
    def roofline(flops: float, bytes_hbm: float, bytes_nvlink: float, seconds: float,
                 peak_flops: float = 1.684e15, peak_hbm: float = 6.53e12, peak_link: float = 7.7e11):
        """Achieved fraction of the roofline: the slowest of compute, HBM and NVLink time at peak
        divided by the measured time."""
        bound = max(flops / peak_flops, bytes_hbm / peak_hbm, bytes_nvlink / peak_link)
        return bound / seconds if seconds > 0 else 0.0
