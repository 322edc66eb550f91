"""``Summarizer`` / ``model_summary`` (legacy/src/momijo/learn/utils/summary.mojo:95-235)."""
from __future__ import annotations


from dataclasses import dataclass, field
from typing import List


@dataclass
class LayerRecord:
    """One row of a summary table (legacy/src/momijo/learn/utils/summary.mojo:74-90)."""
    name: str = ""
    in_shape: List[int] = field(default_factory=list)
    out_shape: List[int] = field(default_factory=list)
    params_count: int = 0
    buffers_count: int = 0
    trainable_params: int = 0


class Summarizer:
    def __init__(self):
        self.rows, self.total = [], 0
        self.records: List[LayerRecord] = []

    def add_record(self, rec: LayerRecord):
        """Typed row: also shows up in ``render`` (shape = output shape)."""
        self.records.append(rec)
        self.add(rec.name, "layer", rec.out_shape, rec.params_count)

    def add(self, name: str, kind: str, shape, n_params: int):
        self.rows.append((name, kind, list(shape), n_params))
        self.total += n_params

    def render(self) -> str:
        lines = ["Name | Type | Shape | Params", "-" * 40]
        for n, k, s, p in self.rows:
            lines.append(f"{n} | {k} | {s} | {p}")
        lines += ["-" * 40, f"Total params: {self.total}"]
        return "\n".join(lines)


def model_summary(model) -> str:
    s = Summarizer()
    for name, mod in model.named_modules():
        own = list(mod.named_parameters(recurse=False))
        if not own and name:
            if not list(mod.children()):
                s.add(name, type(mod).__name__, [], 0)
            continue
        for pn, p in own:
            s.add(f"{name}.{pn}" if name else pn, type(mod).__name__, p.shape, p.numel())
    return s.render()
