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


def _shape_str(shape) -> str:
    return "[" + ", ".join(str(int(d)) for d in shape) + "]"


class Summarizer:
    """Builder of the layer table (summary.mojo:95-235): rows of ``LayerRecord`` plus running totals of parameters,
    trainable parameters and buffers. Layers add themselves through ``summarize(summarizer)``."""

    def __init__(self, title: str = "Model Summary"):
        self.title = title
        self.rows: List[LayerRecord] = []
        self.total_params = self.total_buffers = self.total_trainable = 0

    @property
    def records(self):
        return self.rows

    @property
    def total(self) -> int:
        return self.total_params

    def add_counts(self, name, in_shape, out_shape, params_count: int, buffers_count: int, trainable_params: int):
        self.rows.append(LayerRecord(name, list(in_shape), list(out_shape), params_count, buffers_count, trainable_params))
        self.total_params += params_count
        self.total_buffers += buffers_count
        self.total_trainable += trainable_params

    def add_leaf(self, name, in_shape, out_shape):
        self.add_counts(name, in_shape, out_shape, 0, 0, 0)

    def add_params_generic(self, name, in_shape, out_shape, params, buffers, trainable: bool = True):
        pc = sum(int(t.numel()) for t in params)
        bc = sum(int(t.numel()) for t in buffers)
        self.add_counts(name, in_shape, out_shape, pc, bc, pc if trainable else 0)

    add_params_f64 = add_params_u8 = add_params_generic

    def add_record(self, rec: LayerRecord):
        self.add_counts(rec.name, rec.in_shape, rec.out_shape, rec.params_count, rec.buffers_count, rec.trainable_params)

    def add(self, name: str, kind: str, shape, n_params: int):
        """One row for a parameter tensor: ``kind`` is the owning layer type, ``shape`` the tensor's shape."""
        self.add_counts(f"{name} ({kind})" if kind else name, [], list(shape), n_params, 0, n_params)

    def render(self) -> str:
        w_idx, w_name, w_io, w_p, w_b = 5, 26, 28, 12, 10
        sep = "-" * (w_idx + w_name + w_io + w_p + w_b + 5)
        out = [self.title, sep,
               " ".join(("#".ljust(w_idx), "Name".ljust(w_name), "In -> Out".ljust(w_io), "Params".ljust(w_p),
                         "Buffers".ljust(w_b))), sep]
        for k, r in enumerate(self.rows):
            io = _shape_str(r.in_shape) + " -> " + _shape_str(r.out_shape)
            out.append(" ".join((str(k).ljust(w_idx), r.name.ljust(w_name), io.ljust(w_io),
                                 str(r.params_count).ljust(w_p), str(r.buffers_count).ljust(w_b))))
        out += [sep, f"Total params: {self.total_params} | Trainable: {self.total_trainable} | "
                     f"Buffers: {self.total_buffers}"]
        return "\n".join(out) + "\n"


def summarize_module(mod, s: Summarizer, name: str = None) -> None:
    """Default ``summarize`` of a layer: one row with its own parameters and buffers, then its children."""
    own_p = [p for _, p in mod.named_parameters(recurse=False)]
    own_b = [b for _, b in mod.named_buffers(recurse=False)]
    kids = list(mod.children())
    if own_p or own_b or not kids:
        pc = sum(p.numel() for p in own_p)
        s.add_counts(name or type(mod).__name__, [-1], [-1], pc, sum(b.numel() for b in own_b),
                     sum(p.numel() for p in own_p if p.requires_grad))
    for child in kids:
        (child.summarize if hasattr(child, "summarize") else (lambda ss, c=child: summarize_module(c, ss)))(s)


def model_summary(model) -> str:
    """``model.summarize(summarizer)`` then ``render`` (summary.mojo:237-240)."""
    s = Summarizer("Model Summary")
    if hasattr(model, "summarize"):
        model.summarize(s)
    else:
        summarize_module(model, s)
    return s.render()
