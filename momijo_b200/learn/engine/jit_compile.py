"""JIT facade (legacy/src/momijo/learn/engine/jit_compile.mojo:30-184). ``compile`` returns the
model unchanged in the reference; here ``JITOptions.graph`` captures the model's forward in a
CUDA graph (static shapes), which removes launch overhead without a tracing compiler, and
``check_numerics`` adds a finite check on the outputs."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch


@dataclass
class JITOptions:
    graph: bool = False
    optimize: bool = True
    check_numerics: bool = False
    allow_mixed_precision: bool = True

    # Copy-and-set builders (legacy/src/momijo/learn/engine/jit_compile.mojo:49-67): the receiver is left alone.
    def with_graph(self, on: bool) -> "JITOptions":
        return dataclasses.replace(self, graph=on)

    def with_optimize(self, on: bool) -> "JITOptions":
        return dataclasses.replace(self, optimize=on)

    def with_check_numerics(self, on: bool) -> "JITOptions":
        return dataclasses.replace(self, check_numerics=on)

    def with_mixed_precision(self, on: bool) -> "JITOptions":
        return dataclasses.replace(self, allow_mixed_precision=on)


class GraphExecutor:
    """Runs a callable; with ``graph=True`` on CUDA the first call is captured and replayed."""

    def __init__(self, fn, options: JITOptions | None = None):
        self.fn, self.options = fn, options or JITOptions()
        self._graph = self._static_in = self._static_out = None

    def run(self, batch):
        o = self.options
        if o.graph and isinstance(batch, torch.Tensor) and batch.is_cuda and not torch.is_grad_enabled():
            out = self._run_graph(batch)
        else:
            out = self.fn(batch) if self.fn is not None else batch
        if o.check_numerics and isinstance(out, torch.Tensor) and not torch.isfinite(out).all():
            raise FloatingPointError("non-finite values in the output")
        return out

    __call__ = run

    def _run_graph(self, x):
        if self._graph is None or self._static_in.shape != x.shape:
            self._static_in = x.clone()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    self.fn(self._static_in)
            torch.cuda.current_stream().wait_stream(s)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._static_out = self.fn(self._static_in)
        self._static_in.copy_(x)
        self._graph.replay()
        return self._static_out


def compile(model, options: JITOptions | None = None):
    """Reference semantics: the model comes back unchanged (jit_compile.mojo:115)."""
    return model


def compile_with(model, options: JITOptions, report: "JITReport" = None) -> GraphExecutor:
    """``report``, when given, is filled in place like the reference's out-parameter
    (legacy/src/momijo/learn/engine/jit_compile.mojo:121-135)."""
    if report is not None:
        report.graph_enabled = bool(options.graph)
        for k in ("passes_applied", "lowered_ops"):
            if hasattr(report, k):
                setattr(report, k, 0)
    return GraphExecutor(model, options)


def dry_trace(model, example):
    """Run once without gradients and report output shape/dtype."""
    with torch.no_grad():
        out = model(example)
    return {"shape": list(out.shape), "dtype": str(out.dtype)} if isinstance(out, torch.Tensor) else {}


@dataclass
class JITReport:
    """What a compile call did (legacy/src/momijo/learn/engine/jit_compile.mojo:79-108)."""
    graph_enabled: bool = False
    passes_applied: int = 0
    lowered_ops: int = 0
    fallback_ops: int = 0
    notes: str = ""

    def __str__(self):
        return (f"JITReport(graph={'true' if self.graph_enabled else 'false'}, passes={self.passes_applied}, "
                f"lowered_ops={self.lowered_ops}, fallback_ops={self.fallback_ops}, notes='{self.notes}')")


def compile_report(model, options: JITOptions) -> JITReport:
    """The report the reference's ``compile_with`` fills in: nothing is lowered ahead of time; with
    ``options.graph`` the executor captures a CUDA graph on its first call."""
    return JITReport(graph_enabled=options.graph, notes="CUDA-graph capture on first call" if options.graph
                     else "eager execution")


def prefer_graph(opts: JITOptions) -> bool:
    return bool(opts.graph)


def build_executor(opts: JITOptions, fn=None) -> GraphExecutor:
    """Executor for ``fn`` (identity when omitted) under ``opts``; ``is_valid`` tells whether graph
    capture was asked for (legacy/src/momijo/learn/engine/jit_compile.mojo:181-184)."""
    ex = GraphExecutor(fn, opts)
    ex.is_valid = bool(opts.graph)
    return ex
