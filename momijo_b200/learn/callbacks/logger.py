"""In-memory CSV loggers flushed through a writer, plus a JSONL sink
(legacy/src/momijo/learn/callbacks/logger.mojo:27-201). Only rank 0 flushes by default."""
from __future__ import annotations

import json
from typing import List


def _csv_escape(s: str) -> str:
    s = str(s)
    if any(c in s for c in ',"\n\r'):
        return '"' + s.replace('"', '""') + '"'
    return s


def _join_csv(fields: List[str]) -> str:
    return ",".join(_csv_escape(f) for f in fields)


def _is_rank0() -> bool:
    try:
        import torch.distributed as dist

        return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
    except Exception:
        return True


class CSVLogger:
    def __init__(self, path: str, include_header: bool = True):
        self.path, self.lines = path, []
        if include_header:
            self.lines.append("step,message")

    def log(self, step: int, msg: str):
        self.lines.append(_join_csv([str(step), msg]))

    # Trainer callback protocol
    def on_batch_end(self, step, msg=""):
        self.log(step, msg)

    def to_string(self) -> str:
        return "\n".join(self.lines) + ("\n" if self.lines else "")

    def clear(self):
        self.lines = []

    def flush_with(self, writer=None, rank0_only: bool = True):
        if rank0_only and not _is_rank0():
            return
        if writer is not None:
            writer(self.path, self.to_string())
        else:
            with open(self.path, "w") as f:
                f.write(self.to_string())


class CSVTableLogger:
    def __init__(self, path: str, columns: List[str], include_header: bool = True):
        self.path, self.columns, self.lines = path, list(columns), []
        if include_header:
            self.lines.append(_join_csv(self.columns))

    def log_row(self, values: List[str]):
        vals = [str(v) for v in values][:len(self.columns)]
        vals += [""] * (len(self.columns) - len(vals))
        self.lines.append(_join_csv(vals))

    def log_pairs(self, pairs: List[str]):
        """``["name", "value", ...]`` placed into their columns."""
        row = {pairs[i]: pairs[i + 1] for i in range(0, len(pairs) - 1, 2)}
        self.log_row([row.get(c, "") for c in self.columns])

    def log_scalar(self, step: int, name: str, value):
        self.log_pairs(["step", str(step), name, str(value)])

    def to_string(self) -> str:
        return "\n".join(self.lines) + ("\n" if self.lines else "")

    def clear(self):
        self.lines = []

    def flush_with(self, writer=None, rank0_only: bool = True):
        if rank0_only and not _is_rank0():
            return
        if writer is not None:
            writer(self.path, self.to_string())
        else:
            with open(self.path, "w") as f:
                f.write(self.to_string())


class JSONLLogger:
    """One JSON object per line (step, tokens/s, device-timed step time, ...)."""

    def __init__(self, path: str):
        self.path, self.rows = path, []

    def log(self, **fields):
        self.rows.append(fields)

    def flush(self, rank0_only: bool = True):
        if rank0_only and not _is_rank0():
            return
        with open(self.path, "a") as f:
            for r in self.rows:
                f.write(json.dumps(r) + "\n")
        self.rows = []
