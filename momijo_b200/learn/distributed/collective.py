"""Collective facade (legacy/src/momijo/learn/distributed/collective.mojo:29-232).

Same names and signatures as the reference; ``backend="single"`` keeps its identity semantics.
With ``"gloo"`` (CPU) or ``"nccl"`` (GPU) the calls are real collectives through
torch.distributed. ``all_gather``, ``reduce_scatter``, ``all_to_all``, ``send`` and ``recv`` are
additions in the same style (needed by ZeRO, TP, EP and PP).
"""
from __future__ import annotations

import datetime
import os
from typing import List

import torch
import torch.distributed as dist


class ReduceOp:
    SUM, PROD, MAX, MIN, AVG = 0, 1, 2, 3, 4
    _names = {0: "sum", 1: "prod", 2: "max", 3: "min", 4: "avg"}

    def __init__(self, code: int = 0):
        self.code = code

    @staticmethod
    def sum():
        return ReduceOp(0)

    @staticmethod
    def prod():
        return ReduceOp(1)

    @staticmethod
    def max():
        return ReduceOp(2)

    @staticmethod
    def min():
        return ReduceOp(3)

    @staticmethod
    def avg():
        return ReduceOp(4)

    def __str__(self):
        return self._names[self.code]

    def __eq__(self, o):
        return isinstance(o, ReduceOp) and o.code == self.code

    def to_torch(self):
        return {0: dist.ReduceOp.SUM, 1: dist.ReduceOp.PRODUCT, 2: dist.ReduceOp.MAX,
                3: dist.ReduceOp.MIN, 4: dist.ReduceOp.SUM}[self.code]


_STATE = {"backend": "single", "initialized": False}


def _op(op):
    return op if isinstance(op, ReduceOp) else ReduceOp(int(op))


def _ewise(a, b, op):
    """Two-buffer combine by ReduceOp; avg is treated as sum (collective.mojo:115-156)."""
    c = _op(op).code
    if c in (0, 4):
        return a + b
    if c == 1:
        return a * b
    if c == 2:
        return torch.maximum(a, b) if isinstance(a, torch.Tensor) else max(a, b)
    return torch.minimum(a, b) if isinstance(a, torch.Tensor) else min(a, b)


_ewise_int = _ewise_f64 = _ewise


def init_process_group(backend: str = "single", world_size: int = 1, rank: int = 0,
                       timeout_s: float = 600.0, init_method: str | None = None):
    """``backend`` in {"single", "gloo", "nccl"}. "single" asserts world_size == 1 and rank == 0
    like the reference (collective.mojo:74-79)."""
    if backend == "single":
        assert world_size == 1 and rank == 0, "single backend needs world_size == 1, rank == 0"
        _STATE.update(backend="single", initialized=True)
        return
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(backend=backend, rank=rank, world_size=world_size,
                  timeout=datetime.timedelta(seconds=timeout_s))
        if init_method:
            kw["init_method"] = init_method
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(**kw)
    _STATE.update(backend=backend, initialized=True)


def destroy_process_group():
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
    _STATE.update(backend="single", initialized=False)


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def get_world_size() -> int:
    return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1


def get_rank() -> int:
    return dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0


def _as_tensor(x):
    if isinstance(x, torch.Tensor):
        return x, None
    if isinstance(x, (list, tuple)):
        isf = any(isinstance(v, float) for v in x)
        return torch.tensor(list(x), dtype=torch.float64 if isf else torch.int64), "list"
    if isinstance(x, float):
        return torch.tensor([x], dtype=torch.float64), "scalar"
    if isinstance(x, int):
        return torch.tensor([x], dtype=torch.int64), "scalar"
    return None, "object"


def _dev(t):
    if _STATE["backend"] == "nccl" and not t.is_cuda:
        return t.cuda()
    return t


def _back(t, kind, like):
    if kind is None:
        return t
    t = t.cpu()
    if kind == "list":
        return t.tolist()
    return t.item()


def allreduce(x, op=ReduceOp.SUM, group=None):
    if not is_distributed():
        return x
    t, kind = _as_tensor(x)
    if kind == "object":
        return x
    o = _op(op)
    inplace = kind is None
    tt = _dev(t)
    dist.all_reduce(tt, op=o.to_torch(), group=group)
    if o.code == ReduceOp.AVG:
        tt = tt / get_world_size() if not inplace else tt.div_(get_world_size())
    if inplace and tt is not t:
        t.copy_(tt)
        tt = t
    return _back(tt, kind, x)


all_reduce = allreduce


def allreduce_sum(x, group=None):
    return allreduce(x, ReduceOp.SUM, group)


def allreduce_sum_f64(x, group=None):
    return allreduce(x, ReduceOp.SUM, group)


def broadcast(x, src: int = 0, group=None):
    if not is_distributed():
        assert src == 0
        return x
    t, kind = _as_tensor(x)
    if kind == "object":
        objs = [x]
        dist.broadcast_object_list(objs, src=src, group=group)
        return objs[0]
    tt = _dev(t)
    dist.broadcast(tt, src=src, group=group)
    if kind is None and tt is not t:
        t.copy_(tt)
        tt = t
    return _back(tt, kind, x)


def barrier(group=None):
    if is_distributed():
        dist.barrier(group=group)


def reduce(x, op=ReduceOp.SUM, dst: int = 0, group=None):
    if not is_distributed():
        return x
    t, kind = _as_tensor(x)
    tt = _dev(t.clone() if kind is None else t)
    dist.reduce(tt, dst=dst, op=_op(op).to_torch(), group=group)
    if _op(op).code == ReduceOp.AVG and get_rank() == dst:
        tt = tt / get_world_size()
    return _back(tt, kind, x)


reduce_f64 = reduce_list_int = reduce_list_f64 = reduce


# ---- additions -----------------------------------------------------------------------------
def all_gather(x: torch.Tensor, dim: int = 0, group=None) -> torch.Tensor:
    if not is_distributed():
        return x
    W = dist.get_world_size(group)
    xs = _dev(x.contiguous())
    if _STATE["backend"] == "gloo":
        parts = [torch.empty_like(xs) for _ in range(W)]
        dist.all_gather(parts, xs, group=group)
        return torch.cat(parts, dim=dim)
    out = torch.empty((W,) + tuple(xs.shape), dtype=xs.dtype, device=xs.device)
    dist.all_gather_into_tensor(out, xs, group=group)
    return torch.cat(list(out.unbind(0)), dim=dim)


def reduce_scatter(x: torch.Tensor, op=ReduceOp.SUM, dim: int = 0, group=None) -> torch.Tensor:
    """Sum over ranks, each rank keeps its chunk of ``dim``."""
    if not is_distributed():
        return x
    W = dist.get_world_size(group)
    chunks = [c.contiguous() for c in _dev(x).chunk(W, dim=dim)]
    out = torch.empty_like(chunks[0])
    if _STATE["backend"] == "gloo":  # gloo has no reduce_scatter: all-reduce then slice
        full = _dev(x).clone()
        dist.all_reduce(full, op=_op(op).to_torch(), group=group)
        out = full.chunk(W, dim=dim)[dist.get_rank(group)].contiguous()
    else:
        dist.reduce_scatter(out, chunks, op=_op(op).to_torch(), group=group)
    if _op(op).code == ReduceOp.AVG:
        out = out / W
    return out


def all_to_all(x: torch.Tensor, group=None) -> torch.Tensor:
    """Equal split of dim 0: chunk i goes to rank i."""
    if not is_distributed():
        return x
    xs = _dev(x.contiguous())
    out = torch.empty_like(xs)
    if _STATE["backend"] == "gloo":
        W = dist.get_world_size(group)
        ins = list(xs.chunk(W, 0))
        outs = [torch.empty_like(c) for c in ins]
        dist.all_to_all(outs, ins, group=group)
        return torch.cat(outs, 0)
    dist.all_to_all_single(out, xs, group=group)
    return out


def send(x: torch.Tensor, dst: int, group=None, tag: int = 0):
    if is_distributed():
        dist.send(_dev(x.contiguous()), dst=dst, group=group, tag=tag)


def recv(x: torch.Tensor, src: int, group=None, tag: int = 0):
    if is_distributed():
        dist.recv(x, src=src, group=group, tag=tag)
    return x


def isend(x, dst, group=None, tag=0):
    return dist.isend(_dev(x.contiguous()), dst=dst, group=group, tag=tag) if is_distributed() else None


def irecv(x, src, group=None, tag=0):
    return dist.irecv(x, src=src, group=group, tag=tag) if is_distributed() else None
