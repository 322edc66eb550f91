"""Pipeline parallelism: stage wrapper and the 1F1B schedule.

The reference has no pipeline parallelism (legacy/src/momijo/learn/data/pipeline.mojo is an input pipeline;
its process group asserts a single rank, legacy/src/momijo/learn/distributed/collective.mojo:74-78).
Inter-stage activations and gradients travel over torch.distributed point-to-point (NCCL on GPUs,
gloo on CPU) issued asynchronously, so transfers overlap with compute:

* the last stage posts the receive of the next micro-batch's activation before it computes the
  current one;
* in the steady state a stage sends its activation forward and posts the receive of the matching
  gradient in ONE grouped call, so the gradient is already in flight when the backward starts;
* sends are not waited on until their buffers are reused.

All p2p operations of a communicator run in issue order on one stream, so a receive posted early
blocks every later send of this rank until its peer has sent. A middle stage therefore does not
post its forward receive ahead of time (its own forward send could end up queued behind a receive
whose sender is, transitively, waiting for that send); only the last stage, which never sends
forward, does. Inside a stage any module may be used, including tensor-parallel blocks.

1F1B with ``S`` stages and ``m`` micro-batches: stage ``s`` runs ``S - 1 - s`` warm-up forwards,
then alternates one forward / one backward, then drains the remaining backwards; at most
``S - s`` activations are alive per stage and the bubble fraction is ``(S - 1) / (m + S - 1)``.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def partition_layers(n_layers: int, n_stages: int) -> List[range]:
    """Balanced contiguous split (earlier stages take the remainder)."""
    base, rem = divmod(n_layers, n_stages)
    out, s = [], 0
    for i in range(n_stages):
        n = base + (1 if i < rem else 0)
        out.append(range(s, s + n))
        s += n
    return out


class PipelineStage(nn.Module):
    """One pipeline stage: ``module(x) -> y`` (the first stage gets the micro-batch input, the last
    stage's output goes to the loss)."""

    def __init__(self, module: nn.Module, stage: int, n_stages: int, prev_rank: Optional[int] = None,
                 next_rank: Optional[int] = None, group=None):
        super().__init__()
        self.module, self.stage, self.n_stages = module, stage, n_stages
        self.prev_rank, self.next_rank, self.group = prev_rank, next_rank, group
        self.is_first, self.is_last = stage == 0, stage == n_stages - 1

    def forward(self, x):
        return self.module(x)


class _Works:
    def __init__(self, works):
        self.works = list(works)

    def wait(self):
        for w in self.works:
            w.wait()


class Schedule1F1B:
    def __init__(self, stage: PipelineStage, n_micro: int, act_shape, act_dtype=torch.bfloat16, device=None):
        self.stage, self.n_micro = stage, n_micro
        self.act_shape, self.act_dtype = tuple(act_shape), act_dtype
        self.device = device if device is not None else next(stage.parameters()).device
        self._pending = []
        self._connect()

    def _connect(self):
        """Exchange one dummy element with both neighbours in a single grouped call. The first transfer
        between two ranks sets up their connection and blocks the host until the peer takes part; doing it
        here, where every stage issues the matching calls at the same time, keeps that out of the
        schedule, whose sends and receives are deliberately not issued in lock step (a stage whose host
        waits for a connection while its peer's stream waits for that stage's next launch would hang)."""
        st = self.stage
        if not (dist.is_available() and dist.is_initialized()):
            return
        ops, keep = [], []
        for peer in (st.prev_rank, st.next_rank):
            if peer is None:
                continue
            a = torch.zeros(1, dtype=self.act_dtype, device=self.device)
            b = torch.zeros(1, dtype=self.act_dtype, device=self.device)
            keep += [a, b]
            ops.append(dist.P2POp(dist.isend, a, peer, st.group))
            ops.append(dist.P2POp(dist.irecv, b, peer, st.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            if self.device is not None and torch.device(self.device).type == "cuda":
                torch.cuda.synchronize(self.device)

    # ---- p2p helpers ----
    # Every transfer goes through ``batch_isend_irecv`` (a batch of one): with an eagerly initialised
    # NCCL group, bare isend / irecv calls are serialised like collectives of the whole group.
    def _irecv(self, src):
        buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
        works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, buf, src, self.stage.group)])
        return buf, _Works(works)

    def _isend(self, t, dst):
        t = t.contiguous()
        works = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, dst, self.stage.group)])
        self._pending.append((_Works(works), t))
        if len(self._pending) > 4:
            w, _ = self._pending.pop(0)
            w.wait()

    def _drain(self):
        for w, _ in self._pending:
            w.wait()
        self._pending = []

    def run(self, micro_inputs=None, loss_fn: Optional[Callable] = None, micro_targets=None):
        """Run one training step over ``n_micro`` micro-batches; gradients accumulate in the
        parameters. Returns the mean loss on the last stage (None elsewhere)."""
        st, m, S, s = self.stage, self.n_micro, self.stage.n_stages, self.stage.stage
        warm = min(S - 1 - s, m)
        saved = []          # (input, output) pairs awaiting their backward
        losses = []
        fwd_i = bwd_i = 0
        prefetch_fwd = st.is_last   # see the module docstring: safe only where nothing is sent forward
        next_act = self._irecv(st.prev_rank) if (prefetch_fwd and not st.is_first and m > 0) else None
        grad_in_flight = []   # receives of output gradients posted together with the forward send

        def forward_one(steady=False):
            nonlocal fwd_i, next_act
            if st.is_first:
                x = micro_inputs[fwd_i]
            else:
                buf, w = next_act if next_act is not None else self._irecv(st.prev_rank)
                w.wait()
                x = buf.requires_grad_(True)
                next_act = self._irecv(st.prev_rank) if (prefetch_fwd and fwd_i + 1 < m) else None
            y = st(x)
            if st.is_last:
                loss = loss_fn(y, micro_targets[fwd_i]) if loss_fn is not None else y
                losses.append(loss.detach())
                saved.append((x, loss / m))
            else:
                if steady:
                    # send the activation and post the receive of the oldest pending gradient together
                    yd = y.detach().contiguous()
                    gbuf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
                    works = dist.batch_isend_irecv([dist.P2POp(dist.isend, yd, st.next_rank, st.group),
                                                    dist.P2POp(dist.irecv, gbuf, st.next_rank, st.group)])
                    grad_in_flight.append((gbuf, _Works(works), yd))
                else:
                    self._isend(y.detach(), st.next_rank)
                saved.append((x, y))
            fwd_i += 1

        def backward_one():
            nonlocal bwd_i
            x, y = saved.pop(0)
            if st.is_last:
                y.backward()
            else:
                if grad_in_flight:
                    g, w, _keep = grad_in_flight.pop(0)
                else:
                    g, w = self._irecv(st.next_rank)
                w.wait()
                y.backward(g)
            if not st.is_first:
                self._isend(x.grad, st.prev_rank)
            bwd_i += 1

        for _ in range(warm):
            forward_one()
        for _ in range(m - warm):
            forward_one(steady=True)
            backward_one()
        for _ in range(warm):
            backward_one()
        self._drain()
        if st.is_last and losses:
            return torch.stack([l.float() for l in losses]).mean()
        return None

    @staticmethod
    def bubble_fraction(n_stages: int, n_micro: int) -> float:
        return (n_stages - 1) / (n_micro + n_stages - 1)
