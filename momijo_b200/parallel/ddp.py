"""Data-parallel wrapper over flat gradient storage, with bucketed gradient all-reduce overlapped
with the backward pass.

``DistributedDataParallel`` keeps parameters and gradients in two flat buffers (``FlatParams``). The
gradient buffer is cut into buckets: one per repeated unit of the model (the elements of its largest
``ModuleList``, whose parameters are contiguous in the flat layout) and the remainder. When the
backward pass of a unit has finished (a module backward hook), the all-reduce of its bucket starts
on a side stream and runs under the backward pass of the earlier units (buckets of plain torch
modules, whose gradients arrive through autograd's ``.grad``, start when the last of their gradients
has been accumulated; how a bucket's gradients arrive is learned on the first step, which reduces
everything inside ``step``): with a peer communicator it
is this library's two-shot all-reduce kernel over NVLink peer memory (launched with a reduced grid
so that it fits beside the GEMMs), otherwise an asynchronous torch.distributed all-reduce (gloo on
CPU). ``step`` reduces what is left (the root bucket, and everything on the first step or when
``overlap=False``), waits for the buckets in flight and applies the same fused AdamW step to the
full buffers on every rank.

Reference shape: ``DDP.wrap`` / ``allreduce_grads_mean``
(legacy/src/momijo/learn/distributed/ddp.mojo:52-105) and
``DistributedDataParallel.step_and_sync`` (legacy/src/momijo/learn/distributed/strategies.mojo:218-229),
which skips the update when an inf was found; the reference reduces one opaque blob after the
backward pass, without buckets.
"""
from __future__ import annotations

import contextlib
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from .flat import FlatParams
from .zero import AdamWConfig, default_units


class _GradBucket:
    def __init__(self, lo: int, hi: int, params, unit):
        self.lo, self.hi, self.params, self.unit = lo, hi, params, unit
        self.launched = False
        self.work = None      # torch.distributed async handle
        self.state = None     # peer all-reduce call-site state
        # How this bucket's gradients arrive, learned on the first step: "native" (the backward kernels
        # write main_grad; ready when the unit's backward hook fires), "autograd" (every gradient comes
        # through .grad; ready when the last of them has been accumulated), or None (mixed: no overlap).
        self.mode = None
        self.n_autograd = 0
        self.pending = 0


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, optim: Optional[AdamWConfig] = None, comm=None, group=None,
                 dtype: torch.dtype = None, overlap: bool = True, units=None):
        super().__init__()
        self.module, self.comm, self.group = module, comm, group
        self.optim = optim or AdamWConfig()
        if comm is not None:
            self.world, self.rank = comm.world, comm.rank
        elif dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        p0 = next(module.parameters())
        dtype = dtype or (torch.bfloat16 if p0.is_cuda else p0.dtype)
        alloc = comm.alloc if comm is not None else None
        # total padded to 8 * world elements: the all-reduce kernel works on 16-byte vectors per rank
        self.flat = FlatParams(module, self.world, self.rank, alloc=alloc, dtype=dtype)
        n = self.flat.layout.total
        dev = self.flat.param.device
        self.master = self.flat.param.float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overlap = overlap and self.world > 1
        self._sync_enabled = True
        self.is_cuda = dev.type == "cuda"
        self.side = torch.cuda.Stream(device=dev) if (self.is_cuda and self.world > 1) else None
        self.side_blocks = 148
        self.buckets: List[_GradBucket] = self._make_buckets(units)
        self._learned = False
        for b in self.buckets:
            if b.unit is not None:
                b.unit.register_full_backward_hook(self._make_hook(b))
                for p in b.params:
                    p.register_post_accumulate_grad_hook(self._make_param_hook(b))

    # ---- buckets ----
    def _make_buckets(self, units) -> List[_GradBucket]:
        """Contiguous ranges of the flat gradient buffer: one per unit whose parameters are contiguous
        there, and the gaps between them."""
        lay = self.flat.layout
        off_of = {id(p): o for p, o in zip(lay.params, lay.offsets)}
        ends = list(lay.offsets[1:]) + [lay.total]
        end_of = {id(p): e for p, e in zip(lay.params, ends)}
        spans = []
        for u in (list(units) if units is not None else default_units(self.module)):
            ps = [p for p in u.parameters() if id(p) in off_of]
            if not ps:
                continue
            lo, hi = min(off_of[id(p)] for p in ps), max(end_of[id(p)] for p in ps)
            inside = [p for p in lay.params if lo <= off_of[id(p)] < hi]
            if len(inside) == len(ps) and (hi - lo) % (8 * self.world) == 0 and lo % 8 == 0:
                spans.append((lo, hi, ps, u))
        spans.sort(key=lambda s: s[0])
        out, cur = [], 0
        for lo, hi, ps, u in spans:
            if lo < cur:
                continue   # overlapping units: keep the first
            if lo > cur:
                out.append(_GradBucket(cur, lo, [p for p in lay.params if cur <= off_of[id(p)] < lo], None))
            out.append(_GradBucket(lo, hi, ps, u))
            cur = hi
        if cur < lay.total:
            out.append(_GradBucket(cur, lay.total, [p for p in lay.params if off_of[id(p)] >= cur], None))
        return out

    def _make_hook(self, b):
        def hook(module, grad_input, grad_output):
            if self.overlap and self._sync_enabled and self._learned and b.mode == "native" and not b.launched:
                self._launch(b)
        return hook

    def _make_param_hook(self, b):
        def hook(p):
            if p.grad is None:
                return   # the gradient went into main_grad; autograd had nothing to accumulate
            if not self._learned:
                b.n_autograd += 1
            elif self.overlap and self._sync_enabled and b.mode == "autograd" and not b.launched:
                b.pending -= 1
                if b.pending == 0:
                    self._launch(b)
        return hook

    def _learn_modes(self):
        for b in self.buckets:
            if b.unit is None:
                continue
            if b.n_autograd == 0 and all(not p._mg_fresh for p in b.params):
                b.mode = "native"       # every gradient was written into main_grad by a backward kernel
            elif b.n_autograd == len(b.params) and all(p._mg_fresh for p in b.params):
                b.mode = "autograd"     # every gradient came through .grad
            b.pending = b.n_autograd
        self._learned = True

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate gradients (micro-batches)."""
        old, self._sync_enabled = self._sync_enabled, False
        try:
            yield
        finally:
            self._sync_enabled = old

    def _finalize(self, b):
        for p in b.params:
            if p.grad is not None:
                g = p.grad.to(p.main_grad.dtype)
                if p._mg_fresh:
                    p.main_grad.copy_(g)
                else:
                    p.main_grad.add_(g)
                p.grad = None
                p._mg_fresh = False
            if p._mg_fresh:
                p.main_grad.zero_()
                p._mg_fresh = False

    def _launch(self, b):
        """Average bucket ``b`` over the ranks (in place), without blocking the launching stream."""
        self._finalize(b)
        view = self.flat.grad[b.lo:b.hi]
        if self.comm is not None and view.dtype == torch.bfloat16 and (b.hi - b.lo) % (8 * self.world) == 0:
            if b.state is None:
                b.state = self.comm.new_allreduce_state()
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.side):
                self.side.wait_event(ev)
                self.comm.all_reduce_(view, scale=1.0 / self.world, max_blocks=self.side_blocks, state=b.state)
        else:
            if self.is_cuda:
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(self.side):
                    self.side.wait_event(ev)
                    dist.all_reduce(view, group=self.group)
                    view.div_(self.world)
            else:
                b.work = dist.all_reduce(view, group=self.group, async_op=True)
        b.launched = True

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def sync_gradients(self):
        """Average gradients over the data-parallel group (in place in the flat buffer): reduces the
        buckets that the backward pass has not already sent off and waits for all of them."""
        if self.world == 1:
            self.flat.zero_untouched()
            return
        if not self._learned and self._sync_enabled:
            self._learn_modes()
        for b in self.buckets:
            if b.launched:
                for p in b.params:
                    if p.grad is not None:
                        raise RuntimeError("a parameter of an overlapped bucket received its gradient through "
                                           "autograd's .grad after the bucket was reduced; use overlap=False")
        for b in reversed(self.buckets):
            if not b.launched:
                self._launch(b)
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                self.flat.grad[b.lo:b.hi].div_(self.world)
                b.work = None
            b.launched = False
            b.pending = b.n_autograd
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)

    def step(self, lr: Optional[float] = None, found_inf: bool = False):
        self.sync_gradients()
        if found_inf:  # same protocol as GradScaler.step: skip the update, keep the state
            self.flat.mark_fresh()
            return False
        o = self.optim
        self.step_count += 1
        ops.adamw_flat(self.flat.grad, self.master, self.m, self.v, self.flat.param, lr=o.lr if lr is None else lr,
                       beta1=o.betas[0], beta2=o.betas[1], eps=o.eps, weight_decay=o.weight_decay,
                       step=self.step_count)
        self.flat.mark_fresh()
        return True

    step_and_sync = step

    # ---- checkpoint / resume ----
    def save_checkpoint(self, base: str, extra: Optional[dict] = None) -> None:
        """Every rank holds the same optimizer state, so rank 0 writes it (MNP layout, per-parameter
        ``master`` / ``m`` / ``v`` tensors, step count in ``extra``) and the others wait. The file can also be
        read by ``ShardedDataParallel.load_checkpoint`` of any world size."""
        from . import zero_ckpt

        if self.rank == 0:
            zero_ckpt.save_replicated(self, base, extra)
        if self.world > 1:
            if self.comm is not None:
                self.comm.host_barrier()
            else:
                dist.barrier(self.group)

    def load_checkpoint(self, base: str) -> dict:
        """Restore from ``save_checkpoint`` (or from a sharded engine's checkpoint of any world size) and rebuild
        the bf16 parameters from the master weights."""
        from . import zero_ckpt

        extra = zero_ckpt.read_into(self, base, zero_ckpt.flat_pieces(self))
        self.step_count = int(extra.get("step_count", self.step_count))
        with torch.no_grad():
            self.flat.param.copy_(self.master.to(self.flat.param.dtype))
        self.flat.mark_fresh()
        return extra

    def zero_grad(self):
        self.flat.mark_fresh()
