"""Sharded data parallelism (ZeRO stages 1-3) over bucketed flat buffers.

``ShardedDataParallel`` wraps a module and re-homes its parameters into flat bf16 storage cut into
*buckets*: one per repeated unit of the model (by default the elements of its largest
``ModuleList``: the decoder blocks) plus one "root" bucket for everything else (embeddings, final
norm). Every bucket is split into ``world`` equal shards; a rank keeps fp32 master weights and AdamW
moments for its shard of every bucket (``partition_1d`` semantics per bucket,
legacy/src/momijo/learn/distributed/sharding.mojo:69-85).

One optimizer step of a bucket is ONE kernel over NVLink peer memory (``csrc/comm.cu``):

  gradient reduce-scatter + 1/world scaling + AdamW on the local shard + bf16 write-back

and it is launched on a side stream as soon as the backward pass of the bucket's unit has finished
(a module backward hook), so that it runs under the backward pass of the earlier units; the
parameter all-gather of the bucket follows on the same stream. Only the root bucket, whose
gradients (tied embedding / LM head) are complete at the very end of the backward pass, is
processed inside ``step()``.

Stages (``stage=``):

1. optimizer state sharded; full gradient and parameter buffers stay resident;
2. gradients sharded as well: unit buckets write their gradients into a small pool of rotating
   bucket-sized buffers (``grad_slots``) that is reused as soon as a bucket's reduce-scatter is done;
3. parameters sharded too: each rank keeps the bf16 shard it owns; unit buckets are gathered into a
   rotating window of ``window`` bucket-sized buffers just before their forward (one unit ahead) and
   again before their backward. The root bucket stays resident between steps.

The weight named by a unit's ``zero_first_gemm_weight`` attribute is left out of the bucket
all-gather that precedes a forward pass: the first GEMM that consumes it pulls the missing pieces
from the peers itself (all-gather fused into the GEMM, ``ops.fused_comm.allgather_gemm``; with
stage 3 from the peers' compact shards into the window slot).

With one rank the same class degenerates to the fused AdamW kernel on one flat buffer.

API parity: ``step_sharded`` / ``zero_grad_sharded`` / ``state_dict_sharded`` follow ``ZeroStage1``
(legacy/src/momijo/learn/distributed/sharding.mojo:164-184); ``step`` keeps the contract of
``DistributedDataParallel.step_and_sync`` = reduce, step, zero
(legacy/src/momijo/learn/distributed/strategies.mojo:218-229).
"""
from __future__ import annotations

import contextlib
import json
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import ops
from .flat import FlatParams

_ALIGN = 128  # elements: parameters start on 256-byte boundaries, shards never split a 16-byte vector


@dataclass
class AdamWConfig:
    lr: float = 1e-3
    betas: Tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0


def default_units(module: nn.Module) -> List[nn.Module]:
    """The elements of the ``ModuleList`` / ``Sequential`` (anywhere in the tree) that holds the most
    parameters: the repeated blocks of a decoder. Empty when the model has no such container."""
    best, best_n = None, 0
    for m in module.modules():
        if isinstance(m, (nn.ModuleList, nn.Sequential)) and len(m) > 1:
            n = sum(p.numel() for p in m.parameters())
            if n > best_n:
                best, best_n = m, n
    return list(best) if best is not None else []


class _Bucket:
    """A contiguous group of parameters that is reduced, updated and gathered as one piece."""

    def __init__(self, idx: int, params: List[nn.Parameter], unit: Optional[nn.Module], world: int):
        self.idx, self.params, self.unit = idx, params, unit
        self.offsets = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        unit_sz = _ALIGN * world
        self.size = (off + unit_sz - 1) // unit_sz * unit_sz
        self.shard = self.size // world
        self.off = 0       # element offset in the full flat layout
        self.moff = 0      # element offset of this bucket's shard in the per-rank shard arrays
        self.gview = None  # [size] gradient storage (full buffer slice or pool slot)
        self.pview = None  # [size] parameter storage (full buffer slice or window slot)
        self.gslot = self.pslot = None
        self.launched = False
        self.done_ev = None    # side stream: reduce-scatter + update (+ gather) of this bucket finished
        self.gather_ev = None  # side stream: parameters of this bucket are in their window slot
        self.use_ev = None     # main stream: last kernel reading this bucket's parameters was issued
        self.fused = None      # (parameter, FusedSite, byte range) of the GEMM-gathered weight
        self.handle = {}       # backend-specific cached arguments


class _FusedWeight:
    """Marks a weight whose all-gather is done by the first GEMM that consumes it."""

    def __init__(self, engine, bucket, site, rel_off_bytes):
        self.engine, self.bucket, self.site, self.rel_off_bytes = engine, bucket, site, rel_off_bytes
        self.pending = False
        self.compact_src = None   # stage 3: peer pointers of the ranks' own shards of this bucket

    def gemm(self, x2, w, bias=None, add_aux=None):
        from ..ops.fused_comm import allgather_gemm

        self.pending = False
        return allgather_gemm(self.site, w, x2, gather_a=False, bias=bias, add_aux=add_aux,
                              bn=ops.pick_bn(x2.shape[0], w.shape[0]), comm_ctas=self.engine.fused_comm_ctas,
                              signal=False, wait_peers=False, shard_bytes=self.bucket.shard * 2,
                              flat_off_bytes=self.rel_off_bytes, compact_src=self.compact_src)


class ShardedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, optim: Optional[AdamWConfig] = None, stage: int = 3,
                 comm=None, grad_clip: Optional[float] = None, params=None, grad_scale: float = 1.0,
                 units: Optional[Sequence[nn.Module]] = None, overlap: bool = True, window: int = 3,
                 grad_slots: int = 3, fuse_first_gemm: bool = True, grad_dtype: Optional[torch.dtype] = None):
        """``comm``: a ``parallel.peer.PeerComm`` (NVLink peer memory, CUDA) or a
        ``parallel.peer.TorchDistComm`` (torch.distributed: gloo on CPU); ``None`` = single rank.
        ``params``: restrict the wrapper to these parameters of ``module`` (default: all of them).
        ``grad_scale``: constant factor on the gradients (a rank that owns its parameters outright but
        whose loss is a per-rank mean needs 1/world here). ``grad_clip``: clip by the global gradient
        norm; the update of every bucket then waits for the norm (reduce-scatter during backward, one
        scalar all-reduce, AdamW afterwards). ``units``: the modules that get a bucket each.
        ``grad_dtype`` (single rank only): torch.float32 accumulates micro-batch gradients in fp32.
        ``overlap``: update each unit's bucket from its backward hook (default). A loop that may decide to
        skip a step after the backward pass (a ``GradScaler`` that found an overflow) needs ``overlap=False``:
        with it every bucket is reduced and updated inside ``step()`` and not calling ``step()`` leaves the
        parameters untouched."""
        super().__init__()
        if stage not in (1, 2, 3):
            raise ValueError("stage must be 1, 2 or 3")
        self.module = module
        self.optim = optim or AdamWConfig()
        self.stage = stage
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.grad_clip = grad_clip
        self.grad_scale = grad_scale
        self.overlap = overlap
        self.lr = self.optim.lr
        self.pre_update_hook = None  # called after gradients are final in the flat buffer, before the update
        self.step_count = 0
        self.fused_comm_ctas = 4
        self.side_blocks = 2 * 148   # grid limit of kernels that run beside the backward pass
        self._sync_enabled = True
        self._accum = None   # stages 2-3: accumulated micro-batch gradients of the unit buckets
        if self.world == 1:
            self._init_single(params, grad_dtype)
        else:
            if grad_dtype not in (None, torch.bfloat16):
                raise NotImplementedError("the peer reduce-scatter kernel reads bf16 gradients")
            self._init_sharded(params, units, window, grad_slots, fuse_first_gemm)

    # ------------------------------------------------------------------------------------------
    # single rank: one flat buffer, fused AdamW
    # ------------------------------------------------------------------------------------------
    def _init_single(self, params, grad_dtype=None):
        self.flat = FlatParams(self.module, 1, 0, alloc=None, params=params, grad_dtype=grad_dtype)
        dev = self.flat.param.device
        n = self.flat.layout.total
        self.master = self.flat.param.float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.buckets = []

    def _step_single(self, lr):
        o = self.optim
        self.flat.zero_untouched()
        if self.pre_update_hook is not None:
            self.pre_update_hook(self)
        self.step_count += 1
        gs_dev = None
        if self.grad_clip is not None:
            ops.sq_norm(self.flat.grad, out=self.gnorm_sq)
            gs_dev = torch.clamp(self.grad_clip / (self.gnorm_sq.sqrt() * abs(self.grad_scale) + 1e-6), max=1.0)
        ops.adamw_flat(self.flat.grad, self.master, self.m, self.v, self.flat.param, lr=lr,
                       beta1=o.betas[0], beta2=o.betas[1], eps=o.eps, weight_decay=o.weight_decay,
                       step=self.step_count, grad_scale=self.grad_scale, grad_scale_dev=gs_dev)
        self.flat.mark_fresh()

    # ------------------------------------------------------------------------------------------
    # sharded: buckets, storage, hooks
    # ------------------------------------------------------------------------------------------
    def _init_sharded(self, params, units, window, grad_slots, fuse_first_gemm):
        comm, W, R = self.comm, self.world, self.rank
        source = list(params) if params is not None else list(self.module.parameters())
        seen, plist = set(), []
        for p in source:
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                plist.append(p)
        if not plist:
            raise ValueError("module has no trainable parameters")
        ids = {id(p) for p in plist}
        unit_modules = list(units) if units is not None else default_units(self.module)
        buckets: List[_Bucket] = []
        taken = set()
        for u in unit_modules:
            ps = [p for p in u.parameters() if id(p) in ids and id(p) not in taken]
            if ps:
                taken.update(id(p) for p in ps)
                buckets.append(_Bucket(len(buckets), ps, u, W))
        root = [p for p in plist if id(p) not in taken]
        self.unit_buckets = list(buckets)
        self.root_bucket = None
        if root:
            self.root_bucket = _Bucket(len(buckets), root, None, W)
            buckets.append(self.root_bucket)
        self.buckets = buckets
        off = moff = 0
        for b in buckets:
            b.off, b.moff = off, moff
            off += b.size
            moff += b.shard
        self.total, self.shard_total = off, moff
        dev = plist[0].device
        self.device = dev
        self.is_cuda = dev.type == "cuda"
        dt = torch.bfloat16 if self.is_cuda else plist[0].dtype
        self.dtype = dt
        esz = torch.empty((), dtype=dt).element_size()
        self.elem_size = esz
        max_unit = max([b.size for b in self.unit_buckets], default=0)
        root_sz = self.root_bucket.size if self.root_bucket is not None else 0
        n_units = len(self.unit_buckets)
        if not self.overlap:
            grad_slots = n_units   # every bucket's gradients stay alive until step()
        self.grad_slots = max(1, min(grad_slots, n_units)) if n_units else 0
        self.window = max(2, min(window, n_units)) if n_units else 0

        # ---- gradient storage ----
        if self.stage == 1:
            self.grad_buf = comm.alloc(self.total, dt, dev)
            for b in buckets:
                b.gview = self.grad_buf[b.off:b.off + b.size]
        else:
            self.grad_buf = comm.alloc(root_sz + self.grad_slots * max_unit, dt, dev)
            for i, b in enumerate(self.unit_buckets):
                b.gslot = i % self.grad_slots
                lo = root_sz + b.gslot * max_unit
                b.gview = self.grad_buf[lo:lo + b.size]
            if self.root_bucket is not None:
                self.root_bucket.gview = self.grad_buf[:root_sz]
        self._gslot_last = [None] * max(1, self.grad_slots)

        # ---- parameter storage ----
        self.pshard = None
        if self.stage <= 2:
            self.param_buf = comm.alloc(self.total, dt, dev)
            for b in buckets:
                b.pview = self.param_buf[b.off:b.off + b.size]
        else:
            self.pshard = comm.alloc(self.shard_total, dt, dev)
            self.param_buf = torch.zeros(root_sz + self.window * max_unit, dtype=dt, device=dev)
            for i, b in enumerate(self.unit_buckets):
                b.pslot = i % self.window
                lo = root_sz + b.pslot * max_unit
                b.pview = self.param_buf[lo:lo + b.size]
            if self.root_bucket is not None:
                self.root_bucket.pview = self.param_buf[:root_sz]
        self._pslot_holds = [None] * max(1, self.window)

        # ---- optimizer state for the local shards ----
        self.master = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        self.m = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        self.reduced = torch.zeros(self.shard_total, dtype=torch.float32, device=dev) \
            if self.grad_clip is not None else None
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)

        # ---- initial values, re-homing ----
        with torch.no_grad():
            for b in buckets:
                tmp = torch.zeros(b.size, dtype=dt, device=dev)
                for p, o in zip(b.params, b.offsets):
                    tmp[o:o + p.numel()].copy_(p.detach().reshape(-1).to(dt))
                mine = tmp[R * b.shard:(R + 1) * b.shard]
                self.master[b.moff:b.moff + b.shard].copy_(mine.float())
                if self.pshard is not None:
                    self.pshard[b.moff:b.moff + b.shard].copy_(mine)
                if self.stage <= 2 or b.unit is None:
                    b.pview.copy_(tmp)
                for p, o in zip(b.params, b.offsets):
                    p.data = b.pview[o:o + p.numel()].view(p.shape)
                    p.main_grad = b.gview[o:o + p.numel()].view(p.shape)
                    p._mg_fresh = True
                del tmp
        self.params = plist

        # ---- streams, events, hooks ----
        if self.is_cuda:
            self.side = torch.cuda.Stream(device=dev)
            for b in buckets:
                b.done_ev, b.gather_ev, b.use_ev = (torch.cuda.Event() for _ in range(3))
        else:
            self.side = None
        for i, b in enumerate(self.unit_buckets):
            u = b.unit
            u.register_forward_pre_hook(self._make_pre_forward(i))
            u.register_forward_hook(self._make_post_forward(i))
            u.register_full_backward_pre_hook(self._make_pre_backward(i))
            u.register_full_backward_hook(self._make_post_backward(i))

        # ---- GEMM-fused all-gather of each unit's first weight (CUDA peer memory) ----
        if fuse_first_gemm and self.is_cuda and hasattr(comm, "new_fused_site"):
            for b in self.unit_buckets:
                name = getattr(b.unit, "zero_first_gemm_weight", None)
                w = getattr(b.unit, name, None) if name else None
                if w is None or not any(w is p for p in b.params) or w.dim() != 2:
                    continue
                o = b.offsets[[i for i, p in enumerate(b.params) if p is w][0]]
                fw = _FusedWeight(self, b, comm.new_fused_site(), o * esz)
                if self.stage == 3:
                    fw.compact_src = comm.peer_ptrs(self.pshard[b.moff:b.moff + b.shard])
                b.fused = (w, fw, (o * esz, (o + w.numel()) * esz))
                w._zero_gather = fw
        comm.host_barrier()

    # ---- hooks ----
    def _make_pre_forward(self, i):
        def hook(module, args):
            if self.stage == 3:
                b = self.unit_buckets[i]
                self._ensure_params(b, forward=True)
                if i + 1 < len(self.unit_buckets):
                    self._gather_params(self.unit_buckets[i + 1], forward=True)
        return hook

    def _make_post_forward(self, i):
        def hook(module, args, output):
            if self.stage == 3 and self.is_cuda:
                self.unit_buckets[i].use_ev.record()
        return hook

    def _make_pre_backward(self, i):
        def hook(module, grad_output):
            b = self.unit_buckets[i]
            if self.stage == 3:
                self._ensure_params(b)
                if i > 0:
                    self._gather_params(self.unit_buckets[i - 1])
            if self.stage >= 2:
                prev = self._gslot_last[b.gslot]
                if prev is not None and prev is not b and self.is_cuda:
                    # the pool slot is free once the previous bucket's reduce-scatter has read it
                    torch.cuda.current_stream().wait_event(prev.done_ev)
                self._gslot_last[b.gslot] = b
        return hook

    def _make_post_backward(self, i):
        def hook(module, grad_input, grad_output):
            b = self.unit_buckets[i]
            if self.stage == 3 and self.is_cuda:
                b.use_ev.record()
            if not self._sync_enabled:
                if self.stage >= 2:
                    self._stash_micro_batch(b)
                return
            if self.overlap and not b.launched:
                self._launch(b)
        return hook

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context only accumulate gradients (gradient accumulation over
        micro-batches); the last backward pass runs outside it and is followed by ``step()``.

        Stage 1 keeps the full gradient buffer anyway and the kernels add into it. Stages 2 and 3 hold a
        unit's gradients only in a rotating pool slot, so inside this context every unit's gradients are
        moved, right after its backward pass, into a full-size accumulation buffer that exists only while
        micro-batches are being accumulated (it is allocated on first use and released by ``step()``); the
        last backward pass adds the accumulated part back before its reduce-scatter. The memory saving of
        stage 2 therefore does not hold during accumulation."""
        old, self._sync_enabled = self._sync_enabled, False
        try:
            yield
        finally:
            self._sync_enabled = old

    def _stash_micro_batch(self, b: _Bucket):
        """Move the gradients of unit bucket ``b`` (in its pool slot) into the accumulation buffer and mark
        the slot as free for the next writer."""
        self._finalize_grads(b)
        if self._accum is None:
            self._accum = torch.zeros(sum(u.size for u in self.unit_buckets), dtype=self.dtype, device=self.device)
            self._accum_off, off = {}, 0
            for u in self.unit_buckets:
                self._accum_off[u.idx] = off
                off += u.size
        o = self._accum_off[b.idx]
        self._accum[o:o + b.size].add_(b.gview)
        for p in b.params:
            p._mg_fresh = True   # the next micro-batch starts this slot afresh

    # ---- parameter window (stage 3) ----
    def _gather_params(self, b: _Bucket, forward: bool = False):
        """Bring bucket ``b`` into its window slot (side stream). Before a forward pass the weight that
        its first GEMM gathers itself is left out; before a backward pass everything is fetched."""
        slot = b.pslot
        occ = self._pslot_holds[slot]
        if occ is b:
            return
        fuse = forward and b.fused is not None
        with self._side():
            if occ is not None and self.is_cuda:
                self.side.wait_event(occ.use_ev)
            self.comm.gather_bucket(self, b, compact=True, skip=b.fused[2] if fuse else None)
            if self.is_cuda:
                b.gather_ev.record(self.side)
        if b.fused is not None:
            b.fused[1].pending = fuse
        self._pslot_holds[slot] = b

    def _ensure_params(self, b: _Bucket, forward: bool = False):
        self._gather_params(b, forward)
        if self.is_cuda:
            torch.cuda.current_stream().wait_event(b.gather_ev)

    @contextlib.contextmanager
    def _side(self):
        if self.side is None:
            yield
        else:
            with torch.cuda.stream(self.side):
                yield

    # ---- one bucket: reduce-scatter + update (+ gather) on the side stream ----
    def _finalize_grads(self, b: _Bucket):
        """Fold gradients that arrived through autograd's ``.grad``; zero what received nothing."""
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

    def _launch(self, b: _Bucket):
        self._finalize_grads(b)
        if self._accum is not None and b.unit is not None:
            o = self._accum_off[b.idx]
            b.gview.add_(self._accum[o:o + b.size])
        clip = self.grad_clip is not None
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
        with self._side():
            if self.is_cuda:
                self.side.wait_event(ev)
            self.comm.rs_adamw_bucket(self, b, self.lr, self.step_count + 1, reduce_only=clip,
                                      max_blocks=self.side_blocks)
            if not clip:
                self._after_update(b)
            if self.is_cuda:
                b.done_ev.record(self.side)
        b.launched = True

    def _after_update(self, b: _Bucket):
        """Parameters of the next step: stages 1-2 refill the full buffer now; stage 3 keeps the shard
        and gathers on demand (the root bucket, needed first and last, is gathered right away)."""
        if self.stage <= 2:
            self.comm.gather_bucket(self, b, compact=False, skip=b.fused[2] if b.fused else None,
                                    max_blocks=self.side_blocks)
            if b.fused:
                b.fused[1].pending = True
        elif b.unit is None:
            self.comm.gather_bucket(self, b, compact=True)

    # ---- public step ----
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def set_lr(self, lr: float):
        """Learning rate of the following steps (buckets updated during a backward pass use the rate
        that was set before that pass)."""
        self.lr = float(lr)

    def zero_grad_sharded(self):
        if self.world == 1:
            self.flat.mark_fresh()
        else:
            for p in self.params:
                p._mg_fresh = True

    zero_grad = zero_grad_sharded

    def step_sharded(self, lr: Optional[float] = None):
        return self.step(lr)

    def step(self, lr: Optional[float] = None):
        """Reduce gradients across ranks, update the local shards, republish bf16 parameters."""
        if lr is not None and float(lr) != self.lr:
            if self.world > 1 and any(b.launched for b in self.buckets):
                raise RuntimeError("buckets of this step were already updated with the previous learning rate "
                                   "during the backward pass: call set_lr() before backward()")
            self.lr = float(lr)
        if self.world == 1:
            return self._step_single(self.lr)
        if self.pre_update_hook is not None:
            self.pre_update_hook(self)
        for b in self.buckets:
            if b.launched:
                for p in b.params:
                    if p.grad is not None:
                        raise RuntimeError(
                            "a parameter of an overlapped bucket received its gradient through autograd's .grad "
                            "after the bucket was reduced; construct the engine with overlap=False")
        for b in reversed(self.buckets):
            if not b.launched:
                self._launch(b)
        if self.grad_clip is not None:
            self._clipped_update()
        if self.is_cuda:
            torch.cuda.current_stream().wait_stream(self.side)
        self.step_count += 1
        self._accum = None
        for b in self.buckets:
            b.launched = False
        if self.stage == 3:
            # window slots hold pre-update parameters now
            self._pslot_holds = [None] * len(self._pslot_holds)
        for p in self.params:
            p._mg_fresh = True

    def _clipped_update(self):
        """All buckets have been reduced into ``self.reduced`` (fp32 shards) and the local sum of squares
        accumulated: combine the norm over ranks, then update every bucket with the clip factor."""
        o = self.optim
        with self._side():
            total = self.comm.all_reduce_small(self.gnorm_sq)
            factor = torch.clamp(self.grad_clip / (total.sqrt() + 1e-6), max=1.0)
            for b in self.buckets:
                sl = slice(b.moff, b.moff + b.shard)
                if self.stage <= 2:
                    p_out = b.pview[self.rank * b.shard:(self.rank + 1) * b.shard]
                else:
                    p_out = self.pshard[sl]
                ops.adamw_flat(self.reduced[sl], self.master[sl], self.m[sl], self.v[sl], p_out, lr=self.lr,
                               beta1=o.betas[0], beta2=o.betas[1], eps=o.eps, weight_decay=o.weight_decay,
                               step=self.step_count + 1, grad_scale=1.0, grad_scale_dev=factor)
            self.comm.barrier()   # every rank's shards are final before anyone gathers
            for b in self.buckets:
                self._after_update(b)
            self.gnorm_sq.zero_()

    # ---- inspection ----
    def materialize(self) -> dict:
        """name -> full parameter tensor (a copy), whatever the stage; collective over the ranks."""
        names = {id(p): n for n, p in self.module.named_parameters()}
        out = {}
        if self.world == 1:
            for p in self.flat.params:
                out[names[id(p)]] = p.detach().clone()
            return out
        if self.is_cuda:
            torch.cuda.current_stream().wait_stream(self.side)
        for b in self.buckets:
            if self.stage == 3 and b.unit is not None:
                self._ensure_params(b)
            elif b.fused and b.fused[1].pending:
                self.comm.gather_bucket(self, b, compact=False)
                b.fused[1].pending = False
            if self.is_cuda:
                torch.cuda.synchronize()
            for p, o in zip(b.params, b.offsets):
                out[names[id(p)]] = b.pview[o:o + p.numel()].view(p.shape).detach().clone()
            if self.stage == 3 and b.unit is not None and self.is_cuda:
                b.use_ev.record()
        return out

    def memory_report(self) -> dict:
        """Bytes this rank keeps resident for parameters, gradients and optimizer state."""
        if self.world == 1:
            n = self.flat.layout.total
            return {"stage": self.stage, "world": 1, "param_bytes": n * 2, "grad_bytes": n * 2,
                    "optimizer_bytes": n * 12}
        esz = self.elem_size
        pbytes = self.param_buf.numel() * esz + (self.pshard.numel() * esz if self.pshard is not None else 0)
        rep = {"stage": self.stage, "world": self.world, "buckets": len(self.buckets),
               "param_bytes": pbytes, "grad_bytes": self.grad_buf.numel() * esz,
               "optimizer_bytes": self.shard_total * 12 + (self.shard_total * 4 if self.reduced is not None else 0),
               "unsharded_param_bytes": self.total * esz}
        if self.is_cuda:
            rep["torch_max_allocated"] = torch.cuda.max_memory_allocated()
        return rep

    def state_dict_sharded(self) -> str:
        """Same JSON shape as ``ZeroStage1.state_dict``."""
        return json.dumps({"world_size": self.world, "rank": self.rank})

    # ---- checkpoint / resume ----
    def is_cuda_engine(self) -> bool:
        return bool(self.is_cuda) if self.world > 1 else self.flat.param.is_cuda

    def save_checkpoint(self, base: str, extra: Optional[dict] = None) -> None:
        """Optimizer state (fp32 master weights, AdamW moments, step count) as an MNP checkpoint, one blob per
        rank (``<base>.rank<r>of<W>.bin``); every rank calls it. See ``parallel.zero_ckpt``."""
        from . import zero_ckpt

        if self.world > 1 and self.is_cuda:
            torch.cuda.current_stream().wait_stream(self.side)
        zero_ckpt.save(self, base, extra)

    def load_checkpoint(self, base: str) -> dict:
        """Restore from ``save_checkpoint`` output of a run with any world size (the per-parameter pieces are
        re-split for this run's shards), rebuild the bf16 parameters from the master weights, return ``extra``."""
        from . import zero_ckpt

        return zero_ckpt.load(self, base)

    def load_full_parameters(self, named: dict, reset_moments: bool = True) -> None:
        """Take parameter values from full tensors (``name -> tensor`` as ``module.named_parameters()`` names
        them: a pretrained model, ``materialize()`` of another engine): every rank copies the pieces it owns
        into its fp32 master weights, the AdamW moments restart from zero unless told otherwise, and the bf16
        parameters are republished. Collective."""
        from .zero_ckpt import owned_pieces

        with torch.no_grad():
            for name, lo, hi, at in owned_pieces(self):
                src = named[name].detach().reshape(-1)[lo:hi]
                self.master[at:at + hi - lo].copy_(src.to(device=self.master.device, dtype=torch.float32))
            if reset_moments:
                self.m.zero_()
                self.v.zero_()
        self.republish_from_master()

    def save_weights(self, base: str, extra: Optional[dict] = None) -> None:
        """The model's parameters as ONE ordinary MNP checkpoint (``<base>.json`` + ``<base>.bin``, tensors under
        their ``named_parameters`` names), whatever the stage: rank 0 writes what ``materialize()`` collects,
        so that ``learn.utils.checkpoint.load_state_dict`` of an unsharded model, or ``load_weights`` of an
        engine of any world size, can read it. Collective."""
        from ..learn.utils.checkpoint import save_state_dict
        from .zero_ckpt import _State

        full = self.materialize()
        if self.rank == 0:
            import os
            d = os.path.dirname(base)
            if d:
                os.makedirs(d, exist_ok=True)
            save_state_dict(_State(full), base, extra=extra)
        if self.world > 1:
            self.comm.host_barrier()

    def load_weights(self, base: str, reset_moments: bool = True) -> dict:
        """Read a ``save_weights`` file (or any MNP checkpoint whose tensors carry this module's parameter
        names) into the engine; returns the file's ``extra``. Collective."""
        import json as _json
        from ..learn.utils.checkpoint import read_blob_tensor

        h = _json.load(open(base + ".json"))
        blob = h["files"]["blob"]
        import os
        if not os.path.exists(blob):
            blob = base + ".bin"
        named = {e["name"]: read_blob_tensor(blob, e) for e in h.get("tensors", [])}
        self.load_full_parameters(named, reset_moments)
        return h.get("extra", {})

    def republish_from_master(self) -> None:
        """bf16 parameters := fp32 master weights, on every rank (after a load, or after editing the master
        weights in place). Collective."""
        with torch.no_grad():
            if self.world == 1:
                self.flat.param.copy_(self.master.to(self.flat.param.dtype))
                self.flat.mark_fresh()
                return
            R = self.rank
            if self.is_cuda:
                torch.cuda.current_stream().wait_stream(self.side)
            for b in self.buckets:
                mine = self.master[b.moff:b.moff + b.shard].to(self.dtype)
                if self.pshard is not None:
                    self.pshard[b.moff:b.moff + b.shard].copy_(mine)
                if self.stage <= 2:
                    b.pview[R * b.shard:(R + 1) * b.shard].copy_(mine)
            if self.is_cuda:
                ev = torch.cuda.Event()
                ev.record()
            with self._side():
                if self.is_cuda:
                    self.side.wait_event(ev)
                self.comm.barrier()   # every rank's shards are in place before anyone gathers
                for b in self.buckets:
                    self._after_update(b)
            if self.is_cuda:
                torch.cuda.current_stream().wait_stream(self.side)
            if self.stage == 3:
                self._pslot_holds = [None] * len(self._pslot_holds)
            for b in self.buckets:
                b.launched = False
            for p in self.params:
                p._mg_fresh = True
