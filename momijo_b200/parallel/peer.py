"""Peer-memory runtime: one symmetric heap per rank, peer pointer tables, signal slots, and the
front ends of the collective kernels in ``csrc/comm.cu``.

Bootstrap uses torch.distributed (TCP store + NCCL group) and torch's CUDA symmetric-memory
allocator to map every rank's heap into every other rank's address space (and, where the
hardware offers it, into an NVSwitch multicast object). Everything that moves data afterwards
is this library's own kernels reading and writing peer pointers.

``ProcessGroup`` in the reference is a value struct with ``backend, rank, world_size``
(legacy/src/momijo/learn/distributed/ddp.mojo:18-38); ``PeerComm`` is the handle that struct
was standing in for: communicator + peer window + signal pads.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _C

_ALIGN = 1024


class PeerComm:
    """Symmetric heap + signal slots shared by the ranks of one process group (one node)."""

    SLOTS = 65536

    def __init__(self, group=None, heap_bytes: Optional[int] = None, use_multicast: bool = False):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("PeerComm spans the GPUs of one NVSwitch domain (<= 8 ranks)")
        self.device = torch.device("cuda", torch.cuda.current_device())
        if heap_bytes is None:
            heap_bytes = int(os.environ.get("MOMIJO_PEER_HEAP_MB", "4096")) << 20
        self.heap_bytes = heap_bytes
        try:
            symm.set_backend("CUDA")
        except Exception:
            pass
        self.heap = symm.empty(heap_bytes, dtype=torch.uint8, device=self.device)
        self.hdl = symm.rendezvous(self.heap, self.group)
        self.base_ptrs: List[int] = [int(p) for p in self.hdl.buffer_ptrs]
        self.mc_base = 0
        if use_multicast:
            try:
                if self.hdl.has_multicast_support:
                    self.mc_base = int(self.hdl.multicast_ptr)
            except Exception:
                self.mc_base = 0
        self._off = 0
        self.heap.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.sig = self.alloc(self.SLOTS, torch.int32)
        _C.call("mmj_set_signal_slots", self.SLOTS)   # launchers check their slot ranges against it
        self._sig_ptrs = self.peer_ptrs(self.sig)
        self._next_slot = 0
        self._epochs = {}
        self.counters = torch.zeros(64, dtype=torch.int32, device=self.device)
        self._counter_blocks = []
        self._next_counter = 0
        self.status = _C.status_tensor(self.device)

    # ---- construction helpers ----
    @staticmethod
    def from_default_group(**kw) -> "PeerComm":
        return PeerComm(dist.group.WORLD, **kw)

    # ---- heap ----
    def alloc(self, n: int, dtype: torch.dtype = torch.bfloat16, device=None) -> torch.Tensor:
        """Zero-initialised tensor inside the symmetric heap (same offset on every rank)."""
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self._off + _ALIGN - 1) // _ALIGN * _ALIGN
        if start + nbytes > self.heap_bytes:
            raise MemoryError(f"symmetric heap exhausted: need {start + nbytes} of {self.heap_bytes} bytes "
                              f"(set MOMIJO_PEER_HEAP_MB)")
        self._off = start + nbytes
        return self.heap[start:start + nbytes].view(dtype)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.heap.data_ptr()
        if off < 0 or off >= self.heap_bytes:
            raise ValueError("tensor does not live in the symmetric heap")
        return off

    def peer_ptrs(self, t: torch.Tensor):
        """ctypes array with the address of ``t`` in every rank's heap."""
        off = self.offset_of(t)
        return (ctypes.c_void_p * self.world)(*[b + off for b in self.base_ptrs])

    def mc_ptr(self, t: torch.Tensor):
        return (self.mc_base + self.offset_of(t)) if self.mc_base else None

    # ---- signal slots ----
    def new_slots(self, n: int) -> int:
        base = self._next_slot
        if base + n > self.SLOTS:
            raise RuntimeError("out of signal slots")
        self._next_slot += n
        self._epochs[base] = 0
        return base

    def next_epoch(self, base: int) -> int:
        self._epochs[base] += 1
        return self._epochs[base]

    def new_counter(self, n: int = 1) -> torch.Tensor:
        """``n`` zeroed int32 counters (wrapping block counters / grid flags of one call site)."""
        if self._next_counter + n > self.counters.numel():
            # a fresh block: earlier slices keep pointing into the old tensors, which stay alive
            self._counter_blocks.append(self.counters)
            self.counters = torch.zeros(max(64, n), dtype=torch.int32, device=self.device)
            self._next_counter = 0
        c = self.counters[self._next_counter:self._next_counter + n]
        self._next_counter += n
        return c

    def reset_after_timeout(self):
        """After a bounded wait ran out (``_C.check_status`` raised): blocks that gave up may have left
        wrapping block counters and grid flags mid-count; zero them before the communicator is used
        again. Collective: every rank calls it."""
        for t in self._counter_blocks + [self.counters]:
            t.zero_()
        self.status.zero_()
        self.host_barrier()

    def host_barrier(self):
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # ---- collectives ----
    def barrier(self, slots: Optional[int] = None):
        """Device-side barrier over the signal pads (stream ordered, bounded wait)."""
        if slots is None:
            if not hasattr(self, "_bar_slots"):
                self._bar_slots = self.new_slots(self.world)
            slots = self._bar_slots
        _C.call("mmj_barrier", self._sig_ptrs, self.world, self.rank, slots, self.next_epoch(slots),
                _C.ptr(self.status), _C.current_stream())

    def new_allreduce_state(self):
        """Signal slots, block counters and the grid flag of one all-reduce call site (call sites that may
        run on different streams need one each)."""
        return (self.new_slots(3 * self.world), self.new_counter(2), self.new_counter(1))

    def all_reduce_(self, t: torch.Tensor, scale: float = 1.0, max_blocks: int = 0, state=None):
        """In-place sum all-reduce of a bf16 tensor that lives in the symmetric heap. ``max_blocks`` limits
        the grid of a launch that runs beside other kernels (every block of it must be resident)."""
        if t.dtype != torch.bfloat16:
            raise TypeError("peer all-reduce works on bf16 buffers")
        n = t.numel()
        if n % (8 * self.world):
            raise ValueError("element count must be a multiple of 8 * world")
        if state is None:
            if not hasattr(self, "_ar"):
                self._ar = self.new_allreduce_state()
            state = self._ar
        slots, ctr, flag = state
        _C.call("mmj_allreduce_bf16", self._sig_ptrs, self.peer_ptrs(t), self.mc_ptr(t), n, scale, max_blocks,
                self.world, self.rank, slots, self.next_epoch(slots), _C.ptr(ctr), _C.ptr(flag),
                _C.ptr(self.status), _C.current_stream())
        return t

    def all_gather_rows(self, full: torch.Tensor, site=None):
        """``full`` is a symmetric [rows, cols] buffer whose local row block is filled; pull the
        other ranks' blocks (entry barrier included, so every rank's block is final)."""
        nbytes = full.numel() * full.element_size()
        key = (full.data_ptr(), nbytes)
        if not hasattr(self, "_agr"):
            self._agr = {}
            self._agr_slots = self.new_slots(self.world)
        st = self._agr.get(key)
        if st is None:
            st = (self.peer_ptrs(full),
                  torch.tensor([0, nbytes], dtype=torch.int64, device=self.device))
            self._agr[key] = st
        ptrs, ranges = st
        _C.call("mmj_allgather_ranges", self._sig_ptrs, ptrs, nbytes // self.world, _C.ptr(ranges), 1,
                self.world, self.rank, self._agr_slots, self.next_epoch(self._agr_slots),
                _C.ptr(self.status), _C.current_stream())
        return full

    # ---- bucket operations of ShardedDataParallel ----
    def new_fused_site(self):
        from ..ops.fused_comm import FusedSite

        return FusedSite(self)

    def rs_adamw_bucket(self, eng, b, lr: float, step: int, reduce_only: bool = False, max_blocks: int = 0):
        """Gradient reduce-scatter of bucket ``b`` over peer memory fused with the 1/world scaling and the
        AdamW update of the local shard (one kernel). ``reduce_only``: write the reduced fp32 gradient
        shard and its sum of squares instead of updating (gradient clipping needs the global norm first)."""
        h, o = b.handle, eng.optim
        if "rs" not in h:
            h["rs"] = (self.new_slots(2 * self.world), self.new_counter(1), self.peer_ptrs(b.gview))
        slots, ctr, gptrs = h["rs"]
        shard_off = self.rank * b.shard
        if eng.stage <= 2:
            param_ptr = b.pview.data_ptr()                       # kernel writes at + shard_off
        else:
            param_ptr = eng.pshard.data_ptr() + (b.moff - shard_off) * 2
        mo = b.moff * 4
        _C.call("mmj_rs_adamw", self._sig_ptrs, gptrs, self.mc_ptr(b.gview), param_ptr,
                eng.master.data_ptr() + mo, eng.m.data_ptr() + mo, eng.v.data_ptr() + mo, shard_off, b.shard,
                lr, o.betas[0], o.betas[1], o.eps, o.weight_decay, 1.0 - o.betas[0] ** step,
                1.0 - o.betas[1] ** step, eng.grad_scale, None,
                (eng.reduced.data_ptr() + mo) if reduce_only else None, max_blocks, self.world, self.rank,
                slots, self.next_epoch(slots), _C.ptr(ctr), _C.ptr(eng.gnorm_sq) if reduce_only else None,
                _C.ptr(self.status), _C.current_stream())

    def gather_bucket(self, eng, b, compact: bool, skip=None, max_blocks: int = 0):
        """Pull the shards of bucket ``b`` that other ranks own into ``b.pview``. ``compact``: the peers keep
        only their own shard (``eng.pshard``); otherwise they keep the bucket in the same full layout.
        ``skip``: a byte range of the bucket left to the GEMM that gathers it itself. Follows a kernel
        that ended with a cross-GPU barrier (or an explicit one), so it has no entry barrier."""
        h = b.handle
        key = "gc" if compact else "gf"
        if key not in h:
            src = eng.pshard[b.moff:b.moff + b.shard] if compact else b.pview
            h[key] = self.peer_ptrs(src)
            if not hasattr(self, "_gb_slots"):
                self._gb_slots = self.new_slots(self.world)
        skip_arr = (ctypes.c_longlong * 2)(*skip) if skip is not None else None
        _C.call("mmj_gather_bucket", self._sig_ptrs, h[key], b.pview.data_ptr(), b.shard * 2,
                0 if compact else b.shard * 2, skip_arr, 1 if skip is not None else 0, int(compact),
                max_blocks, self.world, self.rank, self._gb_slots, -1, _C.ptr(self.status),
                _C.current_stream())

    def all_reduce_small(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of a small fp32 tensor (<= 64 values) over the ranks; the same bits on every rank."""
        n = t.numel()
        if not hasattr(self, "_ars"):
            stage = self.alloc(2 * 8 * 64, torch.float32)
            self._ars = (stage, self.peer_ptrs(stage), self.new_slots(self.world))
            self.host_barrier()
        stage, ptrs, slots = self._ars
        out = torch.empty_like(t)
        _C.call("mmj_allreduce_small_f32", self._sig_ptrs, ptrs, _C.ptr(t), _C.ptr(out), n, self.world,
                self.rank, slots, self.next_epoch(slots), _C.ptr(self.status), _C.current_stream())
        return out


class TorchDistComm:
    """The same bucket operations through torch.distributed (gloo on CPU, NCCL on GPUs without peer
    memory): the host-side logic of ``ShardedDataParallel`` (buckets, stages, hooks, clipping) runs and
    is tested with it; the fused peer-memory kernels are ``PeerComm``'s."""

    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)

    def alloc(self, n, dtype=torch.float32, device=None):
        return torch.zeros(n, dtype=dtype, device=device)

    def barrier(self):
        dist.barrier(self.group)

    host_barrier = barrier

    def all_reduce_small(self, t):
        out = t.clone()
        dist.all_reduce(out, group=self.group)
        return out

    def rs_adamw_bucket(self, eng, b, lr, step, reduce_only=False, max_blocks=0):
        from ..ops.optim import adamw_flat

        o = eng.optim
        g = b.gview.float()
        dist.all_reduce(g, group=self.group)
        lo = self.rank * b.shard
        mine = g[lo:lo + b.shard] * (eng.grad_scale / self.world)
        sl = slice(b.moff, b.moff + b.shard)
        if reduce_only:
            eng.reduced[sl].copy_(mine)
            eng.gnorm_sq += mine.pow(2).sum()
            return
        p_out = b.pview[lo:lo + b.shard] if eng.stage <= 2 else eng.pshard[sl]
        adamw_flat(mine, eng.master[sl], eng.m[sl], eng.v[sl], p_out, lr=lr, beta1=o.betas[0], beta2=o.betas[1],
                   eps=o.eps, weight_decay=o.weight_decay, step=step)

    def gather_bucket(self, eng, b, compact, skip=None, max_blocks=0):
        lo = self.rank * b.shard
        mine = (eng.pshard[b.moff:b.moff + b.shard] if compact else b.pview[lo:lo + b.shard]).clone()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        b.pview.copy_(torch.cat(parts))
