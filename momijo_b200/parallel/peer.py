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
        self._sig_ptrs = self.peer_ptrs(self.sig)
        self._next_slot = 0
        self._epochs = {}
        self.counters = torch.zeros(64, dtype=torch.int32, device=self.device)
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
        c = self.counters[self._next_counter:self._next_counter + n]
        self._next_counter += n
        return c

    # ---- collectives ----
    def barrier(self, slots: Optional[int] = None):
        """Device-side barrier over the signal pads (stream ordered, bounded wait)."""
        if slots is None:
            if not hasattr(self, "_bar_slots"):
                self._bar_slots = self.new_slots(self.world)
            slots = self._bar_slots
        _C.call("mmj_barrier", self._sig_ptrs, self.world, self.rank, slots, self.next_epoch(slots),
                _C.ptr(self.status), _C.current_stream())

    def all_reduce_(self, t: torch.Tensor, scale: float = 1.0):
        """In-place sum all-reduce of a bf16 tensor that lives in the symmetric heap."""
        if t.dtype != torch.bfloat16:
            raise TypeError("peer all-reduce works on bf16 buffers")
        n = t.numel()
        if n % (8 * self.world):
            raise ValueError("element count must be a multiple of 8 * world")
        if not hasattr(self, "_ar"):
            self._ar = (self.new_slots(3 * self.world), self.new_counter(2), self.new_counter(1))
        slots, ctr, flag = self._ar
        _C.call("mmj_allreduce_bf16", self._sig_ptrs, self.peer_ptrs(t), self.mc_ptr(t), n, scale,
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

    # ---- ZeRO step (called by ShardedDataParallel) ----
    def reduce_scatter_adamw(self, sdp, lr: float):
        flat, o = sdp.flat, sdp.optim
        if not hasattr(sdp, "_rs"):
            sdp._rs = (self.new_slots(2 * self.world), self.new_counter(1))
            sdp._grad_ptrs = self.peer_ptrs(flat.grad)
        slots, ctr = sdp._rs
        a, _ = flat.layout.shard_range(self.rank)
        step = sdp.step_count
        _C.call("mmj_rs_adamw", self._sig_ptrs, sdp._grad_ptrs, self.mc_ptr(flat.grad),
                _C.ptr(flat.param), _C.ptr(sdp.master), _C.ptr(sdp.m), _C.ptr(sdp.v), a,
                flat.layout.shard, lr, o.betas[0], o.betas[1], o.eps, o.weight_decay,
                1.0 - o.betas[0] ** step, 1.0 - o.betas[1] ** step, 1.0, self.world, self.rank,
                slots, self.next_epoch(slots), _C.ptr(ctr), None, _C.ptr(self.status),
                _C.current_stream())

    def all_gather_params(self, sdp, ranges=None):
        """Pull the parameter shards owned by the other ranks (byte ``ranges`` of the flat buffer,
        default: everything)."""
        flat = sdp.flat
        if not hasattr(sdp, "_ag"):
            sdp._ag_slots = self.new_slots(self.world)
            sdp._param_ptrs = self.peer_ptrs(flat.param)
            sdp._ag = {}
        key = None if ranges is None else tuple(map(tuple, ranges))
        dev_ranges = sdp._ag.get(key)
        if dev_ranges is None:
            rs = [(0, flat.layout.total * 2)] if ranges is None else list(ranges)
            dev_ranges = torch.tensor(rs, dtype=torch.int64, device=self.device).reshape(-1)
            sdp._ag[key] = dev_ranges
        # the reduce-scatter kernel ends with a barrier, so no entry barrier is needed (epoch -1)
        _C.call("mmj_allgather_ranges", self._sig_ptrs, sdp._param_ptrs, flat.layout.shard * 2,
                _C.ptr(dev_ranges), dev_ranges.numel() // 2, self.world, self.rank, sdp._ag_slots,
                -1, _C.ptr(self.status), _C.current_stream())
