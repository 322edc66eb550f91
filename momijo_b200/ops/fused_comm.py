"""Front ends of the fused compute + communication kernels (GEMM with an in-kernel all-gather,
GEMM with a reduce-scatter epilogue) and of the MoE dispatch / combine kernels.

All buffers that peers touch live in the symmetric heap of a ``PeerComm``. A call site owns a
small amount of state (flags, signal slots, epoch counter) kept in a ``FusedSite``.

No counterpart in the reference: its collectives return their input unchanged
(legacy/src/momijo/learn/distributed/collective.mojo:163-232) and its sharding helpers only slice lists
(legacy/src/momijo/learn/distributed/sharding.mojo:130-168); these are the kernels that stand where
``allgather_list`` / ``reduce_scatter_list`` would move data.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _C
from .gemm import TALL, pick_tall, pick_bn, EPI_BIAS, EPI_GELU, EPI_ADD_AUX

bf16 = torch.bfloat16


class FusedSite:
    """Per call-site state for the fused kernels: flag array, signal slots, epoch."""

    def __init__(self, comm, n_flags: int = 4096):
        self.comm = comm
        self.flags = torch.zeros(n_flags, dtype=torch.int32, device=comm.device)
        self.slots = comm.new_slots(2 * comm.world)
        self.epoch = 0
        self.ptr_cache = {}

    def peer_ptrs(self, t):
        key = (t.data_ptr(), t.numel())
        p = self.ptr_cache.get(key)
        if p is None:
            p = self.comm.peer_ptrs(t)
            self.ptr_cache[key] = p
        return p


def signal_shard_ready(site: FusedSite, epoch: int):
    """Tell every peer that this rank's shard for `epoch` is final (stream ordered)."""
    c = site.comm
    _C.call("mmj_signal_peers", c._sig_ptrs, c.world, c.rank, site.slots + c.rank, epoch,
            _C.current_stream())


def allgather_gemm(site: FusedSite, gathered, other, *, gather_a=True, other_mn=False, out=None,
                   bias=None, gelu=False, pre_out=None, add_aux=None, bn=None, comm_ctas=8, tall=None,
                   signal=True, shard_bytes=None, flat_off_bytes=0, wait_peers=True, compact_src=None):
    """D = A @ B^T where one operand is the row-wise concatenation of per-rank shards.

    ``gathered``: symmetric [rows, K] bf16 buffer whose local part is already filled; the kernel
    pulls the other parts while it computes. By default rank r owns rows ``r*rows/world ..``;
    with ``shard_bytes``/``flat_off_bytes`` the matrix is a window of a flat buffer sharded in
    equal byte ranges (ZeRO parameters). ``other`` is the local operand ([N, K], or [K, N] with
    ``other_mn``; for ``gather_a=False`` it plays the role of A).
    ``compact_src``: peer pointer table of the ranks' own shards when every rank keeps only its shard
    (stage-3 parameters); ``gathered`` is then a local buffer that receives the local piece too.
    After the call ``gathered`` holds the full matrix (reusable by the backward pass).
    """
    c = site.comm
    rows, K = gathered.shape
    if shard_bytes is None:
        shard_bytes = (rows // c.world) * gathered.stride(0) * 2
    if gather_a:
        M = rows
        N = other.shape[1] if other_mn else other.shape[0]
    else:
        N = rows
        M = other.shape[1] if other_mn else other.shape[0]
    if bn is None:
        if tall is None:
            tall = pick_tall(M, N, K) and M % 256 == 0 and (not gather_a or (rows // c.world) % 256 == 0)
        bn = 256 if tall else pick_bn(M, N)
        if not gather_a:
            while (rows // c.world) % bn and bn > 64:
                bn //= 2
    if out is None:
        out = torch.empty((M, N), dtype=bf16, device=gathered.device)
    if gelu and pre_out is None:
        pre_out = torch.empty((M, N), dtype=bf16, device=gathered.device)
    epi = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0) | (
        EPI_ADD_AUX if add_aux is not None else 0)
    site.epoch += 1
    if signal:
        signal_shard_ready(site, site.epoch)
    peer_ready = (c.sig.data_ptr() + 4 * site.slots) if wait_peers else None
    n_tiles = -(-rows // (128 if gather_a else bn))
    if n_tiles > site.flags.numel():
        site.flags = torch.zeros(n_tiles, dtype=torch.int32, device=c.device)
    _C.call("mmj_gemm_bf16_allgather", compact_src if compact_src is not None else site.peer_ptrs(gathered),
            _C.ptr(gathered), int(gather_a) | (2 if compact_src is not None else 0),
            _C.ptr(other), gathered.stride(0), other.stride(0), int(other_mn), _C.ptr(out),
            out.stride(0), M, N, K, epi, _C.ptr(bias), _C.ptr(add_aux),
            add_aux.stride(0) if add_aux is not None else 0, _C.ptr(pre_out),
            pre_out.stride(0) if pre_out is not None else 0, bn | (TALL if tall else 0), c.world, c.rank,
            shard_bytes, flat_off_bytes, _C.ptr(site.flags), peer_ready, site.epoch, comm_ctas,
            _C.ptr(c.status), _C.current_stream())
    return (out, pre_out) if gelu else out


def gemm_reduce_scatter(site: FusedSite, a, b, stage, out, *, b_mn=False, residual=None, bn=None, tall=None):
    """out[M/world, N] = reduce-scatter over ranks of (a @ b^T); ``stage`` is a symmetric
    [world, M/world, N] bf16 staging buffer (one slot per source rank)."""
    c = site.comm
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    if bn is None:
        if tall is None:
            tall = pick_tall(M, N, K) and M % 256 == 0
        bn = 256 if tall else pick_bn(M, N)
    rows = M // c.world
    site.epoch += 1
    _C.call("mmj_gemm_bf16_reduce_scatter", _C.ptr(a), a.stride(0), _C.ptr(b), b.stride(0),
            int(b_mn), site.peer_ptrs(stage), N, rows * N, M, N, K, bn | (TALL if tall else 0), c.world, c.rank,
            _C.ptr(c.status), _C.current_stream())
    _C.call("mmj_reduce_slots_bf16", c._sig_ptrs, _C.ptr(stage), rows * N, _C.ptr(out),
            _C.ptr(residual), rows * N, c.world, c.rank, site.slots + c.world, site.epoch,
            _C.ptr(c.status), _C.current_stream())
    return out


def gemm_reduce_scatter_pull(site: FusedSite, a, b, partial, out, *, b_mn=False, residual=None):
    """The result of ``gemm_reduce_scatter`` from two launches: the plain GEMM (full width, no peer stores in
    its epilogue) into ``partial`` (symmetric ``[M, N]``), then every rank sums its own row block over all
    ranks' partials by peer loads (``reduce_pull_kernel``, cross-rank barrier at its entry). Faster than the
    fused kernel for products of a few thousand rows."""
    from .gemm import gemm

    c = site.comm
    M, N = partial.shape
    rows = M // c.world
    gemm(a, b, b_mn=b_mn, out=partial)
    site.epoch += 1
    _C.call("mmj_reduce_pull_bf16", c._sig_ptrs, site.peer_ptrs(partial), _C.ptr(out), _C.ptr(residual), rows * N,
            c.world, c.rank, site.slots + c.world, site.epoch, _C.ptr(c.status), _C.current_stream())
    return out
