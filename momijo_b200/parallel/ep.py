"""Expert parallelism: top-k softmax router, all-to-all dispatch / combine over peer memory, and
grouped expert GEMMs.

The reference has no mixture-of-experts code; the layer style follows its ``Linear`` modules
(legacy/src/momijo/learn/nn/layers.mojo:343-359). Data movement:

  dispatch : every (token, k) row is written by a peer store straight into the contiguous,
             128-row aligned segment of its expert on the destination rank (the per-expert counts
             are exchanged first, also by peer stores, so no host synchronisation is needed);
  experts  : grouped tcgen05 GEMMs over the local experts (per-tile expert table, tile count
             read from the device);
  combine  : every token pulls its k expert outputs from the ranks that computed them and forms
             the router-weighted sum.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as tF

from .. import _C, ops
from ..ops.gemm import EPI_MUL_AUX, EPI_ROW_SCALE, EPI_SILU

bf16 = torch.bfloat16


class MoEDispatcher:
    """Owns the symmetric buffers and signal slots of one MoE layer (or of several layers that
    run strictly one after another)."""

    def __init__(self, comm, n_experts: int, top_k: int, hidden: int, max_tokens: int,
                 capacity_factor: float = 2.0, n_buffers: int = 2):
        self.comm = comm
        W = comm.world
        if n_experts % W:
            raise ValueError("experts must divide evenly over ranks")
        self.E, self.k, self.H = n_experts, top_k, hidden
        self.epr = n_experts // W
        self.max_assign = max_tokens * top_k
        avg_rows = max_tokens * top_k  # rows per rank when routing is balanced
        self.cap_rows = int(math.ceil(capacity_factor * avg_rows / 128) * 128) + 128 * self.epr
        self.max_tiles = self.cap_rows // 128
        dev = comm.device
        self.counts = comm.alloc(W * n_experts, torch.int32)
        self.recv = [comm.alloc(self.cap_rows * hidden, bf16).view(self.cap_rows, hidden)
                     for _ in range(n_buffers)]
        self.yout = [comm.alloc(self.cap_rows * hidden, bf16).view(self.cap_rows, hidden)
                     for _ in range(n_buffers)]
        self._counts_ptrs = comm.peer_ptrs(self.counts)
        self._recv_ptrs = [comm.peer_ptrs(b) for b in self.recv]
        self._y_ptrs = [comm.peer_ptrs(b) for b in self.yout]
        self.local_pos = torch.empty(self.max_assign, dtype=torch.int32, device=dev)
        self.src_row = torch.empty(self.max_assign, dtype=torch.int32, device=dev)
        self.seg_off = torch.empty(W * self.epr * W, dtype=torch.int32, device=dev)
        self.tile_group = torch.zeros(self.max_tiles, dtype=torch.int32, device=dev)
        self.num_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
        self.total_rows = torch.zeros(1, dtype=torch.int32, device=dev)
        self.pad_ranges = torch.zeros(2 * self.epr, dtype=torch.int32, device=dev)
        self.slots = comm.new_slots(3 * W)
        self.ctr = comm.new_counter(1)
        self.which = 0
        self._idx = None

    def _ptrs_of(self, y):
        for b, ptrs in zip(self.yout, self._y_ptrs):
            if y is b or y.data_ptr() == b.data_ptr():
                return ptrs
        for b, ptrs in zip(self.recv, self._recv_ptrs):
            if y is b or y.data_ptr() == b.data_ptr():
                return ptrs
        return self.comm.peer_ptrs(y)

    # -- buffers of the current call --
    def expert_out_buffer(self):
        return self.yout[self.which]

    def dispatch(self, x, expert_idx, row_w: Optional[torch.Tensor] = None, reuse_routing=False):
        """x: [n_tok, H] bf16; expert_idx: [n_tok, k] int32 (global expert ids).
        Returns (recv buffer [cap_rows, H], info dict with the grouped-GEMM tile table).
        With ``reuse_routing`` the counts/offsets of the previous call are kept (backward pass)."""
        c = self.comm
        W = c.world
        n_assign = expert_idx.numel()
        if n_assign > self.max_assign:
            raise ValueError("more assignments than the dispatcher was sized for")
        idx = expert_idx.reshape(-1).contiguous()
        st = _C.ptr(c.status)
        stream = _C.current_stream()
        if not reuse_routing:
            self.which = (self.which + 1) % len(self.recv)
            ep = c.next_epoch(self.slots)
            self._ep = ep
            _C.call("mmj_moe_count", c._sig_ptrs, _C.ptr(idx), n_assign, self.E, self._counts_ptrs,
                    _C.ptr(self.local_pos), W, c.rank, self.slots, ep, st, stream)
            _C.call("mmj_moe_offsets", _C.ptr(self.counts), W, c.rank, self.E, _C.ptr(self.seg_off),
                    _C.ptr(self.tile_group), _C.ptr(self.num_tiles), _C.ptr(self.total_rows),
                    _C.ptr(self.pad_ranges), self.max_tiles, stream)
            self._idx = idx
        else:
            ep = c.next_epoch(self.slots)
            self._ep = ep
        buf = self.recv[self.which]
        _C.call("mmj_moe_zero_pad", _C.ptr(buf), self.H, _C.ptr(self.pad_ranges), self.epr,
                self.cap_rows, stream)
        _C.call("mmj_moe_dispatch", c._sig_ptrs, _C.ptr(x), _C.ptr(idx), _C.ptr(self.local_pos),
                _C.ptr(self.seg_off), self._recv_ptrs[self.which], _C.ptr(self.src_row),
                _C.ptr(row_w), self.cap_rows, n_assign, self.k, self.H, self.E, W, c.rank,
                self.slots + W, ep, _C.ptr(self.ctr), st, stream)
        info = {"tile_group": self.tile_group, "num_tiles": self.num_tiles,
                "total_rows": self.total_rows}
        return buf, info

    def combine(self, y, gate_w, residual=None, n_tokens=None):
        """out[token] = residual[token] + sum_k gate_w[token, k] * y[row(token, k)] where ``y`` is
        a symmetric buffer in recv layout (``expert_out_buffer()``)."""
        c = self.comm
        idx = self._idx
        n_tokens = idx.numel() // self.k if n_tokens is None else n_tokens
        out = torch.empty((n_tokens, self.H), dtype=bf16, device=c.device)
        ptrs = self._ptrs_of(y)
        gw = None if gate_w is None else gate_w.reshape(-1).contiguous().float()
        _C.call("mmj_moe_combine", c._sig_ptrs, ptrs, _C.ptr(idx), _C.ptr(self.src_row), _C.ptr(gw),
                _C.ptr(out), _C.ptr(residual), n_tokens, self.k, self.H, self.E, c.world, c.rank,
                self.slots + 2 * c.world, self._ep, _C.ptr(c.status), _C.current_stream())
        return out

    def gate_grad(self, y, dout):
        """d gate_w[token, k] = <dout[token], y[row(token, k)]>."""
        c = self.comm
        idx = self._idx
        n_assign = idx.numel()
        dg = torch.empty(n_assign, dtype=torch.float32, device=c.device)
        ptrs = self._ptrs_of(y)
        _C.call("mmj_moe_gate_grad", ptrs, _C.ptr(dout), _C.ptr(idx), _C.ptr(self.src_row),
                _C.ptr(dg), n_assign, self.k, self.H, self.E, c.world, _C.current_stream())
        return dg.view(-1, self.k)


def grouped_gemm(a, w, info, *, b_mn=False, out=None, epi_silu=False, mul_aux=None,
                 row_scale=None, bn=128):
    """Rows of ``a`` [cap_rows, K] are grouped by expert in 128-row tiles (``info``); ``w`` is
    [n_local_experts, N, K] (or [n_local_experts, K, N] with ``b_mn``)."""
    G = w.shape[0]
    if b_mn:
        K, N = w.shape[1], w.shape[2]
        group_rows = K
    else:
        N, K = w.shape[1], w.shape[2]
        group_rows = N
    cap = a.shape[0]
    if out is None:
        out = torch.empty((cap, N), dtype=bf16, device=a.device)
    epi = (EPI_SILU if epi_silu else 0) | (EPI_MUL_AUX if mul_aux is not None else 0) | (
        EPI_ROW_SCALE if row_scale is not None else 0)
    w2 = w.reshape(G * w.shape[1], w.shape[2])
    _C.call("mmj_gemm_bf16_grouped", _C.ptr(a), a.stride(0), _C.ptr(w2), w2.stride(0), int(b_mn), G,
            group_rows, _C.ptr(out), out.stride(0), cap, N, K, epi, _C.ptr(mul_aux),
            mul_aux.stride(0) if mul_aux is not None else 0, _C.ptr(row_scale),
            _C.ptr(info["tile_group"]), _C.ptr(info["num_tiles"]), bn,
            _C.ptr(_C.status_tensor(a.device)), _C.current_stream())
    return out


class TopKRouter(nn.Module):
    """Softmax router with top-k selection, renormalised weights and the load-balance auxiliary
    loss  aux = E * sum_e f_e * P_e  (f_e: fraction of assignments, P_e: mean router probability)."""

    def __init__(self, hidden: int, n_experts: int, top_k: int, aux_coef: float = 0.01,
                 dtype=bf16):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_experts, hidden, dtype=dtype))
        nn.init.normal_(self.weight, 0.0, 0.02)
        self.E, self.k, self.aux_coef = n_experts, top_k, aux_coef

    def forward(self, x):
        logits = ops.linear(x, self.weight).float()
        probs = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, self.k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        with torch.no_grad():
            f = torch.zeros(self.E, device=x.device, dtype=torch.float32)
            f.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), device=x.device))
            f = f / idx.numel()
        aux = self.aux_coef * self.E * (f * probs.mean(0)).sum()
        return w, idx.int(), aux
