"""Expert parallelism: top-k softmax router, all-to-all dispatch / combine over peer memory, and
grouped expert GEMMs.

The reference has no mixture-of-experts code; the layer style follows its ``Linear`` modules
(legacy/src/momijo/learn/nn/layers.mojo:343-359). Data movement:

  dispatch : every (token, k) row is written by a peer store straight into the contiguous,
             128-row aligned segment of its expert on the destination rank (the per-expert counts
             are exchanged first, also by peer stores, so no host synchronisation is needed);
  experts  : grouped tcgen05 GEMMs over the local experts (per-tile expert table, tile count
             read from the device; weight gradients use the grouped-K mode);
  combine  : every token pulls its k expert outputs from the ranks that computed them and forms
             the router-weighted sum.

The backward pass reuses the same kernels with the roles swapped: the gradient of combine is a
dispatch of ``dout`` scaled by the router weights, the gradient of dispatch is an unweighted
combine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import _C, ops
from ..ops.gemm import EPI_MUL_AUX, EPI_ROW_SCALE, EPI_SILU

bf16 = torch.bfloat16


@dataclass
class Routing:
    """Device-side routing state of one dispatch (kept for the combine and for the backward)."""
    idx: torch.Tensor            # [n_assign] global expert of each (token, k)
    local_pos: torch.Tensor      # [n_assign] position inside its (source rank, expert) run
    src_row: torch.Tensor        # [n_assign] row inside the destination rank's buffer
    seg_off: torch.Tensor        # [world, experts_per_rank, world]
    tile_group: torch.Tensor     # [max_tiles] local expert of each 128-row tile
    num_tiles: torch.Tensor      # [1]
    total_rows: torch.Tensor     # [1]
    pad_ranges: torch.Tensor     # [experts_per_rank, 2] rows holding no token
    expert_ranges: torch.Tensor  # [experts_per_rank, 2] rows of each local expert (padded)
    n_tokens: int = 0

    def info(self):
        return {"tile_group": self.tile_group, "num_tiles": self.num_tiles}


class MoEDispatcher:
    """Symmetric buffers and signal slots shared by the MoE layers of a model (layers run one
    after another; buffers rotate so a fast rank never overwrites rows a peer still reads)."""

    def __init__(self, comm, n_experts: int, top_k: int, hidden: int, max_tokens: int,
                 capacity_factor: float = 2.0, n_buffers: int = 4):
        self.comm = comm
        W = comm.world
        if n_experts % W:
            raise ValueError("experts must divide evenly over ranks")
        self.E, self.k, self.H = n_experts, top_k, hidden
        self.epr = n_experts // W
        self.max_assign = max_tokens * top_k
        self.cap_rows = int(math.ceil(capacity_factor * self.max_assign / 128) * 128) + 128 * self.epr
        self.max_tiles = self.cap_rows // 128
        self.counts = comm.alloc(W * n_experts, torch.int32)
        self._counts_ptrs = comm.peer_ptrs(self.counts)
        self.bufs = [comm.alloc(self.cap_rows * hidden, bf16).view(self.cap_rows, hidden)
                     for _ in range(n_buffers)]
        self._ptrs = [comm.peer_ptrs(b) for b in self.bufs]
        self._next = 0
        self.slots = comm.new_slots(3 * W)   # count barrier | dispatch barrier | combine barrier
        comm._epochs[self.slots + W] = 0
        comm._epochs[self.slots + 2 * W] = 0
        self.ctr = comm.new_counter(1)

    def next_buffer(self):
        """A symmetric [cap_rows, H] buffer (recv layout) to dispatch into or to fill with expert
        outputs; returns (tensor, peer pointer table)."""
        i = self._next
        self._next = (self._next + 1) % len(self.bufs)
        return self.bufs[i], self._ptrs[i]

    def ptrs_of(self, t):
        for b, p in zip(self.bufs, self._ptrs):
            if t.data_ptr() == b.data_ptr():
                return p
        return self.comm.peer_ptrs(t)

    def route(self, expert_idx) -> Routing:
        """Exchange per-expert counts with all ranks and derive every rank's segment offsets."""
        c, W, dev = self.comm, self.comm.world, self.comm.device
        idx = expert_idx.reshape(-1).to(torch.int32).contiguous()
        n = idx.numel()
        if n > self.max_assign:
            raise ValueError("more assignments than the dispatcher was sized for")
        i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)
        r = Routing(idx, i32(n), i32(n), i32(W * self.epr * W), torch.zeros(self.max_tiles, dtype=torch.int32, device=dev),
                    i32(1), i32(1), i32(2 * self.epr), i32(2 * self.epr), n // self.k)
        ep = c.next_epoch(self.slots)
        st, stream = _C.ptr(c.status), _C.current_stream()
        _C.call("mmj_moe_count", c._sig_ptrs, _C.ptr(idx), n, self.E, self._counts_ptrs, _C.ptr(r.local_pos),
                W, c.rank, self.slots, ep, st, stream)
        _C.call("mmj_moe_offsets", _C.ptr(self.counts), W, c.rank, self.E, _C.ptr(r.seg_off),
                _C.ptr(r.tile_group), _C.ptr(r.num_tiles), _C.ptr(r.total_rows), _C.ptr(r.pad_ranges),
                _C.ptr(r.expert_ranges), self.max_tiles, stream)
        return r

    def dispatch(self, x, r: Routing, row_w: Optional[torch.Tensor] = None):
        """Send every (token, k) row of ``x`` [n_tok, H] to its expert's segment; rows may be scaled
        by ``row_w`` [n_assign]. Returns the local recv-layout buffer [cap_rows, H]."""
        c, W = self.comm, self.comm.world
        buf, ptrs = self.next_buffer()
        stream = _C.current_stream()
        ep = c.next_epoch(self.slots + W)
        _C.call("mmj_moe_zero_pad", _C.ptr(buf), self.H, _C.ptr(r.pad_ranges), self.epr, self.cap_rows, stream)
        rw = None if row_w is None else row_w.reshape(-1).float().contiguous()
        _C.call("mmj_moe_dispatch", c._sig_ptrs, _C.ptr(x.contiguous()), _C.ptr(r.idx), _C.ptr(r.local_pos),
                _C.ptr(r.seg_off), ptrs, _C.ptr(r.src_row), _C.ptr(rw), self.cap_rows, r.idx.numel(), self.k,
                self.H, self.E, W, c.rank, self.slots + W, ep, _C.ptr(self.ctr), _C.ptr(c.status), stream)
        return buf

    def combine(self, y, r: Routing, gate_w=None, residual=None):
        """out[token] = residual[token] + sum_k gate_w[token, k] * y[row(token, k)] where ``y`` is a
        symmetric recv-layout buffer on every rank (``gate_w=None`` means weights of one)."""
        c = self.comm
        out = torch.empty((r.n_tokens, self.H), dtype=bf16, device=c.device)
        gw = None if gate_w is None else gate_w.reshape(-1).float().contiguous()
        ep = c.next_epoch(self.slots + 2 * c.world)
        _C.call("mmj_moe_combine", c._sig_ptrs, self.ptrs_of(y), _C.ptr(r.idx), _C.ptr(r.src_row), _C.ptr(gw),
                _C.ptr(out), _C.ptr(residual), r.n_tokens, self.k, self.H, self.E, self.cap_rows, c.world, c.rank,
                self.slots + 2 * c.world, ep, _C.ptr(c.status), _C.current_stream())
        return out

    def gate_grad(self, y, dout, r: Routing):
        """d gate_w[token, k] = <dout[token], y[row(token, k)]> (``y`` symmetric, final on all ranks)."""
        c = self.comm
        n = r.idx.numel()
        dg = torch.empty(n, dtype=torch.float32, device=c.device)
        _C.call("mmj_moe_gate_grad", self.ptrs_of(y), _C.ptr(dout.contiguous()), _C.ptr(r.idx), _C.ptr(r.src_row),
                _C.ptr(dg), n, self.k, self.H, self.E, c.world, _C.current_stream())
        return dg.view(-1, self.k)


def grouped_gemm(a, w, r: Routing, *, b_mn=False, out=None, mul_aux=None, bn=128):
    """Rows of ``a`` [cap_rows, K] are grouped by expert in 128-row tiles; ``w`` is
    [n_local_experts, N, K] (or [n_local_experts, K, N] with ``b_mn``)."""
    G = w.shape[0]
    K, N = (w.shape[1], w.shape[2]) if b_mn else (w.shape[2], w.shape[1])
    cap = a.shape[0]
    if out is None:
        out = torch.empty((cap, N), dtype=bf16, device=a.device)
    epi = EPI_MUL_AUX if mul_aux is not None else 0
    w2 = w.reshape(G * w.shape[1], w.shape[2])
    _C.call("mmj_gemm_bf16_grouped", _C.ptr(a), a.stride(0), _C.ptr(w2), w2.stride(0), int(b_mn), G,
            w.shape[1], _C.ptr(out), out.stride(0), cap, N, K, epi, _C.ptr(mul_aux),
            mul_aux.stride(0) if mul_aux is not None else 0, None, _C.ptr(r.tile_group),
            _C.ptr(r.num_tiles), bn, _C.ptr(_C.status_tensor(a.device)), _C.current_stream())
    return out


def grouped_gemm_wgrad(dy, x, r: Routing, n_groups: int, out=None, accumulate=False, bn=128):
    """dW[g] = dy_g^T x_g over the rows of each local expert; dy [cap, M], x [cap, N] -> [G, M, N]."""
    cap, M = dy.shape
    N = x.shape[1]
    if out is None:
        out = torch.empty((n_groups, M, N), dtype=bf16, device=dy.device)
        accumulate = False
    _C.call("mmj_gemm_bf16_grouped_k", _C.ptr(dy), dy.stride(0), _C.ptr(x), x.stride(0), _C.ptr(out), N, cap,
            M, N, n_groups, _C.ptr(r.expert_ranges), int(out.dtype == torch.float32), int(accumulate), bn,
            _C.ptr(_C.status_tensor(dy.device)), _C.current_stream())
    return out


class _ExpertsEP(torch.autograd.Function):
    """dispatch -> grouped gate/up GEMM -> SwiGLU -> grouped down GEMM -> weighted combine."""

    @staticmethod
    def forward(ctx, x, gate_w, idx, w_gu, w_down, disp):
        F = w_down.shape[2]
        r = disp.route(idx)
        recv = disp.dispatch(x, r)
        gu = grouped_gemm(recv, w_gu, r)                         # [cap, 2F]
        act = torch.empty((gu.shape[0], F), dtype=bf16, device=x.device)
        _C.call("mmj_swiglu_fwd", _C.ptr(gu), _C.ptr(act), gu.shape[0], F, _C.current_stream())
        ybuf, _ = disp.next_buffer()
        grouped_gemm(act, w_down, r, out=ybuf)                   # [cap, H] symmetric
        out = disp.combine(ybuf, r, gate_w)
        # The symmetric buffers are reused by later layers, and private copies of the dispatched rows
        # and of the expert outputs would cost two [cap_rows, H] tensors per layer; the backward pass
        # dispatches x again and recomputes the expert outputs from `act` instead.
        ctx.save_for_backward(x, gate_w, gu, act, w_gu, w_down)
        ctx.r, ctx.disp, ctx.refs = r, disp, (w_gu, w_down)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.functional import _wgrad_target

        x, gate_w, gu, act, w_gu, w_down = ctx.saved_tensors
        r, disp = ctx.r, ctx.disp
        rw_gu, rw_down = ctx.refs
        F = w_down.shape[2]
        G = w_gu.shape[0]
        dout = dout.contiguous()
        # gradient of the router weights needs the (unweighted) expert outputs of every rank
        ysym, _ = disp.next_buffer()
        grouped_gemm(act, w_down, r, out=ysym)
        disp.comm.barrier()
        dgate = disp.gate_grad(ysym, dout, r)
        # gradient w.r.t. expert outputs: dispatch dout scaled by the router weights
        dy = disp.dispatch(dout, r, row_w=gate_w)
        dact = grouped_gemm(dy, w_down, r, b_mn=True)            # dy [cap,H] x w_down[e] [H,F]
        buf, acc = _wgrad_target(rw_down)
        dw_down = grouped_gemm_wgrad(dy, act, r, G, out=buf, accumulate=acc)
        dgu = torch.empty_like(gu)
        _C.call("mmj_swiglu_bwd", _C.ptr(gu), _C.ptr(dact), _C.ptr(dgu), gu.shape[0], F, _C.current_stream())
        recv = disp.dispatch(x, r)                               # the forward's expert inputs again
        buf2, acc2 = _wgrad_target(rw_gu)
        dw_gu = grouped_gemm_wgrad(dgu, recv, r, G, out=buf2, accumulate=acc2)
        dxbuf, _ = disp.next_buffer()
        grouped_gemm(dgu, w_gu, r, b_mn=True, out=dxbuf)         # dgu [cap,2F] x w_gu[e] [2F,H]
        dx = disp.combine(dxbuf, r, None)
        return (dx, dgate.to(gate_w.dtype), None, None if buf2 is not None else dw_gu,
                None if buf is not None else dw_down, None)


class _RouterTopK(torch.autograd.Function):
    """softmax -> top-k -> renormalise -> per-expert counts / probability sums -> auxiliary loss, as one
    device pass (``csrc/moe_router.cu``); the backward pass is one kernel as well."""

    @staticmethod
    def forward(ctx, logits, k, coef):
        logits = logits.contiguous()
        n, E = logits.shape
        dev = logits.device
        w = torch.empty((n, k), dtype=torch.float32, device=dev)
        idx = torch.empty((n, k), dtype=torch.int32, device=dev)
        cnt = torch.empty(E, dtype=torch.int32, device=dev)
        psum = torch.empty(E, dtype=torch.float32, device=dev)
        aux = torch.empty(1, dtype=torch.float32, device=dev)
        parts = _C.lib().mmj_moe_router_parts()
        pc = torch.empty(parts * E, dtype=torch.int32, device=dev)
        pp = torch.empty(parts * E, dtype=torch.float32, device=dev)
        _C.call("mmj_moe_router_fwd", _C.ptr(logits), logits.stride(0), n, E, k, float(coef), _C.ptr(w), _C.ptr(idx),
                _C.ptr(cnt), _C.ptr(psum), _C.ptr(aux), _C.ptr(pc), _C.ptr(pp), _C.current_stream())
        ctx.save_for_backward(logits, w, idx, cnt)
        ctx.k, ctx.coef = k, float(coef)
        ctx.mark_non_differentiable(idx)
        return w, idx, aux[0]

    @staticmethod
    def backward(ctx, dw, _didx, daux):
        logits, w, idx, cnt = ctx.saved_tensors
        n, E = logits.shape
        dl = torch.empty_like(logits)
        dw = None if dw is None else dw.contiguous().float()
        da = None if daux is None else daux.reshape(1).float().contiguous()
        _C.call("mmj_moe_router_bwd", _C.ptr(logits), logits.stride(0), n, E, ctx.k, _C.ptr(w), _C.ptr(idx),
                _C.ptr(dw), _C.ptr(da), _C.ptr(cnt), ctx.coef, _C.ptr(dl), dl.stride(0), _C.current_stream())
        return dl, None, None


class _AllToAllRows(torch.autograd.Function):
    """``all_to_all_single`` of row blocks with given split sizes; the gradient travels the opposite way."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        import torch.distributed as dist

        ctx.splits, ctx.group = (in_splits, out_splits), group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        import torch.distributed as dist

        in_splits, out_splits = ctx.splits
        dx = dy.new_empty((sum(in_splits),) + tuple(dy.shape[1:]))
        dist.all_to_all_single(dx, dy.contiguous(), output_split_sizes=in_splits, input_split_sizes=out_splits,
                               group=ctx.group)
        return dx, None, None, None


class TopKRouter(nn.Module):
    """Softmax router with top-k selection, renormalised weights and the load-balance auxiliary
    loss ``aux = coef * E * sum_e f_e * P_e`` (f_e: fraction of assignments, P_e: mean router
    probability)."""

    def __init__(self, hidden: int, n_experts: int, top_k: int, aux_coef: float = 0.01, dtype=bf16):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_experts, hidden, dtype=dtype))
        nn.init.normal_(self.weight, 0.0, 0.02)
        self.E, self.k, self.aux_coef = n_experts, top_k, aux_coef

    def forward(self, x):
        if x.is_cuda and x.dtype == bf16 and self.E <= 256 and self.k <= 32:
            return _RouterTopK.apply(ops.linear(x, self.weight), self.k, self.aux_coef)
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


class MoELayer(nn.Module):
    """Routed experts (SwiGLU, expert parallel) plus optional shared experts (dense SwiGLU)."""

    def __init__(self, hidden: int, ffn: int, n_experts: int, top_k: int, n_shared: int = 0,
                 aux_coef: float = 0.01, dispatcher: Optional[MoEDispatcher] = None, world: int = 1,
                 rank: int = 0, dtype=bf16, init_std: float = 0.02, group=None):
        """``dispatcher``: the peer-memory dispatch / combine kernels (CUDA, one NVSwitch domain).
        ``group``: a torch.distributed process group instead: tokens travel by ``all_to_all_single`` (any
        backend: gloo on CPU, NCCL across nodes), the experts run as plain matrix products. Neither: one
        rank holds every expert."""
        super().__init__()
        self.disp = dispatcher
        self.group = group
        if dispatcher is not None:
            self.world, self.rank = dispatcher.comm.world, dispatcher.comm.rank
        elif group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = world, rank
        if n_experts % self.world:
            raise ValueError("experts must divide evenly over ranks")
        self.E, self.k, self.H, self.F = n_experts, top_k, hidden, ffn
        self.epr = n_experts // self.world
        self.router = TopKRouter(hidden, n_experts, top_k, aux_coef, dtype)
        self.w_gu = nn.Parameter(torch.empty(self.epr, 2 * ffn, hidden, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(self.epr, hidden, ffn, dtype=dtype))
        nn.init.normal_(self.w_gu, 0.0, init_std)
        nn.init.normal_(self.w_down, 0.0, init_std)
        self.shared = None
        if n_shared > 0:
            from ..learn.nn.layers import SwiGLU

            self.shared = SwiGLU(hidden, n_shared * ffn, dtype=dtype, init_std=init_std)

    def forward(self, x):
        """x: [n_tok, H] -> ([n_tok, H], aux loss)."""
        w, idx, aux = self.router(x)
        if self.disp is not None and x.is_cuda and x.dtype == bf16:
            y = _ExpertsEP.apply(x, w, idx, self.w_gu, self.w_down, self.disp)
        elif self.group is not None and self.world > 1:
            y = self._experts_all_to_all(x, w, idx)
        else:
            y = self._experts_reference(x, w, idx)
        if self.shared is not None:
            y = y + self.shared(x)
        return y, aux

    def _experts_all_to_all(self, x, w, idx):
        """Expert parallelism over torch.distributed: assignments sorted by expert (experts of one rank are
        adjacent, so this also groups them by destination), per-expert counts exchanged first, rows sent
        with ``all_to_all_single``, every local expert applied to its rows, results sent back the same way
        and summed into their tokens with the gate weights. No capacity limit: nothing is dropped."""
        import torch.distributed as dist

        W, epr, k = self.world, self.epr, self.k
        n = x.shape[0]
        flat_e = idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        tok = torch.div(order, k, rounding_mode="floor")
        counts = torch.bincount(flat_e, minlength=self.E)                 # assignments per expert, [E]
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)      # [W, epr]: from each source rank
        in_splits = counts.view(W, epr).sum(1).tolist()
        out_splits = recv_counts.view(W, epr).sum(1).tolist()
        rows = _AllToAllRows.apply(x[tok], in_splits, out_splits, self.group)
        # received rows come as (source rank, local expert) runs: bring each expert's rows together
        rc = recv_counts.view(W, epr)
        local_e = torch.repeat_interleave(torch.arange(epr, device=x.device).repeat(W), rc.reshape(-1))
        by_e = torch.argsort(local_e, stable=True)
        per_e = rc.sum(0).tolist()
        outs, start = [], 0
        sorted_rows = rows[by_e]
        for j in range(epr):
            r = sorted_rows[start:start + per_e[j]]
            start += per_e[j]
            h = r @ self.w_gu[j].t().to(r.dtype)
            g, u = h.chunk(2, -1)
            outs.append((torch.nn.functional.silu(g) * u) @ self.w_down[j].t().to(r.dtype))
        y_sorted = torch.cat(outs) if outs else rows.new_zeros((0, self.H))
        y_recv = torch.empty_like(y_sorted)
        y_recv[by_e] = y_sorted                                            # back to arrival order
        back = _AllToAllRows.apply(y_recv, out_splits, in_splits, self.group)
        gate = w.reshape(-1)[order].to(torch.float32)
        out = torch.zeros((n, self.H), dtype=torch.float32, device=x.device)
        out = out.index_add(0, tok, back.float() * gate[:, None])
        return out.to(x.dtype)

    def _experts_reference(self, x, w, idx):
        """Dense evaluation with plain torch (single rank holds every expert); used on CPU."""
        if self.world != 1:
            raise RuntimeError("the reference path needs all experts on one rank")
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in range(self.E):
            sel = (idx == e)
            tok, kk = torch.nonzero(sel, as_tuple=True)
            if tok.numel() == 0:
                continue
            h = x[tok] @ self.w_gu[e].t().to(x.dtype)
            g, u = h.chunk(2, -1)
            y = (torch.nn.functional.silu(g) * u) @ self.w_down[e].t().to(x.dtype)
            out.index_add_(0, tok, (y.float() * w[tok, kk].float()[:, None]))
        return out.to(x.dtype)
