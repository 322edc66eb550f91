"""Tensor parallelism with sequence-parallel activations.

The reference has no tensor-parallel code; the layers follow its ``Linear`` style
(legacy/src/momijo/learn/nn/layers.mojo:343-359). Activations between blocks are sharded over the
sequence (rows); a column-parallel linear all-gathers its input rows and a row-parallel linear
reduce-scatters its output rows:

  ColumnParallelLinear: y[M, out/W] = all_gather_rows(x[M/W, in]) @ W_shard[out/W, in]^T
  RowParallelLinear   : y[M/W, out] = reduce_scatter_rows(x[M, in/W] @ W_shard[out, in/W]^T)

With a ``PeerComm`` (NCCL group on one NVSwitch domain, bf16 CUDA tensors) both run as ONE fused
kernel each (``ops.fused_comm``): the all-gather is pulled over NVLink by copy CTAs of the GEMM
kernel while tiles of already-present rows are computed, and the reduce-scatter is performed by
the GEMM epilogue storing every row block into its owner's memory. Their backward passes are the
mirror images (reduce-scatter of dX, all-gather of dY). Without a communicator the same layers
run on torch.distributed collectives (gloo on CPU), which is what the CPU tests use.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from .. import ops
from ..learn.distributed import collective as C
from ..ops.functional import _weight_grad, _bias_grad

bf16 = torch.bfloat16


class SymPool:
    """Rotating symmetric buffers keyed by (shape, dtype): consecutive uses of the same shape get
    different buffers so a fast rank cannot overwrite data a slower peer still reads."""

    def __init__(self, comm, depth: int = 4):
        self.comm, self.depth, self.bufs, self.next = comm, depth, {}, {}

    def get(self, shape, dtype=bf16):
        key = (tuple(shape), dtype)
        lst = self.bufs.setdefault(key, [])
        i = self.next.get(key, 0)
        if len(lst) < self.depth:
            n = 1
            for s in shape:
                n *= s
            lst.append(self.comm.alloc(n, dtype).view(*shape))
        self.next[key] = (i + 1) % self.depth
        return lst[i % len(lst)]


class TPContext:
    """Everything a tensor-parallel layer needs: group, rank/world and (optionally) the peer
    communicator with its buffer pool and per-call-site kernel state."""

    def __init__(self, group=None, comm=None, single: bool = False):
        import torch.distributed as dist

        # collectives of the generic path must stay inside the peer communicator's own group
        self.group = group if group is not None else (comm.group if comm is not None else None)
        self.comm = comm
        if single:
            self.world, self.rank = 1, 0
        elif comm is not None:
            self.world, self.rank = comm.world, comm.rank
        elif dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        self.pool = SymPool(comm) if comm is not None else None
        self._sites = {}
        # Products with fewer gathered rows than this run as two launches (peer all-gather kernel + plain
        # GEMM, plain GEMM + pull reduce-scatter kernel) instead of one fused kernel. Measured at 4 ranks,
        # hidden 5120: at 4096 rows GEMM -> reduce-scatter takes 0.213 ms fused and 0.179 ms as two launches
        # (the epilogue's 64-byte peer stores and the slot pass cost more than they hide under a 0.11 ms
        # product), all-gather -> GEMM 0.307 against 0.293; at 8192 rows the two forms of the reduce-scatter
        # tie and the fused all-gather wins (0.454 against 0.544), at 16384 rows both fused kernels win.
        self.fuse_min_rows = int(os.environ.get("MOMIJO_TP_FUSE_MIN_ROWS", "8192"))

    @staticmethod
    def single():
        """A context of one rank (no communication), whatever process group may be initialised."""
        return TPContext(single=True)

    def site(self, key):
        from ..ops.fused_comm import FusedSite

        s = self._sites.get(key)
        if s is None:
            s = FusedSite(self.comm)
            self._sites[key] = s
        return s

    def fused(self, x) -> bool:
        return self.comm is not None and self.world > 1 and x.is_cuda and x.dtype == bf16


# ---- generic (torch.distributed) path ------------------------------------------------------------
class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return C.all_gather(x.contiguous(), 0, tp.group) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        return (C.reduce_scatter(dy.contiguous(), C.ReduceOp.SUM, 0, tp.group) if tp.world > 1 else dy), None


class _ScatterRowsSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return C.reduce_scatter(x.contiguous(), C.ReduceOp.SUM, 0, tp.group) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        return (C.all_gather(dy.contiguous(), 0, tp.group) if tp.world > 1 else dy), None


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        return C.allreduce(x.clone(), C.ReduceOp.SUM, tp.group) if tp.world > 1 else x

    @staticmethod
    def backward(ctx, dy):
        return dy, None


# ---- fused (peer memory) path -------------------------------------------------------------------
class _AGLinearFused(torch.autograd.Function):
    """all-gather(x rows) -> GEMM, one kernel; backward: GEMM -> reduce-scatter, one kernel."""

    @staticmethod
    def forward(ctx, x_shard, w, b, tp, key):
        from ..ops.fused_comm import allgather_gemm
        from ..ops.gemm import gemm

        rows, K = x_shard.shape
        M = rows * tp.world
        full = tp.pool.get((M, K))
        full[tp.rank * rows:(tp.rank + 1) * rows].copy_(x_shard)
        if M >= tp.fuse_min_rows:
            y = allgather_gemm(tp.site((key, "ag")), full, w, gather_a=True, bias=b)
        else:
            tp.comm.all_gather_rows(full)
            y = gemm(full, w, bias=b)
        ctx.save_for_backward(x_shard, w)
        ctx.tp, ctx.key, ctx.refs = tp, key, (w, b)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.fused_comm import gemm_reduce_scatter, gemm_reduce_scatter_pull

        x_shard, w = ctx.saved_tensors
        tp, key = ctx.tp, ctx.key
        rw, rb = ctx.refs
        dy = dy.contiguous()
        rows, K = x_shard.shape
        M = rows * tp.world
        # dX: partial [M, K] on every rank, summed and scattered over rows by the GEMM epilogue
        dx = torch.empty((rows, K), dtype=bf16, device=dy.device)
        if M >= tp.fuse_min_rows:
            stage = tp.pool.get((tp.world, rows, K))
            gemm_reduce_scatter(tp.site((key, "rs_b")), dy, w, stage, dx, b_mn=True)
        else:
            gemm_reduce_scatter_pull(tp.site((key, "rs_b")), dy, w, tp.pool.get((M, K)), dx, b_mn=True)
        # dW needs the gathered input again (not kept from the forward to save memory)
        full = tp.pool.get((M, K))
        full[tp.rank * rows:(tp.rank + 1) * rows].copy_(x_shard)
        tp.comm.all_gather_rows(full, tp.site((key, "ag_b")))
        dw = _weight_grad(rw, dy, full)
        db = _bias_grad(rb, dy) if rb is not None else None
        return dx, dw, db, None, None


class _LinearRSFused(torch.autograd.Function):
    """GEMM -> reduce-scatter(rows) (+ residual), one kernel + slot reduction; backward:
    all-gather(dy rows) -> GEMM, one kernel."""

    @staticmethod
    def forward(ctx, x, w, b, residual_shard, tp, key):
        from ..ops.fused_comm import gemm_reduce_scatter, gemm_reduce_scatter_pull

        M, K = x.shape
        N = w.shape[0]
        rows = M // tp.world
        out = torch.empty((rows, N), dtype=bf16, device=x.device)
        res = residual_shard
        if b is not None:  # the bias is added once, after the reduction
            res = (residual_shard + b) if residual_shard is not None else b.expand(rows, N).contiguous()
        if M >= tp.fuse_min_rows:
            stage = tp.pool.get((tp.world, rows, N))
            gemm_reduce_scatter(tp.site((key, "rs")), x.contiguous(), w, stage, out, residual=res)
        else:
            gemm_reduce_scatter_pull(tp.site((key, "rs")), x.contiguous(), w, tp.pool.get((M, N)), out, residual=res)
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.key, ctx.refs = tp, key, (w, b)
        ctx.has_res = residual_shard is not None
        return out

    @staticmethod
    def backward(ctx, dy_shard):
        from ..ops.fused_comm import allgather_gemm
        from ..ops.gemm import gemm

        x, w = ctx.saved_tensors
        tp, key = ctx.tp, ctx.key
        rw, rb = ctx.refs
        rows, N = dy_shard.shape
        M = rows * tp.world
        full = tp.pool.get((M, N))
        full[tp.rank * rows:(tp.rank + 1) * rows].copy_(dy_shard)
        if M >= tp.fuse_min_rows:
            dx = allgather_gemm(tp.site((key, "ag_b")), full, w, gather_a=True, other_mn=True)
        else:
            tp.comm.all_gather_rows(full)
            dx = gemm(full, w, b_mn=True)
        dw = _weight_grad(rw, full, x)       # `full` now holds every rank's dy rows
        db = _bias_grad(rb, dy_shard.contiguous()) if rb is not None else None
        if db is not None:
            db = C.allreduce(db, C.ReduceOp.SUM, tp.group)
        return dx, dw, db, (dy_shard if ctx.has_res else None), None, None


# ---- layers ---------------------------------------------------------------------------------------
class ColumnParallelLinear(nn.Module):
    """Weight ``[out/W, in]``. Input rows are sequence-sharded (``gather_input=True``) or already
    replicated; the output keeps all rows and the local slice of the columns."""

    def __init__(self, in_features, out_features, tp: TPContext, bias=True, gather_input=True,
                 dtype=bf16, init_std=0.02, key=None):
        super().__init__()
        if out_features % tp.world:
            raise ValueError("out_features must divide by the tensor-parallel size")
        self.tp, self.gather_input = tp, gather_input
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // tp.world, in_features, dtype=dtype))
        self.bias_t = nn.Parameter(torch.zeros(out_features // tp.world, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, 0.0, init_std)
        self.key = key or id(self)

    def forward(self, x):
        tp = self.tp
        if self.gather_input and tp.fused(x):
            return _AGLinearFused.apply(x.contiguous(), self.weight, self.bias_t, tp, self.key)
        if self.gather_input:
            x = _GatherRows.apply(x, tp)
        return ops.linear(x, self.weight, self.bias_t)


class RowParallelLinear(nn.Module):
    """Weight ``[out, in/W]``. The input holds the local slice of the columns; the output is
    summed over ranks and (``scatter_output=True``) sharded over rows."""

    def __init__(self, in_features, out_features, tp: TPContext, bias=True, scatter_output=True,
                 dtype=bf16, init_std=0.02, key=None):
        super().__init__()
        if in_features % tp.world:
            raise ValueError("in_features must divide by the tensor-parallel size")
        self.tp, self.scatter_output = tp, scatter_output
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp.world, dtype=dtype))
        self.bias_t = nn.Parameter(torch.zeros(out_features, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, 0.0, init_std)
        self.key = key or id(self)

    def forward(self, x, residual=None):
        tp = self.tp
        if self.scatter_output and tp.fused(x):
            return _LinearRSFused.apply(x, self.weight, self.bias_t, residual, tp, self.key)
        y = ops.linear(x, self.weight, None)
        y = _ScatterRowsSum.apply(y, tp) if self.scatter_output else _AllReduceSum.apply(y, tp)
        if self.bias_t is not None:
            y = y + self.bias_t
        return y if residual is None else y + residual


class VocabParallelEmbedding(nn.Module):
    """Embedding rows sharded over ranks; out-of-shard tokens contribute zeros, the partial results
    are summed over ranks and (sequence parallel) scattered over rows."""

    def __init__(self, num_embeddings, embedding_dim, tp: TPContext, dtype=bf16, init_std=0.02,
                 scatter_output=True):
        super().__init__()
        V = (num_embeddings + tp.world - 1) // tp.world
        self.tp, self.vocab_local, self.scatter_output = tp, V, scatter_output
        self.vocab_start = tp.rank * V
        self.weight = nn.Parameter(torch.empty(V, embedding_dim, dtype=dtype))
        nn.init.normal_(self.weight, 0.0, init_std)

    def forward(self, tokens):
        local = tokens - self.vocab_start
        inside = (local >= 0) & (local < self.vocab_local)
        e = ops.embedding(local.clamp(0, self.vocab_local - 1), self.weight)
        e = e * inside.unsqueeze(-1).to(e.dtype)
        e = e.reshape(-1, e.shape[-1])
        return _ScatterRowsSum.apply(e, self.tp) if self.scatter_output else _AllReduceSum.apply(e, self.tp)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy over a vocabulary sharded across ranks: per-shard (max, sum-exp, target
    logit), two tiny all-reduces, then the gradient written in place over the local logits."""

    @staticmethod
    def forward(ctx, logits, targets, vocab_start, v_local, tp):
        from .. import _C

        M = logits.shape[0]
        t1 = targets.reshape(-1).contiguous()
        dev = logits.device
        if logits.is_cuda and logits.dtype == bf16 and logits.stride(0) % 8 == 0:
            mx, sm, tg = (torch.empty(M, dtype=torch.float32, device=dev) for _ in range(3))
            _C.call("mmj_ce_vp_stats", _C.ptr(logits), logits.stride(0), v_local, vocab_start, _C.ptr(t1),
                    _C.ptr(mx), _C.ptr(sm), _C.ptr(tg), M, _C.current_stream())
        else:
            lf = logits[:, :v_local].float()
            mx = lf.max(-1).values
            sm = torch.exp(lf - mx[:, None]).sum(-1)
            loc = t1 - vocab_start
            ins = (loc >= 0) & (loc < v_local)
            tg = torch.where(ins, lf.gather(1, loc.clamp(0, v_local - 1)[:, None])[:, 0], torch.zeros_like(mx))
        gmax = mx.clone()
        if tp.world > 1:
            C.allreduce(gmax, C.ReduceOp.MAX, tp.group)
        sm = sm * torch.exp(mx - gmax)
        packed = torch.stack([sm, tg])
        if tp.world > 1:
            C.allreduce(packed, C.ReduceOp.SUM, tp.group)
        gsum, gtg = packed[0].contiguous(), packed[1]
        loss = (torch.log(gsum) + gmax - gtg).mean()
        ctx.save_for_backward(logits, t1, gmax, gsum)
        ctx.cfg = (vocab_start, v_local)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        from .. import _C

        logits, t1, gmax, gsum = ctx.saved_tensors
        vocab_start, v_local = ctx.cfg
        M = logits.shape[0]
        if logits.is_cuda and logits.dtype == bf16 and logits.stride(0) % 8 == 0:
            ds = dloss.detach().reshape(1).to(torch.float32)
            _C.call("mmj_ce_vp_grad", _C.ptr(logits), logits.stride(0), v_local, vocab_start, _C.ptr(t1),
                    _C.ptr(gmax), _C.ptr(gsum), M, 1.0 / M, _C.ptr(ds), _C.current_stream())
            return logits, None, None, None, None
        else:
            lf = logits.float()
            p = torch.exp(lf - gmax[:, None]) / gsum[:, None]
            p[:, v_local:] = 0
            loc = t1 - vocab_start
            ins = (loc >= 0) & (loc < v_local)
            rows = torch.nonzero(ins)[:, 0]
            p[rows, loc[rows]] -= 1.0
            d = (p / M).to(logits.dtype)
        return d * dloss.to(d.dtype), None, None, None, None


def vocab_parallel_cross_entropy(logits_local, targets, vocab_start, v_local, tp: TPContext):
    return _VocabParallelCE.apply(logits_local, targets, vocab_start, v_local, tp)
