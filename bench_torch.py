"""Stock-PyTorch arms of the benchmark configs (used by ``bench.py --impl torch``).

Nothing here touches this repository's kernels or engine: matrix products are ``F.linear`` (cuBLAS),
attention is ``F.scaled_dot_product_attention``, collectives are torch.distributed (NCCL on GPUs, gloo on
CPU for the tiny test shapes), the optimizer is ``torch.optim.AdamW(fused=True)`` on fp32 parameters
under bf16 autocast. Two models:

* ``TorchLlamaTP``: Megatron-style tensor parallelism with sequence parallelism (all-gather before the
  column-parallel products, reduce-scatter after the row-parallel ones, vocabulary-parallel embedding and
  cross-entropy).
* ``TorchMoEEP``: expert parallelism by ``all_to_all_single`` (tokens sorted by destination expert, one
  ``F.linear`` per local expert), data-parallel dense parameters by an explicit gradient all-reduce.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _world(group=None):
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group=None):
    return dist.get_rank(group) if dist.is_initialized() else 0


class _AllGatherRows(torch.autograd.Function):
    """[M/W, C] -> [M, C]; backward: reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = _world(group)
        if W == 1:
            return x
        out = x.new_empty((x.shape[0] * W,) + x.shape[1:])
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = _world(ctx.group)
        if W == 1:
            return g, None
        out = g.new_empty((g.shape[0] // W,) + g.shape[1:])
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    """[M, C] partial sums -> [M/W, C]; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        W = _world(group)
        if W == 1:
            return x
        out = x.new_empty((x.shape[0] // W,) + x.shape[1:])
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        W = _world(ctx.group)
        if W == 1:
            return g, None
        out = g.new_empty((g.shape[0] * W,) + g.shape[1:])
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, op):
        if _world(group) > 1:
            x = x.clone()
            dist.all_reduce(x, op=op, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None, None


def _rope(x, theta):
    """x: [B, T, H, D], rotate-half convention."""
    B, T, H, D = x.shape
    half = D // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, device=x.device, dtype=torch.float32) / half))
    ang = torch.arange(T, device=x.device, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos()[None, :, None, :].to(x.dtype), ang.sin()[None, :, None, :].to(x.dtype)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)


class TorchLlamaTP(nn.Module):
    """``layers`` / ``first`` / ``last`` select one pipeline stage: the first stage owns the embedding,
    the last one the final norm, the head and the loss; a middle or first stage returns its
    sequence-sharded activation ``[M/W, C]``."""

    def __init__(self, cfg, group=None, layers=None, first=True, last=True):
        super().__init__()
        self.cfg, self.group = cfg, group
        self.first, self.last = first, last
        n_local_layers = cfg.n_layer if layers is None else len(layers)
        W, R = _world(group), _rank(group)
        self.W, self.R = W, R
        c, D = cfg.d_model, cfg.head_dim
        self.hq, self.hkv = cfg.n_head // W, cfg.n_kv_head // W
        v_pad = (cfg.vocab_size + W * 8 - 1) // (W * 8) * (W * 8)
        self.v_local = v_pad // W
        std = cfg.init_std
        P = lambda *s: nn.Parameter(torch.randn(*s) * std)
        if first:
            self.embed = P(self.v_local, c)
        self.layers = nn.ModuleList()
        for _ in range(n_local_layers):
            m = nn.Module()
            m.attn_norm = nn.Parameter(torch.ones(c))
            m.mlp_norm = nn.Parameter(torch.ones(c))
            m.wqkv = P((self.hq + 2 * self.hkv) * D, c)
            m.wo = P(c, self.hq * D)
            m.w_gu = P(2 * cfg.d_ff // W, c)
            m.w_down = P(c, cfg.d_ff // W)
            self.layers.append(m)
        self.replicated = [p for m in self.layers for p in (m.attn_norm, m.mlp_norm)]
        if last:
            self.final_norm = nn.Parameter(torch.ones(c))
            self.head = P(self.v_local, c)
            self.replicated.append(self.final_norm)
        self.batch_shape = None   # (B, T) of a micro-batch, needed by stages that receive activations

    def forward(self, tokens, targets=None):
        cfg, g, W = self.cfg, self.group, self.W
        lo = self.R * self.v_local
        if self.first:
            B, T = tokens.shape
            # vocabulary-parallel embedding: local rows, zeros elsewhere, summed and scattered over rows
            local = tokens.reshape(-1) - lo
            ok = (local >= 0) & (local < self.v_local)
            e = F.embedding(local.clamp(0, self.v_local - 1), self.embed) * ok[:, None].to(self.embed.dtype)
            x = _ReduceScatterRows.apply(e, g)                               # [M/W, C]
        else:
            B, T = self.batch_shape
            x = tokens
        M = B * T
        D = cfg.head_dim
        for m in self.layers:
            h = _AllGatherRows.apply(F.rms_norm(x, (cfg.d_model,), m.attn_norm, cfg.rms_eps), g)
            qkv = F.linear(h, m.wqkv).view(B, T, self.hq + 2 * self.hkv, D)
            q, k, v = qkv.split([self.hq, self.hkv, self.hkv], dim=2)
            q, k = _rope(q, cfg.rope_theta), _rope(k, cfg.rope_theta)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=self.hq != self.hkv)
            a = a.transpose(1, 2).reshape(M, self.hq * D)
            x = x + _ReduceScatterRows.apply(F.linear(a, m.wo), g)
            h = _AllGatherRows.apply(F.rms_norm(x, (cfg.d_model,), m.mlp_norm, cfg.rms_eps), g)
            gu = F.linear(h, m.w_gu)
            gate, up = gu.chunk(2, dim=-1)
            x = x + _ReduceScatterRows.apply(F.linear(F.silu(gate) * up, m.w_down), g)
        if not self.last:
            return x
        h = _AllGatherRows.apply(F.rms_norm(x, (cfg.d_model,), self.final_norm, cfg.rms_eps), g)
        logits = F.linear(h, self.head).float()                              # [M, V/W]
        valid = min(self.v_local, max(0, cfg.vocab_size - lo))
        if valid < self.v_local:
            logits = logits.masked_fill(torch.arange(self.v_local, device=logits.device)[None] >= valid, -1e30)
        mx = _AllReduce.apply(logits.detach().max(-1).values, g, dist.ReduceOp.MAX)
        ex = (logits - mx[:, None]).exp()
        denom = _AllReduce.apply(ex.sum(-1), g, dist.ReduceOp.SUM)
        tl = targets.reshape(-1) - lo
        tok_ok = (tl >= 0) & (tl < self.v_local)
        picked = logits.gather(1, tl.clamp(0, self.v_local - 1)[:, None])[:, 0] * tok_ok.float()
        picked = _AllReduce.apply(picked, g, dist.ReduceOp.SUM)
        return (denom.log() + mx - picked).mean()

    def sync_replicated_grads(self):
        if self.W > 1:
            for p in self.replicated:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.group)


class TorchMoEEP(nn.Module):
    def __init__(self, cfg, group=None):
        super().__init__()
        self.cfg, self.group = cfg, group
        W, R = _world(group), _rank(group)
        self.W, self.R = W, R
        self.epr = cfg.n_experts // W
        c, hd = cfg.d_model, cfg.n_head * cfg.head_dim
        std = cfg.init_std
        P = lambda *s: nn.Parameter(torch.randn(*s) * std)
        v = (cfg.vocab_size + 7) // 8 * 8
        self.wte = P(v, c)
        self.layers = nn.ModuleList()
        self.expert_params = []
        for _ in range(cfg.n_layer):
            m = nn.Module()
            m.attn_norm, m.mlp_norm = nn.Parameter(torch.ones(c)), nn.Parameter(torch.ones(c))
            m.wqkv, m.wo = P(3 * hd, c), P(c, hd)
            m.router = P(cfg.n_experts, c)
            m.w_gu, m.w_down = P(self.epr, 2 * cfg.d_ff_expert, c), P(self.epr, c, cfg.d_ff_expert)
            if cfg.n_shared:
                m.s_gu, m.s_down = P(2 * cfg.d_ff_expert * cfg.n_shared, c), P(c, cfg.d_ff_expert * cfg.n_shared)
            self.expert_params += [m.w_gu, m.w_down]
            self.layers.append(m)
        self.final_norm = nn.Parameter(torch.ones(c))
        self.head = P(v, c)
        ids = {id(p) for p in self.expert_params}
        self.dense_params = [p for p in self.parameters() if id(p) not in ids]

    def _experts(self, m, x, w, idx):
        """x [n, C]; w, idx [n, k]. Returns the weighted sum of the selected experts' outputs."""
        cfg, W, epr = self.cfg, self.W, self.epr
        n, k = idx.shape
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        src_tok = order // k
        send = x[src_tok]                                                     # sorted by global expert
        counts = torch.bincount(flat_e, minlength=cfg.n_experts)
        if W > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)     # [W * epr] per source rank
            in_split = counts.view(W, epr).sum(1).tolist()
            out_split = recv_counts.view(W, epr).sum(1).tolist()
            recv = _AllToAll.apply(send, out_split, in_split, self.group)
            per_src = recv_counts.view(W, epr)
        else:
            recv, per_src = send, counts.view(1, epr)
        # rows arrive grouped by source rank, then by local expert: regroup by expert
        le = torch.repeat_interleave(torch.arange(epr, device=x.device).repeat(per_src.shape[0]), per_src.reshape(-1))
        eorder = torch.argsort(le, stable=True)
        xin = recv[eorder]
        sizes = per_src.sum(0).tolist()
        outs = []
        off = 0
        for e in range(epr):
            xe = xin[off:off + sizes[e]]
            off += sizes[e]
            gate, up = F.linear(xe, m.w_gu[e]).chunk(2, dim=-1)
            outs.append(F.linear(F.silu(gate) * up, m.w_down[e]))
        y = torch.cat(outs) if outs else xin
        back = torch.empty_like(y)
        back[eorder] = y
        if W > 1:
            back = _AllToAll.apply(back, in_split, out_split, self.group)
        contrib = back * w.reshape(-1)[order][:, None].to(back.dtype)
        out = torch.zeros(x.shape, dtype=contrib.dtype, device=x.device)
        out.index_add_(0, src_tok, contrib)
        return out.to(x.dtype)

    def forward(self, tokens, targets):
        cfg = self.cfg
        B, T = tokens.shape
        H, D = cfg.n_head, cfg.head_dim
        x = F.embedding(tokens.reshape(-1), self.wte)
        aux_total = 0.0
        for m in self.layers:
            h = F.rms_norm(x, (cfg.d_model,), m.attn_norm, cfg.rms_eps)
            q, k, v = F.linear(h, m.wqkv).view(B, T, 3, H, D).unbind(2)
            q, k = _rope(q, cfg.rope_theta), _rope(k, cfg.rope_theta)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
            x = x + F.linear(a.transpose(1, 2).reshape(B * T, H * D), m.wo)
            h = F.rms_norm(x, (cfg.d_model,), m.mlp_norm, cfg.rms_eps)
            probs = torch.softmax(F.linear(h, m.router).float(), -1)
            w, idx = torch.topk(probs, cfg.top_k, dim=-1)
            w = w / w.sum(-1, keepdim=True)
            f = torch.bincount(idx.reshape(-1), minlength=cfg.n_experts).float() / idx.numel()
            aux_total = aux_total + cfg.aux_coef * cfg.n_experts * (f * probs.mean(0)).sum()
            y = self._experts(m, h, w, idx)
            if cfg.n_shared:
                gate, up = F.linear(h, m.s_gu).chunk(2, dim=-1)
                y = y + F.linear(F.silu(gate) * up, m.s_down)
            x = x + y
        h = F.rms_norm(x, (cfg.d_model,), self.final_norm, cfg.rms_eps)
        logits = F.linear(h, self.head)[:, :cfg.vocab_size].float()
        return F.cross_entropy(logits, targets.reshape(-1)) + aux_total

    def sync_dense_grads(self):
        if self.W > 1:
            for p in self.dense_params:
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.group)
                    p.grad.div_(self.W)
            for p in self.expert_params:
                if p.grad is not None:
                    p.grad.div_(self.W)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_split, in_split, group):
        ctx.out_split, ctx.in_split, ctx.group = out_split, in_split, group
        out = x.new_empty((sum(out_split),) + x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_split, in_split, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_split),) + g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), ctx.in_split, ctx.out_split, group=ctx.group)
        return out, None, None, None


def run_1f1b(stage, stage_id, n_stages, prev_rank, next_rank, n_micro, act_shape, device, micro_inputs,
             micro_targets, device_type="cuda"):
    """Plain 1F1B over torch.distributed p2p, written out here so that this arm shares no code with the
    package. It follows the usual pairing of transfers: in the steady state a stage sends its activation
    forward and receives the matching gradient in ONE grouped call, and sends a gradient back and receives
    the next activation in one grouped call (NCCL transfers rendezvous, so two stages that each post a send
    first would wait for each other). Activations cross stages in bf16. Returns the mean loss on the last
    stage."""
    first, last = stage_id == 0, stage_id == n_stages - 1
    warm = min(n_stages - 1 - stage_id, n_micro)
    remaining = n_micro - warm
    saved, losses = [], []

    def exchange(send_t=None, send_to=None, recv_from=None):
        ops, buf = [], None
        if send_t is not None and send_to is not None:
            send_t = send_t.contiguous()
            ops.append(dist.P2POp(dist.isend, send_t, send_to))
        if recv_from is not None:
            buf = torch.empty(act_shape, dtype=torch.bfloat16, device=device)
            ops.append(dist.P2POp(dist.irecv, buf, recv_from))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return buf

    def fwd(i, x):
        x = micro_inputs[i] if first else x.requires_grad_(True)
        with torch.autocast(device_type, dtype=torch.bfloat16):
            y = stage(x, micro_targets[i] if last else None)
        if last:
            losses.append(y.detach())
            saved.append((x, y / n_micro))
            return None
        saved.append((x, y))
        return y.detach().to(torch.bfloat16)

    def bwd(g):
        x, y = saved.pop(0)
        if last:
            y.backward()
        else:
            y.backward(g.to(y.dtype))
        return None if first else x.grad

    fi = 0
    for _ in range(warm):
        x = exchange(recv_from=prev_rank)
        y = fwd(fi, x); fi += 1
        exchange(send_t=y, send_to=next_rank)
    x = exchange(recv_from=prev_rank) if remaining > 0 else None
    for k in range(remaining):
        y = fwd(fi, x); fi += 1
        g = exchange(send_t=y, send_to=next_rank, recv_from=next_rank)          # send forward, receive backward
        dx = bwd(g)
        more = k + 1 < remaining
        x = exchange(send_t=dx, send_to=prev_rank, recv_from=prev_rank if more else None)  # send backward, receive forward
    for _ in range(warm):
        g = exchange(recv_from=next_rank)
        dx = bwd(g)
        exchange(send_t=dx, send_to=prev_rank)
    return torch.stack([l.float() for l in losses]).mean() if last else None


def make_step(model, kind, device_type):
    """Returns ``step(tokens) -> loss`` running forward (bf16 autocast), backward, gradient sync and AdamW."""
    fused = device_type == "cuda"
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=fused)

    def step(tok):
        with torch.autocast(device_type, dtype=torch.bfloat16):
            loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if kind == "tp":
            model.sync_replicated_grads()
        else:
            model.sync_dense_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss
    return step
