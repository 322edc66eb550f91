"""Context parallelism for long sequences: Ulysses-style attention.

The reference has no long-context mechanism (its attention builds one score row at a time,
legacy/src/momijo/learn/nn/attention.mojo:122-161). Here a sequence can be split over the ranks of a
``cp_group``: every rank holds ``T / P`` consecutive tokens of each sequence through the whole model
(norms, MLPs and projections are token-local). Attention needs every token, so around the attention
kernel two all-to-all exchanges re-partition the packed Q | K | V projection from *sequence-sharded,
all heads* to *full sequence, heads / P* and the attention output back:

  [B, T/P, (Hq + 2 Hkv) D]  --all-to-all-->  [B, T, (Hq + 2 Hkv) D / P]  --attention-->
  [B, T, Hq D / P]          --all-to-all-->  [B, T/P, Hq D]

Each rank runs the flash-attention kernel on its own heads over the full sequence, so causal masking and
the RoPE positions need no special handling; the communication volume per rank is the size of the local
projection, independent of P. Heads (query and key/value) must divide by P. The exchanges are
differentiable (the backward of an all-to-all is the inverse all-to-all).

``context_parallel_attention`` is the hook: pass ``cp_group`` (a torch.distributed group, or ``None`` /
a group of one rank for the plain single-rank call).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops


def _world(group) -> int:
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


class _SeqToHeads(torch.autograd.Function):
    """[B, T/P, H, D] (all heads, local tokens) -> [B, T, H/P, D] (local heads, all tokens)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = _world(group)
        B, Tl, H, D = x.shape
        # destination rank p gets heads [p H/P, (p+1) H/P): make that the leading dimension
        send = x.reshape(B, Tl, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()      # [P, B, Tl, H/P, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)                                   # recv[p] = rank p's tokens
        return recv.permute(1, 0, 2, 3, 4).reshape(B, P * Tl, H // P, D)

    @staticmethod
    def backward(ctx, g):
        return _HeadsToSeq.apply(g, ctx.group), None


class _HeadsToSeq(torch.autograd.Function):
    """[B, T, H/P, D] -> [B, T/P, H, D]: the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = _world(group)
        B, T, Hl, D = x.shape
        Tl = T // P
        send = x.reshape(B, P, Tl, Hl, D).permute(1, 0, 2, 3, 4).contiguous()             # [P, B, Tl, H/P, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)                                   # recv[p] = heads of rank p
        return recv.permute(1, 2, 0, 3, 4).reshape(B, Tl, P * Hl, D)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHeads.apply(g, ctx.group), None


def context_parallel_attention(qkv, B: int, T_local: int, Hq: int, Hkv: int, D: int, causal: bool = True,
                               scale: Optional[float] = None, rope_theta: Optional[float] = None, cp_group=None):
    """Attention over sequences that are split into ``P = |cp_group|`` consecutive chunks of ``T_local`` tokens.

    ``qkv``: this rank's packed projection ``[B * T_local, (Hq + 2 Hkv) * D]`` (Q | K | V). Returns
    ``[B * T_local, Hq * D]``. ``rope_theta``: apply rotary embeddings at the global positions."""
    P = _world(cp_group)
    if P == 1:
        rope = ops.rope_table(T_local, D, rope_theta, qkv.device) if rope_theta else None
        return ops.attention_packed(qkv, B, T_local, Hq, Hkv, D, causal=causal, scale=scale, rope=rope)
    if Hq % P or Hkv % P:
        raise ValueError(f"context parallel attention needs head counts divisible by the group size "
                         f"(Hq={Hq}, Hkv={Hkv}, P={P})")
    T = T_local * P
    q, k, v = qkv.reshape(B, T_local, Hq + 2 * Hkv, D).split([Hq, Hkv, Hkv], dim=2)
    q = _SeqToHeads.apply(q, cp_group)                    # [B, T, Hq/P, D]
    k = _SeqToHeads.apply(k, cp_group)
    v = _SeqToHeads.apply(v, cp_group)
    hq, hkv = Hq // P, Hkv // P
    packed = torch.cat([q, k, v], dim=2).reshape(B * T, (hq + 2 * hkv) * D)
    rope = ops.rope_table(T, D, rope_theta, qkv.device) if rope_theta else None
    out = ops.attention_packed(packed, B, T, hq, hkv, D, causal=causal, scale=scale, rope=rope)
    out = _HeadsToSeq.apply(out.reshape(B, T, hq, D), cp_group)   # [B, T_local, Hq, D]
    return out.reshape(B * T_local, Hq * D)


def shard_sequence(tokens: torch.Tensor, cp_group=None, dim: int = 1) -> torch.Tensor:
    """This rank's chunk of a ``[B, T, ...]`` tensor (consecutive ``T / P`` positions)."""
    P = _world(cp_group)
    if P == 1:
        return tokens
    r = dist.get_rank(cp_group)
    n = tokens.shape[dim] // P
    return tokens.narrow(dim, r * n, n)
