"""Mixture-of-experts decoder: data-parallel attention, expert-parallel FFN (routed experts with a
top-k softmax router and load-balance auxiliary loss, plus shared experts).

The 16B-class shape of the benchmark config: 28 layers, d_model 2048, 16 heads, 64 routed experts
(SwiGLU, FFN 1408) + 2 shared experts, top-6, aux coefficient 0.01, vocab 102400. No counterpart
exists in the reference; layers follow its ``Linear`` style
(legacy/src/momijo/learn/nn/layers.mojo:343-359).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..parallel.ep import MoEDispatcher, MoELayer


@dataclass
class MoEConfig:
    vocab_size: int = 102400
    n_layer: int = 28
    d_model: int = 2048
    n_head: int = 16
    head_dim: int = 128
    n_experts: int = 64
    n_shared: int = 2
    top_k: int = 6
    d_ff_expert: int = 1408
    aux_coef: float = 0.01
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq: int = 4096
    init_std: float = 0.02
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def moe_16b():
        return MoEConfig()

    def flops_per_token(self, seq: int) -> float:
        """Forward + backward FLOPs per token (matrix products only; top-k routed + shared experts)."""
        c, hd = self.d_model, self.n_head * self.head_dim
        attn_proj = 2 * (3 * c * hd + hd * c)
        experts = 2 * 3 * c * self.d_ff_expert * (self.top_k + self.n_shared)
        router = 2 * c * self.n_experts
        dense = (attn_proj + experts + router) * self.n_layer + 2 * c * self.vocab_size
        attn = 2 * 2 * seq * hd * self.n_layer / 2
        return 3.0 * (dense + attn)

    @staticmethod
    def tiny():
        return MoEConfig(vocab_size=1024, n_layer=2, d_model=256, n_head=4, head_dim=64, n_experts=8,
                         n_shared=1, top_k=2, d_ff_expert=128, max_seq=256)


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, dispatcher=None, group=None):
        super().__init__()
        c, dt = cfg.d_model, cfg.dtype
        self.cfg = cfg
        self.attn_norm = nn.Parameter(torch.ones(c, dtype=dt))
        self.mlp_norm = nn.Parameter(torch.ones(c, dtype=dt))
        qkv = 3 * cfg.n_head * cfg.head_dim
        self.wqkv = nn.Parameter(torch.empty(qkv, c, dtype=dt))
        self.wo = nn.Parameter(torch.empty(c, cfg.n_head * cfg.head_dim, dtype=dt))
        nn.init.normal_(self.wqkv, 0.0, cfg.init_std)
        nn.init.normal_(self.wo, 0.0, cfg.init_std)
        self.moe = MoELayer(c, cfg.d_ff_expert, cfg.n_experts, cfg.top_k, cfg.n_shared, cfg.aux_coef,
                            dispatcher, dtype=dt, init_std=cfg.init_std, group=group)

    def forward(self, delta, res, B, T):
        cfg = self.cfg
        if delta is None:
            h = ops.rms_norm(res, self.attn_norm, cfg.rms_eps)
        else:
            h, res = ops.rms_norm(delta, self.attn_norm, cfg.rms_eps, residual=res)
        qkv = ops.linear(h, self.wqkv)
        rope = ops.rope_table(T, cfg.head_dim, cfg.rope_theta, qkv.device)
        a = ops.attention_packed(qkv, B, T, cfg.n_head, cfg.n_head, cfg.head_dim, causal=True, rope=rope)
        delta = ops.linear(a, self.wo)
        h, res = ops.rms_norm(delta, self.mlp_norm, cfg.rms_eps, residual=res)
        delta, aux = self.moe(h)
        return delta, res, aux


class MoEDecoder(nn.Module):
    """``forward(tokens, targets)`` -> (cross-entropy + auxiliary loss). ``comm``: the peer
    communicator of the expert-parallel group; ``group``: a torch.distributed process group instead (tokens
    travel by ``all_to_all_single``: any backend, no capacity limit); neither: every expert on this rank."""

    def __init__(self, cfg: MoEConfig, comm=None, max_tokens: int = 16384, capacity_factor: float = 2.0,
                 group=None):
        super().__init__()
        self.cfg = cfg
        self.dispatcher = None
        if comm is not None:
            self.dispatcher = MoEDispatcher(comm, cfg.n_experts, cfg.top_k, cfg.d_model, max_tokens,
                                            capacity_factor)
        dt = cfg.dtype
        self.wte = nn.Parameter(torch.empty(ops.pad_vocab(cfg.vocab_size), cfg.d_model, dtype=dt))
        nn.init.normal_(self.wte, 0.0, cfg.init_std)
        self.blocks = nn.ModuleList([MoEBlock(cfg, self.dispatcher, group if comm is None else None)
                                     for _ in range(cfg.n_layer)])
        self.final_norm = nn.Parameter(torch.ones(cfg.d_model, dtype=dt))
        self.lm_head = nn.Parameter(torch.empty(ops.pad_vocab(cfg.vocab_size), cfg.d_model, dtype=dt))
        nn.init.normal_(self.lm_head, 0.0, cfg.init_std)

    def expert_parameters(self):
        """Parameters that differ per rank (not to be averaged across the data-parallel group)."""
        return [p for b in self.blocks for p in (b.moe.w_gu, b.moe.w_down)]

    def forward(self, tokens, targets=None):
        B, T = tokens.shape
        res = ops.embedding(tokens, self.wte).reshape(B * T, self.cfg.d_model)
        delta, aux_total = None, 0.0
        for blk in self.blocks:
            delta, res, aux = blk(delta, res, B, T)
            aux_total = aux_total + aux
        h, _ = ops.rms_norm(delta, self.final_norm, self.cfg.rms_eps, residual=res)
        if targets is None:
            return ops.linear(h, self.lm_head)[:, :self.cfg.vocab_size]
        return ops.lm_head_cross_entropy(h, self.lm_head, targets, self.cfg.vocab_size) + aux_total
