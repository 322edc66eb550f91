"""Llama-style decoder (RMSNorm, rotary embedding, grouped-query attention, SwiGLU), optionally
tensor parallel with sequence-parallel activations.

None of these layer types exist in the reference (its transformer is an attention + hard-tanh FFN
stack without norms, legacy/src/momijo/learn/nn/transformer.mojo:27-61); they follow its layer
style and are backed by the sm_100a kernels: RMSNorm fused with the residual add, RoPE applied in
place on the packed QKV projection, flash attention with GQA, SwiGLU, and for ``tp.world > 1`` the
fused all-gather->GEMM / GEMM->reduce-scatter kernels of ``parallel.tp``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..parallel.tp import (ColumnParallelLinear, RowParallelLinear, TPContext, VocabParallelEmbedding,
                           vocab_parallel_cross_entropy)


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    n_layer: int = 32
    d_model: int = 4096
    n_head: int = 32
    n_kv_head: int = 8
    head_dim: int = 128
    d_ff: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq: int = 4096
    init_std: float = 0.02
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def llama3_8b():
        return LlamaConfig()

    @staticmethod
    def llama2_13b():
        return LlamaConfig(vocab_size=32000, n_layer=40, d_model=5120, n_head=40, n_kv_head=40,
                           head_dim=128, d_ff=13824, rope_theta=10000.0)

    @staticmethod
    def tiny():
        return LlamaConfig(vocab_size=1024, n_layer=2, d_model=256, n_head=4, n_kv_head=2, head_dim=64,
                           d_ff=512, max_seq=256)

    def flops_per_token(self, seq: int) -> float:
        c, f = self.d_model, self.d_ff
        qkv = (self.n_head + 2 * self.n_kv_head) * self.head_dim
        dense = 2 * (c * qkv + self.n_head * self.head_dim * c + 3 * c * f) * self.n_layer + 2 * c * self.vocab_size
        attn = 2 * 2 * seq * self.n_head * self.head_dim * self.n_layer / 2
        return 3.0 * (dense + attn)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, layer_id: int = 0):
        super().__init__()
        W = tp.world
        if cfg.n_head % W or cfg.n_kv_head % W:
            raise ValueError("heads must divide by the tensor-parallel size")
        self.cfg, self.tp = cfg, tp
        self.hq, self.hkv, self.D = cfg.n_head // W, cfg.n_kv_head // W, cfg.head_dim
        c, dt = cfg.d_model, cfg.dtype
        self.attn_norm = nn.Parameter(torch.ones(c, dtype=dt))
        self.mlp_norm = nn.Parameter(torch.ones(c, dtype=dt))
        # held in full by every tensor-parallel rank, each of which sees 1/world of the rows
        self.attn_norm.tp_replicated = True
        self.mlp_norm.tp_replicated = True
        qkv_cols = (cfg.n_head + 2 * cfg.n_kv_head) * cfg.head_dim
        k = lambda n: (layer_id, n)
        self.wqkv = ColumnParallelLinear(c, qkv_cols, tp, bias=False, dtype=dt, init_std=cfg.init_std, key=k("qkv"))
        self.wo = RowParallelLinear(cfg.n_head * cfg.head_dim, c, tp, bias=False, dtype=dt,
                                    init_std=cfg.init_std, key=k("o"))
        self.w_gu = ColumnParallelLinear(c, 2 * cfg.d_ff, tp, bias=False, dtype=dt, init_std=cfg.init_std, key=k("gu"))
        self.w_down = RowParallelLinear(cfg.d_ff, c, tp, bias=False, dtype=dt, init_std=cfg.init_std, key=k("down"))

    def forward(self, delta, res, B, T):
        """``res``: residual stream rows of this rank ([M/W, C]); ``delta``: branch output to add."""
        cfg = self.cfg
        if delta is None:
            h = ops.rms_norm(res, self.attn_norm, cfg.rms_eps)
        else:
            h, res = ops.rms_norm(delta, self.attn_norm, cfg.rms_eps, residual=res)
        qkv = self.wqkv(h)                                           # [M, local qkv cols]
        rope = ops.rope_table(T, self.D, cfg.rope_theta, qkv.device)
        a = ops.attention_packed(qkv, B, T, self.hq, self.hkv, self.D, causal=True, rope=rope)
        delta = self.wo(a)                                           # [M/W, C]
        h, res = ops.rms_norm(delta, self.mlp_norm, cfg.rms_eps, residual=res)
        delta = self.w_down(ops.swiglu(self.w_gu(h)))
        return delta, res


class Llama(nn.Module):
    """``forward(tokens, targets)`` -> mean next-token loss (identical on all tensor-parallel ranks)."""

    def __init__(self, cfg: LlamaConfig, tp: TPContext | None = None, layers=None):
        super().__init__()
        self.cfg = cfg
        self.tp = tp or TPContext()
        dt = cfg.dtype
        self.embed = VocabParallelEmbedding(cfg.vocab_size, cfg.d_model, self.tp, dtype=dt, init_std=cfg.init_std)
        ids = range(cfg.n_layer) if layers is None else layers
        self.blocks = nn.ModuleList([LlamaBlock(cfg, self.tp, i) for i in ids])
        self.final_norm = nn.Parameter(torch.ones(cfg.d_model, dtype=dt))
        self.final_norm.tp_replicated = True
        v_pad = (cfg.vocab_size + self.tp.world * 8 - 1) // (self.tp.world * 8) * (self.tp.world * 8)
        self.v_local = v_pad // self.tp.world
        self.lm_head = ColumnParallelLinear(cfg.d_model, v_pad, self.tp, bias=False, dtype=dt,
                                            init_std=cfg.init_std, key=("head",))

    def hidden(self, tokens):
        B, T = tokens.shape
        res = self.embed(tokens)                       # [M/W, C]
        delta = None
        for blk in self.blocks:
            delta, res = blk(delta, res, B, T)
        h, _ = ops.rms_norm(delta, self.final_norm, self.cfg.rms_eps, residual=res)
        return h

    def forward(self, tokens, targets=None):
        h = self.hidden(tokens)
        logits = self.lm_head(h)                       # [M, V/W]
        if targets is None:
            return logits
        start = self.tp.rank * self.v_local
        valid = min(self.v_local, max(0, self.cfg.vocab_size - start))
        return vocab_parallel_cross_entropy(logits, targets, start, valid, self.tp)


class LlamaStage(nn.Module):
    """One pipeline stage of a (tensor-parallel) Llama: a contiguous range of blocks, plus the
    embedding on the first stage and the final norm / head / loss on the last one. Between stages the
    residual stream travels as one [M/W, C] tensor per tensor-parallel rank (branch output already
    added)."""

    def __init__(self, cfg: LlamaConfig, tp: TPContext, layers: range, first: bool, last: bool):
        super().__init__()
        self.cfg, self.tp, self.first, self.last = cfg, tp, first, last
        dt = cfg.dtype
        self.embed = VocabParallelEmbedding(cfg.vocab_size, cfg.d_model, tp, dtype=dt, init_std=cfg.init_std) \
            if first else None
        self.blocks = nn.ModuleList([LlamaBlock(cfg, tp, i) for i in layers])
        if last:
            self.final_norm = nn.Parameter(torch.ones(cfg.d_model, dtype=dt))
            self.final_norm.tp_replicated = True
            v_pad = (cfg.vocab_size + tp.world * 8 - 1) // (tp.world * 8) * (tp.world * 8)
            self.v_local = v_pad // tp.world
            self.lm_head = ColumnParallelLinear(cfg.d_model, v_pad, tp, bias=False, dtype=dt,
                                                init_std=cfg.init_std, key=("head",))
        self.batch_shape = None  # (B, T) of a micro-batch; set by the caller on non-first stages

    def forward(self, x):
        if self.first:
            B, T = x.shape
            res = self.embed(x)
        else:
            B, T = self.batch_shape
            res = x
        delta = None
        for blk in self.blocks:
            delta, res = blk(delta, res, B, T)
        if not self.last:
            return res + delta if delta is not None else res
        h, _ = ops.rms_norm(delta, self.final_norm, self.cfg.rms_eps, residual=res)
        return h

    def loss(self, h, targets):
        logits = self.lm_head(h)
        start = self.tp.rank * self.v_local
        valid = min(self.v_local, max(0, self.cfg.vocab_size - start))
        return vocab_parallel_cross_entropy(logits, targets, start, valid, self.tp)
