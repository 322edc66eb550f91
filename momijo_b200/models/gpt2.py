"""GPT-2 style decoder (pre-LayerNorm, learned positions, GELU MLP, tied LM head).

The reference has no decoder model; it offers ``Linear``, ``LayerNorm1d`` and a forward-only
``MultiHeadAttention`` (legacy/src/momijo/learn/nn/attention.mojo:40-60,
legacy/src/momijo/learn/nn/transformer.mojo:27-61). This model is assembled from the same kinds
of layers, each backed by an sm_100a kernel: tcgen05 GEMMs with fused bias/GELU epilogues, flash
attention, LayerNorm fused with the residual add, and a fused LM-head cross-entropy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_ff: int = 3072
    max_seq: int = 1024
    init_std: float = 0.02
    ln_eps: float = 1e-5
    dtype: torch.dtype = torch.bfloat16

    @property
    def padded_vocab(self) -> int:
        return ops.pad_vocab(self.vocab_size)

    @staticmethod
    def small():
        return GPT2Config()

    @staticmethod
    def tiny():
        return GPT2Config(vocab_size=1000, n_layer=2, n_head=2, d_model=128, d_ff=512, max_seq=256)

    def num_params(self) -> int:
        c, f = self.d_model, self.d_ff
        per = (3 * c * c + 3 * c) + (c * c + c) + (c * f + f) + (f * c + c) + 4 * c
        return self.padded_vocab * c + self.max_seq * c + self.n_layer * per + 2 * c

    def flops_per_token(self, seq: int) -> float:
        """Training FLOPs per token (forward + backward), matmuls and attention."""
        c, f = self.d_model, self.d_ff
        dense = 2 * (3 * c * c + c * c + 2 * c * f) * self.n_layer + 2 * c * self.padded_vocab
        attn = 2 * 2 * seq * c * self.n_layer / 2  # causal: half of the score matrix
        return 3.0 * (dense + attn)


class GPT2Block(nn.Module):
    # sharded data parallel: the all-gather of this weight is fused into the GEMM that first uses it
    zero_first_gemm_weight = "w_qkv"

    def __init__(self, cfg: GPT2Config):
        super().__init__()
        c, f, dt = cfg.d_model, cfg.d_ff, cfg.dtype
        p = lambda *s: nn.Parameter(torch.empty(*s, dtype=dt))
        self.ln1_g, self.ln1_b = p(c), p(c)
        self.w_qkv, self.b_qkv = p(3 * c, c), p(3 * c)
        self.w_o, self.b_o = p(c, c), p(c)
        self.ln2_g, self.ln2_b = p(c), p(c)
        self.w_fc, self.b_fc = p(f, c), p(f)
        self.w_proj, self.b_proj = p(c, f), p(c)
        self.cfg = cfg

    def forward(self, delta, res, B, T):
        cfg = self.cfg
        H, D = cfg.n_head, cfg.d_model // cfg.n_head
        if delta is None:
            h = ops.layer_norm(res, self.ln1_g, self.ln1_b, cfg.ln_eps)
        else:
            h, res = ops.layer_norm(delta, self.ln1_g, self.ln1_b, cfg.ln_eps, residual=res)
        qkv = ops.linear(h, self.w_qkv, self.b_qkv)
        a = ops.attention_packed(qkv, B, T, H, H, D, causal=True)
        delta = ops.linear(a, self.w_o, self.b_o)
        h, res = ops.layer_norm(delta, self.ln2_g, self.ln2_b, cfg.ln_eps, residual=res)
        delta = ops.mlp_gelu(h, self.w_fc, self.b_fc, self.w_proj, self.b_proj)
        return delta, res


class GPT2(nn.Module):
    """``forward(tokens, targets)`` returns the mean next-token loss; ``logits(tokens)`` the logits."""

    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        dt = cfg.dtype
        self.wte = nn.Parameter(torch.empty(cfg.padded_vocab, cfg.d_model, dtype=dt))
        self.wpe = nn.Parameter(torch.empty(cfg.max_seq, cfg.d_model, dtype=dt))
        self.blocks = nn.ModuleList([GPT2Block(cfg) for _ in range(cfg.n_layer)])
        self.lnf_g = nn.Parameter(torch.empty(cfg.d_model, dtype=dt))
        self.lnf_b = nn.Parameter(torch.empty(cfg.d_model, dtype=dt))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: int | None = None):
        g = None
        if seed is not None:
            g = torch.Generator(device="cpu").manual_seed(seed)
        std = self.cfg.init_std
        for name, p in self.named_parameters():
            if name.endswith("_g"):
                p.fill_(1.0)
            elif name.endswith("_b") or ".b_" in name:
                p.zero_()
            else:
                s = std / math.sqrt(2 * self.cfg.n_layer) if name.endswith(("w_o", "w_proj")) else std
                p.copy_((torch.randn(p.shape, generator=g) * s).to(p.dtype))

    def hidden(self, tokens):
        B, T = tokens.shape
        res = ops.embedding(tokens, self.wte, self.wpe, T).reshape(B * T, self.cfg.d_model)
        delta = None
        for blk in self.blocks:
            delta, res = blk(delta, res, B, T)
        h, _ = ops.layer_norm(delta, self.lnf_g, self.lnf_b, self.cfg.ln_eps, residual=res)
        return h

    def forward(self, tokens, targets=None):
        h = self.hidden(tokens)
        if targets is None:
            return self.logits_from_hidden(h, tokens.shape)
        return ops.lm_head_cross_entropy(h, self.wte, targets, self.cfg.vocab_size)

    def logits_from_hidden(self, h, shape):
        lg = ops.linear(h, self.wte)[:, :self.cfg.vocab_size]
        return lg.reshape(*shape, self.cfg.vocab_size)

    def logits(self, tokens):
        return self.forward(tokens, None)
