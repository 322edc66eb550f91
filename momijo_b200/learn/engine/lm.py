"""Language-model training step used by the trainer and the benchmark.

``train_step_e2e(engine, host_tokens)`` is the whole user-visible step: copy the pinned host
batch to the device, forward, backward, optimizer step, and read the loss back to the host.
"""
from __future__ import annotations

import torch


def train_step(engine, tokens: torch.Tensor):
    """tokens: int64 [B, T+1] on the device. Returns the device loss tensor."""
    loss = engine(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    engine.step()
    return loss


def train_step_e2e(engine, host_tokens: torch.Tensor) -> float:
    """host_tokens: pinned int64 [B, T+1]. Includes the H2D copy and the D2H loss read."""
    dev = next(engine.parameters()).device
    tok = host_tokens.to(dev, non_blocking=True)
    return float(train_step(engine, tok).detach())
