"""Ulysses-style context-parallel attention on two gloo ranks == single-rank attention on the full sequence,
forward and gradients (causal, GQA, RoPE at global positions)."""
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B, T, HQ, HKV, D = 2, 32, 4, 2, 16


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs():
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, T, (HQ + 2 * HKV) * D, generator=g)
    dy = torch.randn(B, T, HQ * D, generator=g)
    return qkv, dy


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import context_parallel_attention, shard_sequence

    dist.init_process_group("gloo", rank=rank, world_size=world)
    qkv, dy = _inputs()
    mine = shard_sequence(qkv, dist.group.WORLD).clone().requires_grad_(True)
    Tl = T // world
    y = context_parallel_attention(mine.reshape(B * Tl, -1), B, Tl, HQ, HKV, D, causal=True, rope_theta=10000.0,
                                   cp_group=dist.group.WORLD)
    y.backward(shard_sequence(dy, dist.group.WORLD).reshape(B * Tl, -1))
    torch.save({"y": y.detach().reshape(B, Tl, -1), "g": mine.grad}, out + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_context_parallel_attention_matches_full_sequence(tmp_path):
    from momijo_b200.parallel import context_parallel_attention

    qkv, dy = _inputs()
    full = qkv.clone().requires_grad_(True)
    y = context_parallel_attention(full.reshape(B * T, -1), B, T, HQ, HKV, D, causal=True, rope_theta=10000.0)
    y.backward(dy.reshape(B * T, -1))
    out = str(tmp_path / "cp.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    parts = [torch.load(out + f".{r}") for r in range(2)]
    ys = torch.cat([p["y"] for p in parts], dim=1)
    gs = torch.cat([p["g"] for p in parts], dim=1)
    assert torch.allclose(ys, y.detach().reshape(B, T, -1), atol=1e-5)
    assert torch.allclose(gs, full.grad, atol=1e-5)
