"""ShardedDataParallel host logic on CPU: two gloo ranks (buckets per block, stages 1-3, parameter window,
gradient pool, clipping by the global norm) end up with the parameters of one process that runs plain
torch AdamW on the concatenated batch."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _MGLinear(torch.autograd.Function):
    """A linear layer that, like the native kernels' front ends, writes its weight and bias gradients
    straight into ``main_grad`` during its own backward call and hands autograd ``None`` for them."""

    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.refs = (w, b)
        return x @ w.t() + b

    @staticmethod
    def backward(ctx, dy):
        from momijo_b200.ops.functional import _wgrad_target

        x, w = ctx.saved_tensors
        rw, rb = ctx.refs
        out = []
        for p, g in ((rw, dy.t() @ x), (rb, dy.sum(0))):
            buf, acc = _wgrad_target(p)
            if buf is None:
                out.append(g)
            else:
                buf.copy_(buf + g if acc else g)
                out.append(None)
        return dy @ w, out[0], out[1]


class _Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.a, self.b = nn.Linear(c, 2 * c), nn.Linear(2 * c, c)

    def forward(self, x):
        h = torch.tanh(_MGLinear.apply(x, self.a.weight, self.a.bias))
        return x + _MGLinear.apply(h, self.b.weight, self.b.bias)


class _Net(nn.Module):
    def __init__(self, c=24, n=5):
        super().__init__()
        self.inp = nn.Linear(8, c)
        self.blocks = nn.ModuleList([_Block(c) for _ in range(n)])
        self.out = nn.Linear(c, 4)

    def forward(self, x):
        x = self.inp(x)
        for b in self.blocks:
            x = b(x)
        return self.out(x)


def _net():
    torch.manual_seed(0)
    return _Net()


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(4, 8, 8, generator=g), torch.randn(4, 8, 4, generator=g)


def _worker(rank, world, port, out, stage, clip, overlap=True):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    eng = ShardedDataParallel(_net(), AdamWConfig(lr=1e-2, weight_decay=0.1), stage=stage, comm=TorchDistComm(),
                              grad_clip=clip, overlap=overlap, window=2, grad_slots=2)
    assert len(eng.buckets) == 6   # five blocks + root
    lo, hi = rank * 4, rank * 4 + 4
    for s in range(xs.shape[0]):
        loss = ((eng(xs[s, lo:hi]) - ys[s, lo:hi]) ** 2).mean()
        loss.backward()
        eng.step()
    full = eng.materialize()
    rep = eng.memory_report()
    if rank == 0:
        torch.save({"params": full, "report": rep}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("stage", [1, 2, 3])
@pytest.mark.parametrize("clip", [None, 0.05])
def test_sharded_stages_match_plain_adamw(tmp_path, stage, clip):
    xs, ys = _data()
    net = _net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for s in range(xs.shape[0]):
        opt.zero_grad()
        ((net(xs[s]) - ys[s]) ** 2).mean().backward()
        if clip is not None:
            torch.nn.utils.clip_grad_norm_(net.parameters(), clip)
        opt.step()
    out = str(tmp_path / "p.pt")
    mp.spawn(_worker, args=(2, _free_port(), out, stage, clip), nprocs=2, join=True)
    got = torch.load(out)
    for name, p in net.named_parameters():
        assert torch.allclose(got["params"][name], p.detach(), atol=3e-5), (name, (got["params"][name] - p).abs().max())
    rep = got["report"]
    assert rep["stage"] == stage and rep["buckets"] == 6
    full = rep["unsharded_param_bytes"]
    if stage == 1:
        assert rep["grad_bytes"] == full and rep["param_bytes"] == full
    if stage >= 2:
        assert rep["grad_bytes"] < full
    if stage == 3:
        assert rep["param_bytes"] < full


def _ddp_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, DistributedDataParallel

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    eng = DistributedDataParallel(_net(), AdamWConfig(lr=1e-2, weight_decay=0.1), dtype=torch.float32)
    lo, hi = rank * 4, rank * 4 + 4
    sent = []
    for s in range(xs.shape[0]):
        loss = ((eng(xs[s, lo:hi]) - ys[s, lo:hi]) ** 2).mean()
        loss.backward()
        sent.append(sum(b.launched for b in eng.buckets))
        eng.step()
    if rank == 0:
        torch.save({"params": {n: p.detach().clone() for n, p in eng.module.named_parameters()}, "sent": sent,
                    "modes": [b.mode for b in eng.buckets]}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_ddp_overlaps_and_matches_plain_adamw(tmp_path):
    xs, ys = _data()
    net = _net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for s in range(xs.shape[0]):
        opt.zero_grad()
        ((net(xs[s]) - ys[s]) ** 2).mean().backward()
        opt.step()
    out = str(tmp_path / "d.pt")
    mp.spawn(_ddp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    for name, p in net.named_parameters():
        assert torch.allclose(got["params"][name], p.detach(), atol=3e-5), name
    # first step learns how gradients arrive; afterwards the five block buckets leave during backward
    assert got["sent"][0] == 0 and all(n == 5 for n in got["sent"][1:]), got["sent"]
    assert got["modes"].count("native") == 5


def _accum_worker(rank, world, port, out, stage):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    eng = ShardedDataParallel(_net(), AdamWConfig(lr=1e-2, weight_decay=0.1), stage=stage, comm=TorchDistComm(),
                              window=2, grad_slots=2)
    lo = rank * 4
    for s in range(xs.shape[0]):
        # this rank's four rows as two micro-batches of two: the first only accumulates
        with eng.no_sync():
            (((eng(xs[s, lo:lo + 2]) - ys[s, lo:lo + 2]) ** 2).mean() / 2).backward()
        assert eng._accum is not None or stage == 1
        (((eng(xs[s, lo + 2:lo + 4]) - ys[s, lo + 2:lo + 4]) ** 2).mean() / 2).backward()
        eng.step()
        assert eng._accum is None
    full = eng.materialize()
    if rank == 0:
        torch.save({"params": full}, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("stage", [1, 2, 3])
def test_gradient_accumulation_over_micro_batches_matches_the_full_batch(tmp_path, stage):
    xs, ys = _data()
    net = _net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for s in range(xs.shape[0]):
        opt.zero_grad()
        ((net(xs[s]) - ys[s]) ** 2).mean().backward()
        opt.step()
    out = str(tmp_path / "a.pt")
    mp.spawn(_accum_worker, args=(2, _free_port(), out, stage), nprocs=2, join=True)
    got = torch.load(out)
    for name, p in net.named_parameters():
        assert torch.allclose(got["params"][name], p.detach(), atol=3e-5), (stage, name)


class _Loader:
    """The loader protocol of the fit loop: ``dataset.__len__``, ``batch_size``, ``get_batch(step)``."""

    def __init__(self, xs, ys):
        self.xs, self.ys = xs, ys
        self.dataset = list(range(xs.shape[0] * xs.shape[1]))
        self.batch_size = xs.shape[1]

    def get_batch(self, step):
        return self.xs[step], self.ys[step]


def _trainer_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.learn.engine.trainer import Trainer
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()                                   # 4 steps x 8 rows
    lo = rank * 4
    # two micro-batches of two rows per optimizer step and rank
    mx = xs[:, lo:lo + 4].reshape(8, 2, 8)
    my = ys[:, lo:lo + 4].reshape(8, 2, 4)
    eng = ShardedDataParallel(_net(), AdamWConfig(lr=1e-2, weight_decay=0.1), stage=3, comm=TorchDistComm(),
                              window=2, grad_slots=2)
    tr = Trainer(epochs=1, grad_accum_steps=2, verbose=False)
    tr.set_optimizer(eng).set_loss(lambda p, t: ((p - t) ** 2).mean())
    tr.fit(eng, _Loader(mx, my))
    assert eng.step_count == 4
    full = eng.materialize()
    if rank == 0:
        torch.save({"params": full}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_fit_loop_accumulates_micro_batches_through_a_sharded_engine(tmp_path):
    xs, ys = _data()
    net = _net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    for s in range(xs.shape[0]):
        opt.zero_grad()
        ((net(xs[s]) - ys[s]) ** 2).mean().backward()
        opt.step()
    out = str(tmp_path / "t.pt")
    mp.spawn(_trainer_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    for name, p in net.named_parameters():
        assert torch.allclose(got["params"][name], p.detach(), atol=3e-5), name
