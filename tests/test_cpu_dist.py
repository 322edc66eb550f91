"""CPU plumbing config: MLP 784->256(ReLU)->10, fp32, batch 64 per rank, softmax cross-entropy,
SGD lr 0.01 momentum 0.9, 100 steps, seed 0. Two gloo ranks (data parallel through
``momijo_b200.learn.distributed``) must reproduce the single-process run on the concatenated
batch: same losses and all-reduced gradients equal to the single-process gradients."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STEPS = 100


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _build():
    import momijo_b200.learn as L

    torch.manual_seed(0)
    return L.Sequential(L.Linear(784, 256, dtype=torch.float32), L.ReLU(), L.Linear(256, 10, dtype=torch.float32))


def _data(world):
    g = torch.Generator().manual_seed(0)
    xs = torch.randn(STEPS, 64 * world, 784, generator=g)
    ys = torch.randint(0, 10, (STEPS, 64 * world), generator=g)
    return xs, ys


def _single(world):
    import momijo_b200.learn as L

    net = _build()
    opt = L.SGD(net.parameters(), lr=0.01, momentum=0.9)
    xs, ys = _data(world)
    losses, g0 = [], None
    for s in range(STEPS):
        loss = torch.nn.functional.cross_entropy(net(xs[s]), ys[s])
        opt.zero_grad()
        loss.backward()
        if s == 0:
            g0 = [p.grad.clone() for p in net.parameters()]
        opt.step()
        losses.append(loss.item())
    return losses, g0, [p.detach().clone() for p in net.parameters()]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import momijo_b200.learn as L
    from momijo_b200.learn import distributed as D

    pg = L.init_process_group("gloo", rank, world)
    assert D.get_rank() == rank and D.get_world_size() == world and L.get_rank_world() == (rank, world, True)
    net = _build()
    ddp = D.DistributedDataParallel(net)
    ddp.broadcast_parameters(0)
    opt = L.SGD(net.parameters(), lr=0.01, momentum=0.9)
    xs, ys = _data(world)
    losses, g0 = [], None
    for s in range(STEPS):
        x, y = xs[s, rank * 64:(rank + 1) * 64], ys[s, rank * 64:(rank + 1) * 64]
        loss = torch.nn.functional.cross_entropy(ddp(x), y)
        loss.backward()
        if s == 0:
            ddp.allreduce_gradients(average=True)
            g0 = [p.grad.clone() for p in net.parameters()]
            opt.step()
            opt.zero_grad()
        else:
            ddp.step_and_sync(opt, found_inf=False, average=True)
        losses.append(D.allreduce(loss.item(), D.ReduceOp.AVG))
    # facade checks with real semantics
    assert D.allreduce([1, 2]) == [world, 2 * world]
    assert D.broadcast(rank + 5, 0) == 5
    assert D.all_gather(torch.tensor([float(rank)])).tolist() == [float(r) for r in range(world)]
    assert D.reduce_scatter(torch.arange(2.0 * world)).tolist() == [2.0 * world * rank, world * (2 * rank + 1.0)]
    if rank == 0:
        torch.save({"losses": losses, "g0": g0, "params": [p.detach() for p in net.parameters()]}, out)
    D.barrier()
    L.destroy_process_group(pg)


def test_gloo_two_ranks_match_single_process(tmp_path):
    world = 2
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out)
    losses, g0, params = _single(world)
    for a, b in zip(got["g0"], g0):
        assert torch.allclose(a, b, atol=1e-6), "all-reduced gradients differ from single process"
    assert max(abs(a - b) for a, b in zip(got["losses"], losses)) < 1e-4
    for a, b in zip(got["params"], params):
        assert torch.allclose(a, b, atol=1e-5)
    assert losses[-1] < losses[0]
