"""parallel.DistributedDataParallel and HybridEngine on CPU: two gloo ranks with different batches end up
with the same parameters as one process on the concatenated batch."""
import os
import socket
import sys

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


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(5, 8, 16, generator=g), torch.randn(5, 8, 4, generator=g)


def _train(engine, xs, ys, lo, hi):
    for s in range(xs.shape[0]):
        loss = ((engine(xs[s, lo:hi]) - ys[s, lo:hi]) ** 2).mean()
        loss.backward()
        engine.step()
    return [p.detach().clone() for p in engine.module.parameters()]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, DistributedDataParallel

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    eng = DistributedDataParallel(_net(), AdamWConfig(lr=1e-2), dtype=torch.float32)
    params = _train(eng, xs, ys, rank * 4, rank * 4 + 4)
    if rank == 0:
        torch.save(params, out)
    dist.barrier()
    dist.destroy_process_group()


def test_ddp_two_ranks_match_single_process(tmp_path):
    from momijo_b200.parallel import AdamWConfig, DistributedDataParallel, HybridEngine

    xs, ys = _data()
    ref = _train(DistributedDataParallel(_net(), AdamWConfig(lr=1e-2), dtype=torch.float32), xs, ys, 0, 8)
    out = str(tmp_path / "p.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    for a, b in zip(ref, got):
        assert torch.allclose(a, b, atol=2e-5), (a - b).abs().max()
    # the same run through the hybrid engine (everything local) and through torch's own AdamW
    hyb = HybridEngine(_net(), AdamWConfig(lr=1e-2))
    for p in hyb.module.parameters():
        assert hasattr(p, "main_grad")
    net = _net()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    for s in range(xs.shape[0]):
        opt.zero_grad()
        ((net(xs[s]) - ys[s]) ** 2).mean().backward()
        opt.step()
    for a, b in zip(ref, net.parameters()):
        assert torch.allclose(a, b.detach(), atol=2e-5)


def test_found_inf_skips_update():
    from momijo_b200.parallel import AdamWConfig, DistributedDataParallel

    eng = DistributedDataParallel(_net(), AdamWConfig(lr=1e-2), dtype=torch.float32)
    before = [p.detach().clone() for p in eng.module.parameters()]
    xs, ys = _data()
    ((eng(xs[0]) - ys[0]) ** 2).mean().backward()
    assert eng.step(found_inf=True) is False
    for a, b in zip(before, eng.module.parameters()):
        assert torch.equal(a, b.detach())
