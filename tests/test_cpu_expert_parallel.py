"""Expert parallelism over torch.distributed (gloo, two ranks): the all-to-all path of ``MoELayer`` gives the
outputs and gradients of one process that holds every expert."""
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel.ep import MoELayer

    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, F, E, k, n = 16, 24, 4, 2, 10
    torch.manual_seed(0)                                         # the same full model on every rank
    ref = MoELayer(H, F, E, k, n_shared=1, world=1, dtype=torch.float32)
    ep = MoELayer(H, F, E, k, n_shared=1, group=dist.group.WORLD, dtype=torch.float32)
    epr = E // world
    with torch.no_grad():
        ep.router.weight.copy_(ref.router.weight)
        ep.w_gu.copy_(ref.w_gu[rank * epr:(rank + 1) * epr])
        ep.w_down.copy_(ref.w_down[rank * epr:(rank + 1) * epr])
        for a, b in zip(ep.shared.parameters(), ref.shared.parameters()):
            a.copy_(b)
    torch.manual_seed(10 + rank)                                 # every rank routes its own tokens
    x = torch.randn(n, H)
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    y_ref, aux_ref = ref(x1)
    y_ep, aux_ep = ep(x2)
    assert torch.allclose(y_ep, y_ref, atol=1e-5), (y_ep - y_ref).abs().max()
    assert torch.allclose(aux_ep, aux_ref, atol=1e-6)
    dy = torch.randn(n, H)
    (y_ref * dy).sum().backward()
    (y_ep * dy).sum().backward()
    assert torch.allclose(x2.grad, x1.grad, atol=1e-5)
    assert torch.allclose(ep.router.weight.grad, ref.router.weight.grad, atol=1e-5)
    # an expert's weights see the tokens of every rank: compare with the sum of the single-process gradients
    for name in ("w_gu", "w_down"):
        full = getattr(ref, name).grad.clone()
        dist.all_reduce(full)
        got = getattr(ep, name).grad
        assert torch.allclose(got, full[rank * epr:(rank + 1) * epr], atol=1e-5), name
    dist.barrier()
    dist.destroy_process_group()


def test_all_to_all_expert_parallel_matches_one_process():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
