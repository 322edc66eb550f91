"""Checkpoint / resume of ShardedDataParallel: the optimizer state written per rank in the MNP layout is
restored by a run with the same or another world size, and training continues as if never interrupted."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

from test_cpu_zero_stages import ROOT, _data, _free_port, _net


def _step(eng, xs, ys, s, lo, hi):
    dt = next(eng.module.parameters()).dtype   # a single-rank engine re-homes its parameters as bf16
    loss = ((eng(xs[s, lo:hi].to(dt)).float() - ys[s, lo:hi]) ** 2).mean()
    loss.backward()
    eng.step()


def test_single_rank_resume_is_exact(tmp_path):
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel

    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    a = ShardedDataParallel(_net(), cfg)
    for s in range(2):
        _step(a, xs, ys, s, 0, 8)
    base = str(tmp_path / "ck" / "opt")
    a.save_checkpoint(base, extra={"note": "after two steps"})
    assert os.path.exists(base + ".json") and os.path.exists(base + ".bin")
    _step(a, xs, ys, 2, 0, 8)
    want = a.materialize()

    b = ShardedDataParallel(_net(), cfg)
    extra = b.load_checkpoint(base)
    assert extra["note"] == "after two steps" and extra["step_count"] == 2 and b.step_count == 2
    _step(b, xs, ys, 2, 0, 8)
    got = b.materialize()
    for k in want:
        assert torch.equal(got[k], want[k]), k


def _worker(rank, world, port, tmp, stage):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    lo, hi = rank * 4, rank * 4 + 4
    base = os.path.join(tmp, "opt")

    def make():
        return ShardedDataParallel(_net(), cfg, stage=stage, comm=TorchDistComm(), window=2, grad_slots=2)

    a = make()
    for s in range(2):
        _step(a, xs, ys, s, lo, hi)
    a.save_checkpoint(base)
    assert os.path.exists(f"{base}.rank{rank}of{world}.bin")
    _step(a, xs, ys, 2, lo, hi)
    want = a.materialize()

    # same world size: exact continuation
    b = make()
    extra = b.load_checkpoint(base)
    assert extra["world"] == world and b.step_count == 2
    _step(b, xs, ys, 2, lo, hi)
    got = b.materialize()
    for k in want:
        assert torch.equal(got[k], want[k]), (stage, k)

    # one rank reads the two-rank checkpoint (the pieces are re-split for its single flat buffer), writes
    # it again as a one-rank checkpoint, and two ranks read that: every element of master / m / v comes back
    from momijo_b200.parallel.zero_ckpt import owned_pieces

    fresh = make()
    fresh.load_checkpoint(base)
    params_after_load = fresh.materialize()       # fp32 parameters republished from the master weights
    base1 = os.path.join(tmp, "opt_one_rank")
    if rank == 0:
        c = ShardedDataParallel(_net(), cfg)
        c.load_checkpoint(base)
        assert c.step_count == 2
        for name, lo_, hi_, at in owned_pieces(c):
            assert torch.equal(c.master[at:at + hi_ - lo_], params_after_load[name].reshape(-1)[lo_:hi_]), name
        c.save_checkpoint(base1)
    dist.barrier()
    d = make()
    d.load_checkpoint(base1)
    for k in ("master", "m", "v"):
        assert torch.equal(getattr(d, k), getattr(fresh, k)), (stage, k)
    assert d.step_count == 2
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("stage", [1, 3])
def test_two_rank_resume_and_resharding(tmp_path, stage):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path), stage), nprocs=2, join=True)


def _hybrid_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, HybridEngine
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    lo, hi = rank * 4, rank * 4 + 4
    base = os.path.join(tmp, "hybrid")

    def make():
        net = _net().to(torch.bfloat16)   # one dtype for both parts, as on the GPU
        # the blocks are data parallel (sharded), the input / output layers are each rank's own
        dp = [p for b in net.blocks for p in b.parameters()]
        return HybridEngine(net, cfg, dp_comm=TorchDistComm(), dp_params=dp)

    a = make()
    for s in range(2):
        _step(a, xs, ys, s, lo, hi)
    a.save_checkpoint(base)
    assert os.path.exists(f"{base}.local{rank}.bin") and os.path.exists(f"{base}.dp.rank{rank}of{world}.bin")
    _step(a, xs, ys, 2, lo, hi)
    b = make()
    b.load_checkpoint(base)
    _step(b, xs, ys, 2, lo, hi)
    for (n1, p1), (n2, p2) in zip(a.module.named_parameters(), b.module.named_parameters()):
        if n1.startswith("blocks"):
            continue   # sharded storage: compared through materialize below
        assert torch.equal(p1, p2), n1
    wa, wb = a.dp.materialize(), b.dp.materialize()
    for k in wa:
        if k.startswith("blocks"):
            assert torch.equal(wa[k], wb[k]), k
    dist.barrier()
    dist.destroy_process_group()


def test_hybrid_engine_resume(tmp_path):
    port = _free_port()
    mp.spawn(_hybrid_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)


def _ddp_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.parallel import AdamWConfig, DistributedDataParallel, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    lo, hi = rank * 4, rank * 4 + 4
    base = os.path.join(tmp, "ddp")
    a = DistributedDataParallel(_net(), cfg, dtype=torch.float32)
    for s in range(2):
        _step(a, xs, ys, s, lo, hi)
    a.save_checkpoint(base, extra={"epoch": 7})
    assert os.path.exists(base + ".bin")
    _step(a, xs, ys, 2, lo, hi)
    b = DistributedDataParallel(_net(), cfg, dtype=torch.float32)
    extra = b.load_checkpoint(base)
    assert extra["epoch"] == 7 and b.step_count == 2
    _step(b, xs, ys, 2, lo, hi)
    assert torch.equal(a.flat.param, b.flat.param)
    # the same file restores a sharded engine: its step then matches the replicated one's
    c = ShardedDataParallel(_net(), cfg, stage=2, comm=TorchDistComm(), window=2, grad_slots=2)
    c.load_checkpoint(base)
    _step(c, xs, ys, 2, lo, hi)
    got = c.materialize()
    for n, p in a.module.named_parameters():
        assert torch.allclose(got[n], p.detach(), rtol=0, atol=2e-6), n
    dist.barrier()
    dist.destroy_process_group()


def test_ddp_resume_and_load_into_sharded_engine(tmp_path):
    port = _free_port()
    mp.spawn(_ddp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)


def _weights_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from momijo_b200.learn.utils.checkpoint import load_state_dict
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel
    from momijo_b200.parallel.peer import TorchDistComm

    dist.init_process_group("gloo", rank=rank, world_size=world)
    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    lo, hi = rank * 4, rank * 4 + 4
    base = os.path.join(tmp, "w", "model")
    a = ShardedDataParallel(_net(), cfg, stage=3, comm=TorchDistComm(), window=2, grad_slots=2)
    for s in range(2):
        _step(a, xs, ys, s, lo, hi)
    a.save_weights(base, extra={"tag": "two steps"})
    want = a.materialize()
    # an unsharded model reads the file through the ordinary MNP loader
    plain = _net()
    assert load_state_dict(plain, base)
    for n, p in plain.named_parameters():
        assert torch.equal(p.detach(), want[n]), n
    # another engine (other stage) takes the same weights; its moments start from zero
    torch.manual_seed(123)
    other = _net()
    for p in other.parameters():
        p.data.normal_()
    b = ShardedDataParallel(other, cfg, stage=1, comm=TorchDistComm())
    assert b.load_weights(base)["tag"] == "two steps"
    got = b.materialize()
    for k in want:
        assert torch.equal(got[k], want[k]), k
    assert float(b.m.abs().sum()) == 0.0 and float(b.v.abs().sum()) == 0.0
    _step(b, xs, ys, 2, lo, hi)    # and trains on
    dist.barrier()
    dist.destroy_process_group()


def test_save_weights_is_an_ordinary_checkpoint_and_loads_into_any_engine(tmp_path):
    port = _free_port()
    mp.spawn(_weights_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)


def test_model_checkpoint_callback_writes_engine_weights_and_optimizer_state(tmp_path):
    from momijo_b200.learn.callbacks.model_checkpoint import ModelCheckpoint
    from momijo_b200.parallel import AdamWConfig, ShardedDataParallel

    xs, ys = _data()
    cfg = AdamWConfig(lr=1e-2, weight_decay=0.1)
    a = ShardedDataParallel(_net(), cfg)
    for s in range(2):
        _step(a, xs, ys, s, 0, 8)
    cb = ModelCheckpoint(str(tmp_path / "run"))
    path = cb.save(a, step=2, extra={"epoch": 0})
    assert os.path.exists(path + ".json") and os.path.exists(path + ".optim.bin")
    last = os.path.join(str(tmp_path / "run"), "last.mnp")
    _step(a, xs, ys, 2, 0, 8)
    b = ShardedDataParallel(_net(), cfg)
    b.load_checkpoint(last + ".optim")     # master weights, moments and step: everything a resume needs
    _step(b, xs, ys, 2, 0, 8)
    wa, wb = a.materialize(), b.materialize()
    for k in wa:
        assert torch.equal(wa[k], wb[k]), k
