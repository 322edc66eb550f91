"""Checkpoint and resume of the sharded engine: optimizer state per rank in the MNP layout (readable by a run
with another number of ranks), full weights as one ordinary MNP checkpoint.

    python examples/parallel/checkpoint_resume.py                         # one process, tiny GPT-2 on CPU or GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29500 examples/parallel/checkpoint_resume.py        # the same with two ranks
"""
import os
import tempfile

import torch
import torch.distributed as dist

from momijo_b200.models import GPT2, GPT2Config
from momijo_b200.parallel import AdamWConfig, ShardedDataParallel


def _engine(comm, cuda):
    torch.manual_seed(0)
    model = GPT2(GPT2Config.tiny())
    if cuda:
        model = model.cuda()
    return ShardedDataParallel(model, AdamWConfig(lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1), comm=comm,
                               overlap=cuda)


def main(argv=None):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    comm = None
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        from momijo_b200.parallel.peer import PeerComm, TorchDistComm
        comm = PeerComm.from_default_group() if cuda else TorchDistComm()
    cfg = GPT2Config.tiny()
    g = torch.Generator().manual_seed(100 + rank)
    batches = [torch.randint(0, cfg.vocab_size, (2, 65), generator=g) for _ in range(3)]
    batches = [b.cuda() for b in batches] if cuda else batches

    def step(engine, tok):
        loss = engine(tok[:, :-1], tok[:, 1:])
        loss.backward()
        engine.step()
        return loss.item()

    folder = tempfile.mkdtemp(prefix="momijo_ckpt_") if rank == 0 else None
    if world > 1:
        box = [folder]
        dist.broadcast_object_list(box, src=0)
        folder = box[0]
    a = _engine(comm, cuda)
    losses = [step(a, batches[0]), step(a, batches[1])]
    a.save_checkpoint(os.path.join(folder, "optimizer"), extra={"next_batch": 2})
    a.save_weights(os.path.join(folder, "weights"))
    uninterrupted = step(a, batches[2])

    b = _engine(comm, cuda)                     # a fresh process would do exactly this
    extra = b.load_checkpoint(os.path.join(folder, "optimizer"))
    resumed = step(b, batches[extra["next_batch"]])
    if rank == 0:
        print(f"losses before the checkpoint: {losses[0]:.4f} {losses[1]:.4f}")
        print(f"third step, uninterrupted: {uninterrupted:.6f}   after resume: {resumed:.6f}")
        print("files:", sorted(os.listdir(folder)))
    assert abs(uninterrupted - resumed) < 1e-6 * max(1.0, abs(uninterrupted)), (uninterrupted, resumed)
    if world > 1:
        dist.destroy_process_group()
    return {"losses": losses, "uninterrupted": uninterrupted, "resumed": resumed}


if __name__ == "__main__":
    main()
