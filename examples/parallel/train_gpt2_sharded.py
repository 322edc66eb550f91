"""GPT-2 training through the sharded data-parallel engine. One process per GPU:

    python examples/parallel/train_gpt2_sharded.py                       # one GPU (or CPU, tiny model)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 examples/parallel/train_gpt2_sharded.py --model small

With more than one rank the gradient reduce-scatter, the AdamW update of the local shard and the
parameter all-gather run as this library's peer-memory kernels."""
import argparse
import os

import torch
import torch.distributed as dist

from momijo_b200.models import GPT2, GPT2Config
from momijo_b200.parallel import AdamWConfig, ShardedDataParallel


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny", choices=["tiny", "small"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=2)
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    comm = None
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        if cuda:
            from momijo_b200.parallel.peer import PeerComm
            comm = PeerComm.from_default_group()
        else:
            from momijo_b200.parallel.peer import TorchDistComm
            comm = TorchDistComm()
    cfg = GPT2Config.small() if args.model == "small" else GPT2Config.tiny()
    torch.manual_seed(0)
    model = GPT2(cfg)
    if cuda:
        model = model.cuda()
    engine = ShardedDataParallel(model, AdamWConfig(lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1), comm=comm,
                                 overlap=cuda)
    g = torch.Generator().manual_seed(100 + rank)
    T = min(cfg.max_seq, 128)
    losses = []
    for step in range(args.steps):
        tok = torch.randint(0, cfg.vocab_size, (args.batch, T + 1), generator=g)
        tok = tok.cuda() if cuda else tok
        loss = engine(tok[:, :-1], tok[:, 1:])
        loss.backward()
        engine.step()
        losses.append(loss.item())
        if rank == 0:
            print(f"step {step} loss {losses[-1]:.4f}")
    if world > 1:
        dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
