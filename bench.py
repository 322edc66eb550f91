#!/usr/bin/env python
"""Headline benchmark: GPT-2 small training throughput (tokens/s over all GPUs of one node).

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference|torch]

Model/config: 12 layers, d_model 768, 12 heads, MLP 3072 GELU, pre-LayerNorm, vocab 50257,
learned positions, seq 1024, micro-batch 16 per GPU, bf16 parameters/activations, fp32 AdamW
master state, sharded data parallel (ZeRO-3 style) for N > 1. Synthetic uniform-random tokens,
random-init weights ~N(0, 0.02).

Timing: W untimed warm-up steps, then exactly K steps between CUDA events on the launching
stream, bracketed by a barrier + synchronize; the maximum over ranks is reported. A second
timed region measures the same K steps end to end through the public API, including the
host->device copy of every step's tokens from pinned memory and the device->host read of the
loss. Each step touches the 0.25 GB of bf16 weights plus several GB of activations, far more
than the 126 MB L2, so no explicit L2 flush is needed between iterations.

``--impl reference`` must run the unmodified reference; it is pure Mojo with no build files and
no Mojo toolchain exists in this image, so that arm reports ``unavailable``. ``--impl torch``
runs the same model as stock PyTorch (cuBLAS + SDPA, FSDP for N > 1) for orientation; for
``--config llama8b-tp`` and ``moe16b-ep`` it runs the arms in ``bench_torch.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--model", default="gpt2-small", choices=["gpt2-small", "gpt2-tiny"])
    ap.add_argument("--config", default="gpt2", choices=["gpt2", "llama8b-tp", "moe16b-ep", "llama13b-pptp"],
                    help="gpt2: the headline config (sharded data parallel). The others are the tensor-, "
                         "expert- and pipeline-parallel configs; they need the GPUs named in their docstrings.")
    ap.add_argument("--layers", type=int, default=0,
                    help="override the layer count (for smoke runs; the result is then marked 'reduced')")
    ap.add_argument("--baseline", type=int, default=1,
                    help="1 (default): after the native arm, time the stock-PyTorch arm of the same config in the "
                         "same process group and report value / that as vs_baseline; 0: skip it")
    ap.add_argument("--zero-stage", type=int, default=3, choices=[1, 2, 3],
                    help="sharding stage of the headline config for N > 1")
    ap.add_argument("--fuse-first-gemm", type=int, default=1,
                    help="stages 1-2: gather each block's first weight inside the GEMM that consumes it")
    ap.add_argument("--tp-fuse-min-rows", type=int, default=-1,
                    help="tensor-parallel products with fewer gathered rows run as two launches instead of one "
                         "fused kernel (-1: the library default)")
    ap.add_argument("--torch-variant", default="autocast", choices=["autocast", "bf16-master"],
                    help="stock-PyTorch arm of the headline config: fp32 parameters under bf16 autocast, or bf16 "
                         "parameters with an fp32 master copy")
    return ap.parse_args()


def reference_unavailable():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is 100% Mojo with no setup.py/pyproject (pip: 'not installable') "
                       "and no Mojo toolchain exists in this image; it also has no multi-rank path "
                       "(init_process_group asserts world_size == 1)",
    }))
    return 0


def init_dist(n):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local))
    return rank, world, local


def barrier_sync(world):
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed(fn_step, steps, world):
    """Time exactly `steps` calls of fn_step on the device; max over ranks, in ms per step."""
    import torch
    from momijo_b200.utils import max_over_ranks

    barrier_sync(world)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn_step(i)
    b.record()
    barrier_sync(world)
    return max_over_ranks(a.elapsed_time(b)) / steps


def build_ours(cfg, world, rank, local, stage=3, fuse_first_gemm=True):
    import torch
    from momijo_b200 import ops
    from momijo_b200.models import GPT2
    from momijo_b200.parallel import ShardedDataParallel, AdamWConfig

    torch.manual_seed(1234)
    model = GPT2(cfg).cuda()
    comm = None
    if world > 1:
        from momijo_b200.parallel.peer import PeerComm

        comm = PeerComm.from_default_group()
    engine = ShardedDataParallel(model, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1),
                                 stage=stage, comm=comm, fuse_first_gemm=fuse_first_gemm)
    return engine


def build_torch(cfg, world, local, variant="autocast"):
    """Stock PyTorch arm: same architecture with nn.Linear / SDPA / F.cross_entropy. Returns
    ``(net, opt, finish)``; ``finish()`` runs the optimizer step (and zeroes the gradients).

    ``variant``: "autocast" keeps fp32 parameters and runs the forward under bf16 autocast (the usual
    single-GPU recipe; weights are re-cast every step); "bf16-master" keeps bf16 parameters and applies
    AdamW to an fp32 master copy (the same precision recipe as the native arm). With N > 1 both are FSDP
    full-shard with ``MixedPrecision(param_dtype=bf16)`` over fp32 shards, one FSDP unit per block."""
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(s):
            super().__init__()
            c, f = cfg.d_model, cfg.d_ff
            s.ln1, s.ln2 = nn.LayerNorm(c), nn.LayerNorm(c)
            s.qkv, s.o = nn.Linear(c, 3 * c), nn.Linear(c, c)
            s.fc, s.proj = nn.Linear(c, f), nn.Linear(f, c)

        def forward(s, x):
            B, T, C = x.shape
            q, k, v = s.qkv(s.ln1(x)).view(B, T, 3, cfg.n_head, C // cfg.n_head).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + s.o(a.transpose(1, 2).reshape(B, T, C))
            return x + s.proj(F.gelu(s.fc(s.ln2(x)), approximate="tanh"))

    class Net(nn.Module):
        def __init__(s):
            super().__init__()
            s.wte = nn.Embedding(cfg.padded_vocab, cfg.d_model)
            s.wpe = nn.Embedding(cfg.max_seq, cfg.d_model)
            s.blocks = nn.ModuleList([Block() for _ in range(cfg.n_layer)])
            s.lnf = nn.LayerNorm(cfg.d_model)

        def forward(s, tok, tgt):
            B, T = tok.shape
            x = s.wte(tok) + s.wpe(torch.arange(T, device=tok.device))
            for b in s.blocks:
                x = b(x)
            logits = F.linear(s.lnf(x), s.wte.weight)[..., :cfg.vocab_size]
            return F.cross_entropy(logits.float().reshape(-1, cfg.vocab_size), tgt.reshape(-1))

    torch.manual_seed(1234)
    net = Net().cuda()
    for p in net.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, 0.0, 0.02)
    if world > 1:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, MixedPrecision
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy

        net = FSDP(net, mixed_precision=MixedPrecision(param_dtype=torch.bfloat16,
                                                       reduce_dtype=torch.bfloat16),
                   auto_wrap_policy=ModuleWrapPolicy({Block}), use_orig_params=True, device_id=local)
    elif variant == "bf16-master":
        net = net.to(torch.bfloat16)
        params = [p for p in net.parameters()]
        masters = [p.detach().float().clone().requires_grad_(True) for p in params]
        opt = torch.optim.AdamW(masters, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

        def finish():
            for m, p in zip(masters, params):
                m.grad = p.grad.float()
            opt.step()
            with torch.no_grad():
                torch._foreach_copy_(params, masters)
            for p in params:
                p.grad = None

        return net, opt, finish
    opt = torch.optim.AdamW(net.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                            fused=True)

    def finish():
        opt.step()
        opt.zero_grad(set_to_none=True)

    return net, opt, finish


def _pinned_batches(vocab, shape, seed, n=4):
    import torch

    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, shape, generator=g).pin_memory() for _ in range(n)]


def setup_llama_tp(args, rank, world, local):
    """Llama-3-8B shape (32L, d4096, 32q/8kv heads of 128, SwiGLU 14336, vocab 128256), seq 4096, global
    batch 8 sequences, tensor parallel over all ranks with sequence parallelism; every rank feeds the same
    tokens. Fused all-gather->GEMM and GEMM->reduce-scatter kernels over peer memory; AdamW (fp32 master)
    on each rank's own weight shards."""
    import torch
    from momijo_b200 import ops
    from momijo_b200.models import Llama, LlamaConfig
    from momijo_b200.parallel import AdamWConfig, HybridEngine
    from momijo_b200.parallel.tp import TPContext

    cfg = LlamaConfig.llama3_8b()
    if args.layers:
        cfg.n_layer = args.layers
    B, T = 8, cfg.max_seq
    comm = None
    if world > 1:
        from momijo_b200.parallel.peer import PeerComm

        comm = PeerComm.from_default_group(heap_bytes=12 << 30)
    tp = TPContext(comm=comm) if comm is not None else TPContext.single()
    if args.tp_fuse_min_rows >= 0:
        tp.fuse_min_rows = args.tp_fuse_min_rows
    torch.manual_seed(1234 + rank)
    with torch.device("cuda"):
        model = Llama(cfg, tp)
    engine = HybridEngine(model, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1), rep_comm=comm)
    host_tok = _pinned_batches(cfg.vocab_size, (B, T + 1), 1000)   # same seed on every rank: same tokens
    dev_tok = [t.cuda() for t in host_tok]

    def step_device(i):
        t = dev_tok[i % len(dev_tok)]
        loss = engine(t[:, :-1], t[:, 1:])
        loss.backward()
        engine.step()
        return loss

    def step_e2e(i):
        t = host_tok[i % len(host_tok)].cuda(non_blocking=True)
        loss = engine(t[:, :-1], t[:, 1:])
        loss.backward()
        engine.step()
        return float(loss)

    info = {"tokens_per_step": B * T, "scaling": "strong", "flops_per_token": cfg.flops_per_token(T),
            "h2d_bytes": B * (T + 1) * 8,
            "config": {"model": f"llama-3-8b shape ({cfg.n_layer}L d4096 32q/8kv hd128 ff14336 vocab128256 seq4096)",
                       "global_batch": B, "seq_len": T, "parallelism": f"tp{world}+sp",
                       "optimizer": "AdamW fp32 master on local shards, step inside the timed region",
                       "l2": "working set of tens of GB per step >> 126 MB L2; no flush"}}
    return step_device, step_e2e, info


def setup_moe_ep(args, rank, world, local):
    """16B-class MoE (28L, d2048, 16 heads, 64 routed experts of FFN 1408 + 2 shared, top-6, aux 0.01, vocab
    102400), seq 4096, micro-batch 4 per GPU: experts split over all ranks (fused dispatch / grouped GEMM /
    combine over peer memory), attention and the other dense parameters data parallel with the fused
    reduce-scatter + sharded AdamW."""
    import torch
    from momijo_b200 import ops
    from momijo_b200.models import MoEConfig, MoEDecoder
    from momijo_b200.parallel import AdamWConfig, HybridEngine

    cfg = MoEConfig.moe_16b()
    if args.layers:
        cfg.n_layer = args.layers
    B, T = 4, cfg.max_seq
    comm = None
    if world > 1:
        from momijo_b200.parallel.peer import PeerComm

        comm = PeerComm.from_default_group(heap_bytes=16 << 30)
    torch.manual_seed(1234 + rank)
    with torch.device("cuda"):
        model = MoEDecoder(cfg, comm, max_tokens=B * T, capacity_factor=2.0)
    experts = {id(p) for p in model.expert_parameters()}
    dense = [p for p in model.parameters() if id(p) not in experts]
    if world > 1:
        # dense parameters start identical on every rank
        import torch.distributed as dist
        for p in dense:
            dist.broadcast(p.data, 0)
    engine = HybridEngine(model, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1),
                          dp_comm=comm, dp_params=dense if world > 1 else None,
                          local_grad_scale=1.0 / world)
    host_tok = _pinned_batches(cfg.vocab_size, (B, T + 1), 1000 + rank)
    dev_tok = [t.cuda() for t in host_tok]

    def step_device(i):
        t = dev_tok[i % len(dev_tok)]
        loss = engine(t[:, :-1], t[:, 1:])
        loss.backward()
        engine.step()
        return loss

    def step_e2e(i):
        t = host_tok[i % len(host_tok)].cuda(non_blocking=True)
        loss = engine(t[:, :-1], t[:, 1:])
        loss.backward()
        engine.step()
        return float(loss)

    info = {"tokens_per_step": B * T * world, "scaling": "weak", "flops_per_token": cfg.flops_per_token(T),
            "h2d_bytes": B * (T + 1) * 8,
            "config": {"model": f"moe-16b shape ({cfg.n_layer}L d2048 16H 64 experts ff1408 top6 + 2 shared vocab102400 seq4096)",
                       "global_batch": B * world, "seq_len": T, "parallelism": f"ep{world}+dp{world}-attention",
                       "optimizer": "AdamW fp32 master (experts local, dense sharded), step inside the timed region",
                       "l2": "working set of tens of GB per step >> 126 MB L2; no flush"}}
    return step_device, step_e2e, info


def setup_llama_pptp(args, rank, world, local):
    """Llama-2-13B shape (40L, d5120, 40 heads, SwiGLU 13824, vocab 32000): 2 pipeline stages x 4-way tensor
    parallel on 8 GPUs, 1F1B over 16 micro-batches of 1 x 4096 tokens; activations between stages go over
    NCCL p2p, tensor parallelism uses the fused kernels inside each stage."""
    import torch
    import torch.distributed as dist
    from momijo_b200 import ops
    from momijo_b200.models import LlamaConfig
    from momijo_b200.models.llama import LlamaStage
    from momijo_b200.parallel import AdamWConfig, HybridEngine
    from momijo_b200.parallel.peer import PeerComm
    from momijo_b200.parallel.pp import PipelineStage, Schedule1F1B, partition_layers
    from momijo_b200.parallel.tp import TPContext

    if world % 2:
        raise SystemExit("--config llama13b-pptp needs an even number of GPUs (2 pipeline stages)")
    cfg = LlamaConfig.llama2_13b()
    if args.layers:
        cfg.n_layer = args.layers
    S, TP = 2, world // 2
    n_micro, T = 16, cfg.max_seq
    stage_id, tp_rank = rank // TP, rank % TP
    groups = [dist.new_group(list(range(s * TP, (s + 1) * TP))) for s in range(S)]
    comm = PeerComm(groups[stage_id], heap_bytes=6 << 30) if TP > 1 else None
    tp = TPContext(comm=comm) if comm is not None else TPContext.single()
    if args.tp_fuse_min_rows >= 0:
        tp.fuse_min_rows = args.tp_fuse_min_rows
    layers = partition_layers(cfg.n_layer, S)[stage_id]
    torch.manual_seed(1234 + rank)
    with torch.device("cuda"):
        module = LlamaStage(cfg, tp, layers, first=stage_id == 0, last=stage_id == S - 1)
    module.batch_shape = (1, T)
    # 16 micro-batch gradients are summed before one update: accumulate them in fp32
    engine = HybridEngine(module, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1), rep_comm=comm,
                          local_grad_dtype=torch.float32)
    stage = PipelineStage(module, stage_id, S, prev_rank=rank - TP if stage_id > 0 else None,
                          next_rank=rank + TP if stage_id < S - 1 else None)
    sched = Schedule1F1B(stage, n_micro, (T // TP, cfg.d_model), torch.bfloat16, torch.device("cuda", local))
    host_tok = _pinned_batches(cfg.vocab_size, (n_micro, T + 1), 1000)  # same tokens on every rank
    dev_tok = [t.cuda() for t in host_tok]

    def run(t):
        inputs = [t[m:m + 1, :-1] for m in range(n_micro)]
        targets = [t[m:m + 1, 1:] for m in range(n_micro)]
        loss = sched.run(inputs if stage.is_first else None, module.loss if stage.is_last else None,
                         targets if stage.is_last else None)
        engine.step()
        return loss

    def step_device(i):
        return run(dev_tok[i % len(dev_tok)])

    def step_e2e(i):
        loss = run(host_tok[i % len(host_tok)].cuda(non_blocking=True))
        return float(loss) if loss is not None else None

    info = {"tokens_per_step": n_micro * T, "scaling": "strong", "flops_per_token": cfg.flops_per_token(T),
            "h2d_bytes": n_micro * (T + 1) * 8,
            "config": {"model": f"llama-2-13b shape ({cfg.n_layer}L d5120 40H ff13824 vocab32000 seq4096)",
                       "global_batch": n_micro, "seq_len": T, "parallelism": f"pp2 x tp{TP}, 1F1B, {n_micro} micro-batches",
                       "optimizer": "AdamW fp32 master on local shards, fp32 gradient accumulation over the micro-batches, "
                                    "step inside the timed region",
                       "l2": "working set of tens of GB per step >> 126 MB L2; no flush"}}
    return step_device, step_e2e, info


def setup_torch_arm(args, rank, world, local):
    """Stock-PyTorch arm of the tensor- and expert-parallel configs (``bench_torch.py``): same shapes, batch
    sizes and token streams as the native setups, NCCL collectives, cuBLAS, SDPA, fused AdamW on fp32
    parameters under bf16 autocast."""
    import torch
    import torch.distributed as dist
    from bench_torch import TorchLlamaTP, TorchMoEEP, make_step
    from momijo_b200.models import LlamaConfig, MoEConfig

    tp = args.config == "llama8b-tp"
    cfg = LlamaConfig.llama3_8b() if tp else MoEConfig.moe_16b()
    if args.layers:
        cfg.n_layer = args.layers
    B, T = (8, cfg.max_seq) if tp else (4, cfg.max_seq)
    torch.manual_seed(1234 + rank)
    with torch.device("cuda"):
        model = TorchLlamaTP(cfg) if tp else TorchMoEEP(cfg)
    if not tp and world > 1:
        for p in model.dense_params:
            dist.broadcast(p.data, 0)
    step = make_step(model, "tp" if tp else "ep", "cuda")
    host_tok = _pinned_batches(cfg.vocab_size, (B, T + 1), 1000 if tp else 1000 + rank)
    dev_tok = [t.cuda() for t in host_tok]

    def step_device(i):
        return step(dev_tok[i % len(dev_tok)])

    def step_e2e(i):
        return float(step(host_tok[i % len(host_tok)].cuda(non_blocking=True)))

    name = (f"llama-3-8b shape ({cfg.n_layer}L d4096 32q/8kv hd128 ff14336 vocab128256 seq4096)" if tp else
            f"moe-16b shape ({cfg.n_layer}L d2048 16H 64 experts ff1408 top6 + 2 shared vocab102400 seq4096)")
    info = {"tokens_per_step": B * T * (1 if tp else world), "scaling": "strong" if tp else "weak",
            "flops_per_token": cfg.flops_per_token(T), "h2d_bytes": B * (T + 1) * 8,
            "config": {"model": name, "global_batch": B * (1 if tp else world), "seq_len": T,
                       "parallelism": (f"tp{world}+sp" if tp else f"ep{world}+dp{world}-attention") + " (torch.distributed, cuBLAS, SDPA)",
                       "optimizer": "torch.optim.AdamW(fused) on fp32 parameters, bf16 autocast, step inside the timed region",
                       "l2": "working set of tens of GB per step >> 126 MB L2; no flush"}}
    return step_device, step_e2e, info


def setup_torch_pptp(args, rank, world, local):
    """Stock-PyTorch arm of the pipeline x tensor parallel config: the same 2 x (N/2) layout, Megatron-style
    tensor parallel stages (``bench_torch.TorchLlamaTP``), 1F1B over NCCL p2p, fused AdamW on fp32 parameters
    under bf16 autocast."""
    import torch
    import torch.distributed as dist
    from bench_torch import TorchLlamaTP, run_1f1b
    from momijo_b200.models import LlamaConfig
    from momijo_b200.parallel.pp import partition_layers

    if world % 2:
        raise SystemExit("--config llama13b-pptp needs an even number of GPUs (2 pipeline stages)")
    cfg = LlamaConfig.llama2_13b()
    if args.layers:
        cfg.n_layer = args.layers
    S, TP = 2, world // 2
    n_micro, T = 16, cfg.max_seq
    stage_id = rank // TP
    groups = [dist.new_group(list(range(s * TP, (s + 1) * TP))) for s in range(S)]
    layers = partition_layers(cfg.n_layer, S)[stage_id]
    torch.manual_seed(1234 + rank)
    with torch.device("cuda"):
        stage = TorchLlamaTP(cfg, groups[stage_id], layers=layers, first=stage_id == 0, last=stage_id == S - 1)
    stage.batch_shape = (1, T)
    opt = torch.optim.AdamW(stage.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    host_tok = _pinned_batches(cfg.vocab_size, (n_micro, T + 1), 1000)
    dev_tok = [t.cuda() for t in host_tok]
    dev = torch.device("cuda", local)

    def run(t):
        inputs = [t[m:m + 1, :-1] for m in range(n_micro)]
        targets = [t[m:m + 1, 1:] for m in range(n_micro)]
        loss = run_1f1b(stage, stage_id, S, rank - TP if stage_id > 0 else None,
                        rank + TP if stage_id < S - 1 else None, n_micro, (T // TP, cfg.d_model), dev,
                        inputs, targets)
        stage.sync_replicated_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step_device(i):
        return run(dev_tok[i % len(dev_tok)])

    def step_e2e(i):
        loss = run(host_tok[i % len(host_tok)].cuda(non_blocking=True))
        return float(loss) if loss is not None else None

    info = {"tokens_per_step": n_micro * T, "scaling": "strong", "flops_per_token": cfg.flops_per_token(T),
            "h2d_bytes": n_micro * (T + 1) * 8,
            "config": {"model": f"llama-2-13b shape ({cfg.n_layer}L d5120 40H ff13824 vocab32000 seq4096)",
                       "global_batch": n_micro, "seq_len": T,
                       "parallelism": f"pp2 x tp{TP}, 1F1B, {n_micro} micro-batches (torch.distributed, cuBLAS, SDPA)",
                       "optimizer": "torch.optim.AdamW(fused) on fp32 parameters, bf16 autocast, step inside the timed region",
                       "l2": "working set of tens of GB per step >> 126 MB L2; no flush"}}
    return step_device, step_e2e, info


def setup_gpt2(args, rank, world, local, impl):
    """Headline config: GPT-2 small, micro-batch 16 x 1024 per GPU, sharded data parallel for N > 1."""
    import torch
    from momijo_b200.models import GPT2Config

    cfg = GPT2Config.small() if args.model == "gpt2-small" else GPT2Config.tiny()
    B, T = args.micro_batch, min(args.seq, cfg.max_seq)
    tokens_per_step = B * T * world

    # synthetic data: uniform random token ids, staged in pinned host memory
    g = torch.Generator().manual_seed(1000 + rank)
    n_batches = 4
    host_tok = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).pin_memory()
                for _ in range(n_batches)]
    dev_tok = [t.cuda() for t in host_tok]
    extra = {}

    if impl == "ours":
        engine = build_ours(cfg, world, rank, local, stage=args.zero_stage, fuse_first_gemm=bool(args.fuse_first_gemm))

        def step_device(i):
            t = dev_tok[i % n_batches]
            loss = engine(t[:, :-1], t[:, 1:])
            loss.backward()
            engine.step()
            return loss

        from momijo_b200.learn.engine.lm import train_step_e2e

        def step_e2e(i):
            return train_step_e2e(engine, host_tok[i % n_batches])

        par = "single" if world == 1 else f"zero{args.zero_stage}-dp{world}"
        optim = "AdamW fp32 master, step inside the timed region"
        if world > 1:
            extra["memory"] = engine.memory_report()
    else:
        variant = args.torch_variant
        net, opt, finish = build_torch(cfg, world, local, variant)

        def torch_step(t):
            if variant == "bf16-master" and world == 1:
                loss = net(t[:, :-1], t[:, 1:])
            else:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = net(t[:, :-1], t[:, 1:])
            loss.backward()
            finish()
            return loss

        def step_device(i):
            return torch_step(dev_tok[i % n_batches])

        def step_e2e(i):
            return float(torch_step(host_tok[i % n_batches].cuda(non_blocking=True)))

        par = ("single" if world == 1 else f"fsdp-full-shard-dp{world}") + " (stock PyTorch: cuBLAS, SDPA, NCCL)"
        optim = ("torch.optim.AdamW(fused) on fp32 parameters, bf16 autocast" if variant == "autocast" or world > 1
                 else "bf16 parameters, torch.optim.AdamW(fused) on an fp32 master copy") + ", step inside the timed region"

    info = {
        "tokens_per_step": tokens_per_step,
        "scaling": "weak",
        "flops_per_token": cfg.flops_per_token(T),
        "h2d_bytes": B * (T + 1) * 8,
        "config": {
            "model": "gpt2-small (12L d768 12H ff3072 vocab50257 seq1024)" if args.model == "gpt2-small" else args.model,
            "global_batch": B * world,
            "seq_len": T,
            "parallelism": par,
            "optimizer": optim,
            "l2": "per-step working set (0.25 GB weights + GBs of activations) >> 126 MB L2; no flush",
        },
        "extra": extra,
    }
    return step_device, step_e2e, info


def run_arm(args, impl, rank, world, local):
    """Build one arm (native or stock PyTorch) of the selected config, time it, free it. Returns the
    result dict on rank 0 (None elsewhere, or when the arm does not exist)."""
    import gc

    import torch

    if args.config == "gpt2":
        setup = lambda: setup_gpt2(args, rank, world, local, impl)
    elif impl == "torch":
        if args.config == "llama13b-pptp":
            setup = lambda: setup_torch_pptp(args, rank, world, local)
        else:
            setup = lambda: setup_torch_arm(args, rank, world, local)
    else:
        fn = {"llama8b-tp": setup_llama_tp, "moe16b-ep": setup_moe_ep, "llama13b-pptp": setup_llama_pptp}[args.config]
        setup = lambda: fn(args, rank, world, local)
    step_device, step_e2e, info = setup()
    out = time_arm(args, impl, rank, world, local, step_device, step_e2e, info)
    del step_device, step_e2e, info, setup
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return reference_unavailable()
    if os.environ.get("MOMIJO_DUMP_STACKS_AFTER"):
        # debugging aid for a run that stops making progress: print every thread's Python stack after N seconds
        import faulthandler

        faulthandler.dump_traceback_later(float(os.environ["MOMIJO_DUMP_STACKS_AFTER"]), repeat=False)

    rank, world, local = init_dist(args.gpus)
    out = run_arm(args, args.impl, rank, world, local)
    if args.impl == "ours" and args.baseline:
        # The reference has no buildable multi-GPU (or GPU) path, so the baseline named for this benchmark is
        # the same model and config in stock PyTorch (cuBLAS, SDPA, NCCL: FSDP / tensor / expert / pipeline
        # parallel), timed here with the same steps, warm-up, data and clocks, right after the native arm.
        try:
            base = run_arm(args, "torch", rank, world, local)
        except Exception as e:  # the comparison must never cost the native number
            base = {"error": f"{type(e).__name__}: {e}"[:300]} if rank == 0 else None
        if rank == 0 and out is not None and base is not None:
            if "value" in base:
                out["vs_baseline"] = out["value"] / base["value"]
                out["baseline"] = {"impl": base["config"]["parallelism"], "value": base["value"],
                                   "ms_per_step": base["ms_per_step"], "e2e": base["e2e"]["value"],
                                   "e2e_ratio": out["e2e"]["value"] / base["e2e"]["value"],
                                   "optimizer": base["config"]["optimizer"], "clocks": base["clocks"],
                                   "loss_after_timed_steps": base["loss_after_timed_steps"]}
            else:
                out["baseline"] = base
    if rank == 0 and out is not None:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


def time_arm(args, impl, rank, world, local, step_device, step_e2e, info):
    import torch
    from momijo_b200 import _C
    from momijo_b200.utils import ClockSampler

    for i in range(max(args.warmup, 3)):
        step_device(i)
    torch.cuda.synchronize()

    sampler = ClockSampler(local).start() if rank == 0 else None
    launches0 = _C.launches
    last = []
    def counted(i):
        r = step_device(i)
        if i == args.steps - 1:
            last.append(r)
    ms = timed(counted, args.steps, world)
    launches = _C.launches - launches0
    ms_e2e = timed(step_e2e, args.steps, world)
    clocks = sampler.stop() if sampler is not None else None
    loss_val = float(last[0].detach()) if last and last[0] is not None else None
    if impl == "ours":
        _C.check_status()
    if rank != 0:
        return None
    tokens_per_step = info["tokens_per_step"]
    tok_s = tokens_per_step / (ms / 1e3)
    tok_s_e2e = tokens_per_step / (ms_e2e / 1e3)
    out = {
        "metric": "train tokens/s/box (device-timed, max over ranks)",
        "value": tok_s,
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": info["scaling"],
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init weights N(0,0.02)",
        "impl": impl,
        "config": info["config"],
        "e2e": {
            "value": tok_s_e2e,
            "unit": "tokens/s",
            "ms_per_step": ms_e2e,
            "h2d_bytes_per_step": info["h2d_bytes"],
            "d2h_bytes_per_step": 4,
        },
        "gpu_launches": launches if impl == "ours" else 0,
        "clocks": clocks,
        "loss_after_timed_steps": loss_val,
        "model_tflops": info["flops_per_token"] * tok_s / 1e12,
    }
    out.update(info.get("extra", {}))
    if args.layers:
        out["reduced"] = f"layer count overridden to {args.layers}: not a result for the named model"
    return out


if __name__ == "__main__":
    sys.exit(main())
