"""Microbenchmarks of the fused compute + collective kernels, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29650 -m momijo_b200.ops.bench_comm [--small]

Every number is timed on the device with CUDA events after warm-up, with a host barrier before the
timed loop, and the maximum over ranks is reported. Each row carries its roofline: the slower of
(FLOPs / measured GEMM peak) and (bytes that must cross NVLink per GPU / 770 GB/s measured peer-copy
bandwidth; for the HBM-bound optimizer step also bytes / measured copy bandwidth), and the achieved
fraction target / measured. NCCL (+ a plain local GEMM where one follows) is timed beside each as the
unfused baseline.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import _C, ops
from ..utils.timing import max_over_ranks
from .bench_kernels import peaks

bf16 = torch.bfloat16
LINK = 770e9


def timed(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return max_over_ranks(a.elapsed_time(b)) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--tp-shape", default="",
                    help="rows,hidden,ffn of the tensor-parallel section (default: the Llama-8B MLP at 32768 rows), "
                         "e.g. 4096,5120,13824 for one 4096-token micro-batch of the Llama-13B shape")
    ap.add_argument("--only", default="all_reduce,zero,tp,moe",
                    help="comma list of sections: all_reduce, zero, tp (all-gather->GEMM, GEMM->reduce-scatter), moe")
    args = ap.parse_args()
    only = set(args.only.split(","))
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from ..ops.fused_comm import FusedSite, allgather_gemm, gemm_reduce_scatter
    from ..parallel.ep import MoEDispatcher
    from ..parallel.peer import PeerComm
    from ..parallel.zero import AdamWConfig, ShardedDataParallel

    comm = PeerComm.from_default_group(heap_bytes=(2 << 30) if args.small else (12 << 30))
    W, R = world, rank
    flops_peak, hbm, tag = peaks()
    rows = []

    def emit(**kw):
        rows.append(kw)
        if rank == 0:
            print(json.dumps(kw), flush=True)

    frac = (W - 1) / W
    # ---- all-reduce (two-shot, peer loads) ----
    for mb in ([] if "all_reduce" not in only else [16] if args.small else [64, 512]):
        n = mb * (1 << 20) // 2
        t = comm.alloc(n, bf16)
        t.fill_(1.0)
        ms = timed(lambda: comm.all_reduce_(t, scale=1.0 / W))
        x = torch.ones(n, dtype=bf16, device="cuda")
        ms_nccl = timed(lambda: dist.all_reduce(x))
        link_bytes = 2 * frac * n * 2
        emit(op="all_reduce_bf16", MB=mb, world=W, ms=ms, busbw_GBs=link_bytes / ms / 1e6,
             roofline_ms=link_bytes / LINK * 1e3, frac_of_roofline=link_bytes / LINK * 1e3 / ms, nccl_ms=ms_nccl)

    # ---- ZeRO step: reduce-scatter + AdamW in one kernel, then parameter all-gather ----
    for n_param in ([] if "zero" not in only else [8 << 20] if args.small else [130023424, 1 << 30]):
        class Box(torch.nn.Module):
            def __init__(s):
                super().__init__()
                s.w = torch.nn.Parameter(torch.zeros(n_param, dtype=bf16, device="cuda"))
        sdp = ShardedDataParallel(Box(), AdamWConfig(lr=1e-4), stage=1, comm=comm)
        sdp.grad_buf.fill_(0.01)
        b0 = sdp.buckets[0]

        def zstep():
            comm.rs_adamw_bucket(sdp, b0, 1e-4, 1)
            comm.gather_bucket(sdp, b0, compact=False)
        ms = timed(zstep)
        ms_rs = timed(lambda: comm.rs_adamw_bucket(sdp, b0, 1e-4, 1))
        N = sdp.total
        link_bytes = 2 * frac * N * 2              # RS pulls + AG pulls, per GPU
        hbm_bytes = N * 2 + (N // W) * (2 + 12 * 2 + 2) + N * 2   # read grads, update shard, write gathered params
        roof = max(link_bytes / LINK, hbm_bytes / hbm) * 1e3
        g = torch.full((N,), 0.01, dtype=bf16, device="cuda")
        gs = torch.empty(N // W, dtype=bf16, device="cuda")
        pfull = torch.empty(N, dtype=bf16, device="cuda")
        master = torch.zeros(N // W, device="cuda")
        m1, v1 = torch.zeros_like(master), torch.zeros_like(master)

        def nccl_step():
            dist.reduce_scatter_tensor(gs, g)
            ops.adamw_flat(gs, master, m1, v1, gs, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0,
                           step=1, grad_scale=1.0 / W)
            dist.all_gather_into_tensor(pfull, gs)
        ms_nccl = timed(nccl_step)
        emit(op="zero_step(rs+adamw | allgather)", params=N, world=W, ms=ms, rs_adamw_ms=ms_rs, roofline_ms=roof,
             frac_of_roofline=roof / ms, nccl_rs_adamw_ag_ms=ms_nccl)
        del sdp, g, gs, pfull, master, m1, v1

    if "tp" in only:
        # ---- all-gather -> GEMM and GEMM -> reduce-scatter (Llama-8B MLP shapes at this world size) ----
        M = 2048 * W if args.small else 32768
        C = 1024 if args.small else 4096
        Fl = (4096 if args.small else 14336) // W
        if args.tp_shape:
            M, C, Fl = (int(v) for v in args.tp_shape.split(","))
            Fl //= W
        site = FusedSite(comm)
        xa = comm.alloc(M * C, bf16).view(M, C)
        xa.normal_()
        w_gu = (torch.randn(2 * Fl, C, device="cuda") * 0.02).to(bf16)
        out = torch.empty(M, 2 * Fl, dtype=bf16, device="cuda")
        ms = timed(lambda: allgather_gemm(site, xa, w_gu, gather_a=True, out=out))
        fl = 2.0 * M * 2 * Fl * C
        link_bytes = frac * M * C * 2
        roof = max(fl / flops_peak, link_bytes / LINK) * 1e3
        ms_gemm = timed(lambda: ops.gemm(xa, w_gu, out=out))
        xs = xa[R * (M // W):(R + 1) * (M // W)].clone()
        xfull = torch.empty(M, C, dtype=bf16, device="cuda")

        def nccl_ag_gemm():
            dist.all_gather_into_tensor(xfull, xs)
            torch.matmul(xfull, w_gu.t(), out=out)
        ms_nccl = timed(nccl_ag_gemm)

        # the same product from two launches: peer-pull all-gather kernel, then the plain GEMM at full width
        def peer_ag_then_gemm():
            comm.all_gather_rows(xa)
            ops.gemm(xa, w_gu, out=out)
        ms_two = timed(peer_ag_then_gemm)
        by_ctas = {str(n): timed(lambda n=n: allgather_gemm(site, xa, w_gu, gather_a=True, out=out, comm_ctas=n))
                   for n in (4, 16)}
        emit(op="allgather->gemm", M=M, N=2 * Fl, K=C, world=W, ms=ms, tflops=fl / ms / 1e9, roofline_ms=roof,
             frac_of_roofline=roof / ms, local_gemm_only_ms=ms_gemm, nccl_allgather_plus_cublas_ms=ms_nccl,
             peer_allgather_then_gemm_ms=ms_two, fused_ms_by_comm_ctas=by_ctas)

        site2 = FusedSite(comm)
        a = (torch.randn(M, Fl, device="cuda")).to(bf16)
        w_down = (torch.randn(C, Fl, device="cuda") * 0.02).to(bf16)
        stage = comm.alloc(M * C, bf16)
        o = torch.empty(M // W, C, dtype=bf16, device="cuda")
        ms = timed(lambda: gemm_reduce_scatter(site2, a, w_down, stage, o))
        fl = 2.0 * M * C * Fl
        roof = max(fl / flops_peak, link_bytes / LINK) * 1e3
        full = torch.empty(M, C, dtype=bf16, device="cuda")

        def nccl_gemm_rs():
            torch.matmul(a, w_down.t(), out=full)
            dist.reduce_scatter_tensor(o, full)
        ms_nccl = timed(nccl_gemm_rs)
        ms_gemm2 = timed(lambda: ops.gemm(a, w_down, out=full))
        # the same result from two launches: plain GEMM into a symmetric buffer, then the pull reduce-scatter kernel
        from .fused_comm import gemm_reduce_scatter_pull
        site3 = FusedSite(comm)
        partial = comm.alloc(M * C, bf16).view(M, C)
        ms_pull = timed(lambda: gemm_reduce_scatter_pull(site3, a, w_down, partial, o))
        emit(op="gemm->reduce_scatter", M=M, N=C, K=Fl, world=W, ms=ms, tflops=fl / ms / 1e9, roofline_ms=roof,
             frac_of_roofline=roof / ms, cublas_plus_nccl_reduce_scatter_ms=ms_nccl, local_gemm_only_ms=ms_gemm2,
             gemm_then_pull_reduce_scatter_ms=ms_pull)

    # ---- MoE dispatch / combine at the 16B shape (top-6 of 64 experts, hidden 2048, 16384 tokens per rank) ----
    n_tok, H, E, k = (2048, 1024, 8 * W, 2) if args.small else (16384, 2048, 64, 6)
    if E % W == 0 and "moe" in only:
        torch.manual_seed(50 + R)
        x = torch.randn(n_tok, H, device="cuda").to(bf16)
        idx = torch.rand(n_tok, E, device="cuda").topk(k, dim=-1).indices.int()
        gw = torch.rand(n_tok, k, device="cuda")
        disp = MoEDispatcher(comm, n_experts=E, top_k=k, hidden=H, max_tokens=n_tok, capacity_factor=1.5)
        state = {}

        def do_dispatch():
            state["r"] = disp.route(idx)
            state["recv"] = disp.dispatch(x, state["r"])
        ms_d = timed(do_dispatch)
        y, _ = disp.next_buffer()
        ms_c = timed(lambda: disp.combine(y, state["r"], gw))
        link_bytes = frac * n_tok * k * H * 2
        roof = link_bytes / LINK * 1e3
        send = torch.empty(n_tok * k, H, dtype=bf16, device="cuda")
        recvb = torch.empty(n_tok * k, H, dtype=bf16, device="cuda")
        ms_a2a = timed(lambda: dist.all_to_all_single(recvb, send))
        emit(op="moe_route+dispatch", tokens=n_tok, top_k=k, hidden=H, world=W, ms=ms_d, roofline_ms=roof,
             frac_of_roofline=roof / ms_d, nccl_all_to_all_only_ms=ms_a2a)
        emit(op="moe_combine", tokens=n_tok, top_k=k, hidden=H, world=W, ms=ms_c, roofline_ms=roof,
             frac_of_roofline=roof / ms_c, nccl_all_to_all_only_ms=ms_a2a)
    _C.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
