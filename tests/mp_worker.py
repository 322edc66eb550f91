"""Worker for the multi-GPU tests: one process per GPU, launched by tests/test_gpu_multi.py as
``python -m torch.distributed.run --nproc-per-node N tests/mp_worker.py <scenario>``.

Every scenario compares a peer-memory kernel of this library against a plain torch / NCCL
reference of the same operation and prints ``SCENARIO_OK <name>`` on rank 0 when all ranks agree.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from momijo_b200 import _C, ops  # noqa: E402
from momijo_b200.parallel.peer import PeerComm  # noqa: E402

bf16 = torch.bfloat16


def close(a, b, tol, what):
    a, b = a.float(), b.float()
    err = ((a - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()
    assert err < tol, f"{what}: relative max error {err}"


def sc_allreduce(comm):
    torch.manual_seed(comm.rank)
    n = 8 * comm.world * 1000
    x = comm.alloc(n, bf16)
    src = (torch.randn(n, device="cuda")).to(bf16)
    for it in range(3):
        x.copy_(src)
        ref = src.float().clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        dist.barrier()
        comm.all_reduce_(x)
        torch.cuda.synchronize()
        close(x, ref, 2e-2, "allreduce")
    comm.barrier()
    torch.cuda.synchronize()


def sc_zero(comm):
    """2+ rank sharded engine == single-rank engine on the concatenated batch."""
    from momijo_b200.models import GPT2, GPT2Config
    from momijo_b200.parallel import ShardedDataParallel, AdamWConfig

    cfg = GPT2Config.tiny()
    torch.manual_seed(0)
    m_dist = GPT2(cfg).cuda()
    torch.manual_seed(0)
    m_ref = GPT2(cfg).cuda()
    oc = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    eng = ShardedDataParallel(m_dist, oc, comm=comm)
    ref = ShardedDataParallel(m_ref, oc)
    g = torch.Generator().manual_seed(7)
    B = 2
    for step in range(3):
        full = torch.randint(0, cfg.vocab_size, (B * comm.world, 129), generator=g).cuda()
        mine = full[comm.rank * B:(comm.rank + 1) * B]
        loss = eng(mine[:, :-1], mine[:, 1:])
        loss.backward()
        eng.step()
        lr_ = ref(full[:, :-1], full[:, 1:])
        lr_.backward()
        ref.step()
    torch.cuda.synchronize()
    close(eng.flat.param, ref.flat.param, 2e-2, "zero params after 3 steps")
    a, b = eng.flat.layout.shard_range(comm.rank)
    close(eng.master, ref.master[a:b], 2e-2, "zero master shard")


def sc_ag_gemm(comm):
    from momijo_b200.ops.fused_comm import FusedSite, allgather_gemm

    W, R = comm.world, comm.rank
    torch.manual_seed(1)
    M, N, K = 256 * W, 384, 512
    full_ref = (torch.randn(M, K, device="cuda")).to(bf16)  # same on all ranks (same seed)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(bf16)
    site = FusedSite(comm)
    xa = comm.alloc(M * K, bf16).view(M, K)
    rows = M // W
    for it in range(2):
        xa.zero_()
        xa[R * rows:(R + 1) * rows].copy_(full_ref[R * rows:(R + 1) * rows])
        torch.cuda.synchronize()
        dist.barrier()
        out = allgather_gemm(site, xa, w, gather_a=True, comm_ctas=4)
        torch.cuda.synchronize()
        close(out, full_ref.float() @ w.float().t(), 2e-2, "allgather(A) -> gemm")
        close(xa, full_ref, 1e-6, "gathered A copy")
        dist.barrier()
    # gathered B: weight rows sharded, unaligned window of a flat buffer
    site2 = FusedSite(comm)
    Nw = 128 * W + 64
    flat = comm.alloc(Nw * K + 4096, bf16)
    wfull = (torch.randn(Nw, K, device="cuda") * 0.05).to(bf16)
    off = 1024
    total = flat.numel()
    shard = total // W
    view = flat[off:off + Nw * K].view(Nw, K)
    flat.zero_()
    lo, hi = R * shard, (R + 1) * shard
    src = torch.zeros(total, dtype=bf16, device="cuda")
    src[off:off + Nw * K] = wfull.reshape(-1)
    flat[lo:hi].copy_(src[lo:hi])
    x = (torch.randn(512, K, device="cuda")).to(bf16)
    torch.cuda.synchronize()
    dist.barrier()
    out = allgather_gemm(site2, view, x, gather_a=False, comm_ctas=4, shard_bytes=shard * 2,
                         flat_off_bytes=off * 2)
    torch.cuda.synchronize()
    close(out, x.float() @ wfull.float().t(), 2e-2, "allgather(B) -> gemm")
    dist.barrier()


def sc_gemm_rs(comm):
    from momijo_b200.ops.fused_comm import FusedSite, gemm_reduce_scatter

    W, R = comm.world, comm.rank
    torch.manual_seed(100 + R)
    M, N, K = 256 * W, 512, 256
    a = (torch.randn(M, K, device="cuda")).to(bf16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(bf16)
    site = FusedSite(comm)
    rows = M // W
    stage = comm.alloc(W * rows * N, bf16)
    out = torch.empty(rows, N, dtype=bf16, device="cuda")
    part = (a.float() @ b.float().t())
    ref = part.clone()
    dist.all_reduce(ref)
    for it in range(2):
        dist.barrier()
        gemm_reduce_scatter(site, a, b, stage, out)
        torch.cuda.synchronize()
        close(out, ref[R * rows:(R + 1) * rows], 3e-2, "gemm -> reduce-scatter")


def sc_moe(comm):
    from momijo_b200.parallel.ep import MoEDispatcher

    W, R = comm.world, comm.rank
    torch.manual_seed(50 + R)
    n_tok, H, E, k = 300, 256, 4 * W, 2
    x = torch.randn(n_tok, H, device="cuda").to(bf16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(n_tok)]).int()
    gw = torch.rand(n_tok, k, device="cuda")
    disp = MoEDispatcher(comm, n_experts=E, top_k=k, hidden=H, max_tokens=n_tok)
    for it in range(2):
        recv, info = disp.dispatch(x, idx)
        # identity experts scaled by (global expert id + 1): check routing end to end
        epr = E // W
        y = disp.expert_out_buffer()
        tg = info["tile_group"][: int(info["num_tiles"].item())]
        scale = (tg.float() + 1 + R * epr).repeat_interleave(128)[:, None]
        rows = scale.shape[0]
        y[:rows] = (recv[:rows].float() * scale).to(bf16)
        out = disp.combine(y, gw)
        torch.cuda.synchronize()
        ref = (x.float()[:, None, :] * (idx.float() + 1)[:, :, None] * gw[:, :, None]).sum(1)
        close(out, ref, 3e-2, "moe dispatch/combine")


def sc_timeout(comm):
    """A wait on a flag that nobody sets returns an error status; the context stays usable."""
    slot = comm.new_slots(1)
    st = comm.status
    st.zero_()
    _C.call("mmj_wait_flag", comm.sig.data_ptr() + 4 * slot, 1, _C.ptr(st), _C.current_stream())
    torch.cuda.synchronize()
    assert st[0].item() == 6, st.tolist()
    st.zero_()
    y = torch.ones(4, device="cuda") * 2
    assert y.sum().item() == 8


SCENARIOS = {"allreduce": sc_allreduce, "zero": sc_zero, "ag_gemm": sc_ag_gemm,
             "gemm_rs": sc_gemm_rs, "moe": sc_moe, "timeout": sc_timeout}


def main():
    names = sys.argv[1:] or list(SCENARIOS)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = PeerComm.from_default_group(heap_bytes=512 << 20)
    for name in names:
        SCENARIOS[name](comm)
        _C.check_status()
        dist.barrier()
        if comm.rank == 0:
            print(f"SCENARIO_OK {name}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
