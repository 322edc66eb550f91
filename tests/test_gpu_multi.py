"""Multi-GPU tests: peer-memory collectives and fused compute+communication kernels, run as one
process per GPU (needs >= 2 GPUs). NVLS is switched off so that a rank ending early cannot
disturb the others."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(scenarios, nproc=None, timeout=600):
    n = nproc or min(torch.cuda.device_count(), 8)   # every visible GPU of the node
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(HERE, "mp_worker.py"), *scenarios]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    out = r.stdout + r.stderr
    # the first traceback names the cause; the tail is the launcher's summary of every rank
    first = out.find("Traceback")
    shown = (out[first:first + 3000] + "\n...\n" if first >= 0 else "") + out[-2500:]
    assert r.returncode == 0, shown
    for s in scenarios:
        assert f"SCENARIO_OK {s}" in out, shown


def test_peer_allreduce_and_timeout_status():
    _run(["allreduce", "timeout"])


def test_zero_engine_matches_single_rank():
    _run(["zero"])


def test_bucketed_ddp_matches_single_rank():
    _run(["ddp"])


def test_nvls_allreduce_path():
    _run(["allreduce_nvls"])


def test_fused_allgather_gemm_and_gemm_reduce_scatter():
    _run(["ag_gemm", "gemm_rs"])


def test_moe_dispatch_combine_and_layer():
    _run(["moe", "moe_layer", "moe_drop"])


def test_tensor_parallel_llama_matches_single_rank():
    _run(["tp_llama", "tp_llama_two_launch"])


def test_fused_collectives_are_deterministic():
    _run(["determinism"])
