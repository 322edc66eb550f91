"""Device-side timing helpers (CUDA events on the launching stream, max over ranks)."""
from __future__ import annotations

import torch


def cuda_time_ms(fn, iters: int = 10, warmup: int = 3, flush_l2: bool = True):
    """Median / min time of ``fn()`` in milliseconds; an L2-sized buffer is rewritten between
    iterations so every run starts from a cold L2."""
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.int8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2], times[0]


def max_over_ranks(value: float) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if torch.cuda.is_available() else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
