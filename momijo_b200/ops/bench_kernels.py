"""Per-kernel microbenchmarks with roofline fractions.

    python -m momijo_b200.ops.bench_kernels --op gemm|attn|attn_kernel|norm|ce|adamw|misc|all [--small]

Each kernel is timed with CUDA events on the launching stream after warm-up, with an L2-sized
buffer rewritten between iterations. Achieved FLOP/s or bytes/s are reported against the measured
peaks in MEASURED_PEAKS.json at the repository root (fallback 1.59 PFLOP/s, 6.65 TB/s). ``--small``
runs one reduced case per op, sized for a profiler capture (a few hundred MB on the device).
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from .. import ops
from ..utils.timing import cuda_time_ms

bf16 = torch.bfloat16


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops"] * 1e12, p["hbm_gbs"] * 1e9, "measured"
    except Exception:
        return 1.59e15, 6.65e12, "fallback"


def bench_gemm(small):
    flops_peak, _, tag = peaks()
    shapes = [(16384, 2304, 768, False, False), (8192, 8192, 4096, False, False)] if small else [
        (16384, 2304, 768, False, False), (16384, 768, 768, False, False),
        (16384, 3072, 768, False, False), (16384, 768, 3072, False, False),
        (16384, 50304, 768, False, False), (16384, 768, 50304, False, True),
        (50304, 768, 16384, True, True), (3072, 768, 16384, True, True),
        (8192, 8192, 8192, False, False), (32768, 4096, 4096, False, False),
        (32768, 14336, 4096, False, False)]
    rows = []
    for M, N, K, a_mn, b_mn in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(bf16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(bf16)
        out = torch.empty(M, N, device="cuda", dtype=bf16)
        med, best = cuda_time_ms(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out), iters=5 if small else 10)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        tmed, tbest = cuda_time_ms(lambda: torch.matmul(A, B, out=out), iters=5 if small else 10)
        fl = 2.0 * M * N * K
        rows.append({"op": "gemm", "M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn,
                     "ms": med, "tflops": fl / med / 1e9, f"frac_of_{tag}_peak": fl / (med * 1e-3) / flops_peak,
                     "cublas_ms": tmed, "vs_cublas": tmed / med})
    return rows


def bench_attn(small):
    flops_peak, _, tag = peaks()
    cfgs = [(2, 1024, 12, 12, 64), (1, 2048, 16, 4, 128)] if small else [(16, 1024, 12, 12, 64), (2, 4096, 32, 8, 128),
                                                     (8, 4096, 16, 16, 128)]
    rows = []
    for B, T, Hq, Hkv, D in cfgs:
        cols = (Hq + 2 * Hkv) * D
        qkv = (torch.randn(B * T, cols, device="cuda")).to(bf16).requires_grad_(True)
        dy = torch.randn(B * T, Hq * D, device="cuda").to(bf16)
        f = lambda: ops.attention_packed(qkv, B, T, Hq, Hkv, D, causal=True)
        med, _ = cuda_time_ms(f, iters=5 if small else 10)
        out = f()
        bmed, _ = cuda_time_ms(lambda: out.backward(dy, retain_graph=True), iters=5 if small else 10)
        fl = 4.0 * B * Hq * T * T * D / 2
        q = torch.randn(B, Hq, T, D, device="cuda", dtype=bf16, requires_grad=True)
        k = torch.randn(B, Hkv, T, D, device="cuda", dtype=bf16, requires_grad=True)
        v = torch.randn(B, Hkv, T, D, device="cuda", dtype=bf16, requires_grad=True)
        sd = lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True,
                                                                      enable_gqa=Hq != Hkv)
        smed, _ = cuda_time_ms(sd, iters=5 if small else 10)
        so = sd()
        go = torch.randn_like(so)
        sbmed, _ = cuda_time_ms(lambda: so.backward(go, retain_graph=True), iters=5 if small else 10)
        rows.append({"op": "attn", "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "D": D, "fwd_ms": med,
                     "fwd_tflops": fl / med / 1e9, f"fwd_frac_of_{tag}_peak": fl / (med * 1e-3) / flops_peak,
                     "bwd_ms": bmed, "bwd_tflops": 2.5 * fl / bmed / 1e9,
                     "sdpa_fwd_ms": smed, "sdpa_bwd_ms": sbmed})
    return rows


def bench_attn_kernel(small):
    """Kernel-level timing of the attention forward: back-to-back launches over rotating inputs that together
    exceed L2, CUDA events around the whole batch (no per-call host overhead in the number)."""
    import math

    from .. import _C

    rows = []
    cfgs = [(2, 1024, 12, 12, 64)] if small else [(16, 1024, 12, 12, 64), (2, 4096, 32, 8, 128),
                                                    (8, 4096, 16, 16, 128), (4, 4096, 16, 16, 64)]
    n = 24
    for B, T, Hq, Hkv, D in cfgs:
        cols = (Hq + 2 * Hkv) * D
        nb = max(3, int(300e6 // (B * T * cols * 2)) + 1)
        qs = [torch.randn(B * T, cols, device="cuda").to(bf16) for _ in range(nb)]
        out = torch.empty(B * T, Hq * D, dtype=bf16, device="cuda")
        lse = torch.empty(B, Hq, T, dtype=torch.float32, device="cuda")
        st = _C.status_tensor("cuda")

        def fwd(q):
            _C.call("mmj_attn_fwd", _C.ptr(q), cols, 0, _C.ptr(q), cols, Hq * D, _C.ptr(q), cols, (Hq + Hkv) * D,
                    _C.ptr(out), Hq * D, 0, _C.ptr(lse), B, T, Hq, Hkv, D, 1.0 / math.sqrt(D), 1, _C.ptr(st),
                    _C.current_stream())

        q4 = [torch.randn(B, Hq, T, D, device="cuda", dtype=bf16) for _ in range(nb)]
        k4 = [torch.randn(B, Hkv, T, D, device="cuda", dtype=bf16) for _ in range(nb)]
        v4 = [torch.randn(B, Hkv, T, D, device="cuda", dtype=bf16) for _ in range(nb)]
        sd = lambda i: torch.nn.functional.scaled_dot_product_attention(q4[i], k4[i], v4[i], is_causal=True,
                                                                        enable_gqa=Hq != Hkv)
        res = []
        for f in (lambda i: fwd(qs[i]), sd):
            for i in range(4):
                f(i % nb)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(n):
                f(i % nb)
            b.record()
            torch.cuda.synchronize()
            res.append(a.elapsed_time(b) / n)
        _C.check_status()
        fl = 4.0 * B * Hq * T * T * D / 2
        rows.append({"op": "attn_fwd_kernel", "B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "D": D, "fwd_ms": res[0],
                     "fwd_tflops": fl / res[0] / 1e9, "sdpa_fwd_ms": res[1], "speed_vs_sdpa": res[1] / res[0]})
    return rows


def bench_norm(small):
    """LayerNorm forward and backward launchers timed directly (no autograd, no allocation in the timed call).
    ``MOMIJO_NORM_STREAM=0`` selects the row-per-CTA kernels."""
    from .. import _C

    _, bw_peak, tag = peaks()
    rows = []
    for R, C in ([(131072, 768)] if small else [(16384, 768), (32768, 4096), (262144, 768)]):
        x = torch.randn(R, C, device="cuda").to(bf16)
        g = torch.ones(C, device="cuda", dtype=bf16)
        b = torch.zeros(C, device="cuda", dtype=bf16)
        y, dy, dx = torch.empty_like(x), torch.randn_like(x), torch.empty_like(x)
        mean = torch.empty(R, device="cuda")
        rstd = torch.empty(R, device="cuda")
        dg, db = torch.empty_like(g), torch.empty_like(b)
        nparts = _C.lib().mmj_norm_bwd_parts(R)
        scratch = torch.empty(2 * nparts * C, device="cuda")
        st = _C.ptr(_C.status_tensor(x.device))
        f = lambda: _C.call("mmj_norm_fwd", _C.ptr(x), None, None, _C.ptr(g), _C.ptr(b), _C.ptr(y), _C.ptr(mean),
                            _C.ptr(rstd), R, C, 1e-5, 0, st, _C.current_stream())
        bk = lambda: _C.call("mmj_norm_bwd", _C.ptr(dy), _C.ptr(x), _C.ptr(g), _C.ptr(mean), _C.ptr(rstd), None,
                             _C.ptr(dx), _C.ptr(dg), _C.ptr(db), _C.ptr(scratch), R, C, 0, 0, st,
                             _C.current_stream())
        med, _ = cuda_time_ms(f)
        bmed, _ = cuda_time_ms(bk)
        _C.check_status()
        by = 2.0 * R * C * 2
        rows.append({"op": "layernorm", "rows": R, "C": C, "fwd_ms": med, "fwd_GBs": by / med / 1e6,
                     f"fwd_frac_of_{tag}_bw": by / (med * 1e-3) / bw_peak, "bwd_ms": bmed,
                     "bwd_GBs": 1.5 * by / bmed / 1e6,
                     f"bwd_frac_of_{tag}_bw": 1.5 * by / (bmed * 1e-3) / bw_peak})
    return rows


def bench_ce(small):
    _, bw_peak, tag = peaks()
    R, V = (2048, 50257) if small else (16384, 50257)
    Vp = ops.pad_vocab(V)
    logits = torch.randn(R, Vp, device="cuda").to(bf16)
    tgt = torch.randint(0, V, (R,), device="cuda")
    from .. import _C

    lr = torch.empty(R, device="cuda")
    f = lambda: _C.call("mmj_ce_fwd_bwd", _C.ptr(logits), Vp, V, _C.ptr(tgt), _C.ptr(lr), R, 1.0 / R,
                        None, -100, 1, _C.current_stream())
    med, _ = cuda_time_ms(f)
    by = 2.0 * R * Vp * 2
    return [{"op": "softmax_ce_fwd_bwd", "rows": R, "V": V, "ms": med, "GBs": by / med / 1e6,
             f"frac_of_{tag}_bw": by / (med * 1e-3) / bw_peak}]


def bench_adamw(small):
    _, bw_peak, tag = peaks()
    n = 16 * 1024 * 1024 if small else 124 * 1024 * 1024
    g = torch.randn(n, device="cuda").to(bf16)
    w, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p = torch.empty(n, device="cuda", dtype=bf16)
    f = lambda: ops.adamw_flat(g, w, m, v, p, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                               weight_decay=0.1, step=3)
    med, _ = cuda_time_ms(f)
    by = n * (2 + 12 + 12 + 2)
    return [{"op": "adamw", "n": n, "ms": med, "GBs": by / med / 1e6,
             f"frac_of_{tag}_bw": by / (med * 1e-3) / bw_peak}]


def bench_misc(small):
    """The remaining bandwidth-bound kernels, one case each (bytes = algorithmic reads + writes): RoPE, SwiGLU,
    GELU, embedding, bias-gradient column sum, sum of squares, direct / GEMM convolution, pooling, the MoE
    router and the vision filters. Runs on the CPU paths too (tiny sizes) so that the calls stay checked
    where there is no GPU."""
    from . import conv as C
    from ..parallel.ep import _RouterTopK
    from ..vision import kernels as VK

    cuda = torch.cuda.is_available()
    dev = "cuda" if cuda else "cpu"
    _, bw_peak, tag = peaks()
    big = cuda and not small
    rows_out = []

    once = os.environ.get("MOMIJO_BENCH_ONCE", "0") == "1"   # one launch per kernel: for a profiler capture

    def run(name, fn, nbytes, **extra):
        if cuda and once:
            fn()
            torch.cuda.synchronize()
            med = float("nan")
        elif cuda:
            med, _ = cuda_time_ms(fn)
        else:
            fn()
            med = float("nan")
        r = {"op": name, "ms": med, "GBs": nbytes / med / 1e6 if cuda else float("nan"),
             f"frac_of_{tag}_bw": nbytes / (med * 1e-3) / bw_peak if cuda else float("nan")}
        r.update(extra)
        rows_out.append(r)

    R, Cc = (32768, 4096) if big else ((8192, 4096) if cuda else (64, 128))
    dt = bf16
    x = torch.randn(R, Cc, device=dev).to(dt)
    # RoPE in place on 32 heads of 128
    D = 128
    T = 4096 if cuda else 64
    tab = ops.rope_table(T, D, 10000.0, x.device)
    run("rope", lambda: ops.rope_inplace(x, tab, 0, Cc // D, D, T), 2.0 * R * Cc * 2, rows=R, cols=Cc)
    gu = torch.randn(R, 2 * Cc, device=dev).to(dt).requires_grad_(True)
    run("swiglu_fwd", lambda: ops.swiglu(gu), 3.0 * R * Cc * 2, rows=R, cols=Cc)
    y = ops.swiglu(gu)
    dy = torch.randn_like(y)
    run("swiglu_bwd", lambda: y.backward(dy, retain_graph=True), 5.0 * R * Cc * 2, rows=R, cols=Cc)
    xa = x.detach().clone().requires_grad_(True)
    run("gelu_fwd", lambda: ops.activation(xa, "gelu"), 2.0 * R * Cc * 2, rows=R, cols=Cc)
    ya = ops.activation(xa, "gelu")
    dya = torch.randn_like(ya)
    run("gelu_bwd", lambda: ya.backward(dya, retain_graph=True), 3.0 * R * Cc * 2, rows=R, cols=Cc)
    # embedding gather + scatter-add
    V, Ce = (50304, 1024) if cuda else (512, 64)
    ntok = 65536 if cuda else 256
    wte = torch.randn(V, Ce, device=dev).to(dt).requires_grad_(True)
    tok = torch.randint(0, V, (ntok // 1024 if cuda else 1, 1024 if cuda else ntok), device=dev)
    run("embedding_fwd", lambda: ops.embedding(tok, wte), 2.0 * ntok * Ce * 2, tokens=ntok, C=Ce)
    e = ops.embedding(tok, wte)
    de = torch.randn_like(e)
    run("embedding_bwd", lambda: e.backward(de, retain_graph=True), 3.0 * ntok * Ce * 2, tokens=ntok, C=Ce)
    # bias gradient (column sum) and gradient norm
    from .functional import _colsum
    xc = torch.randn(R, 2048 if cuda else 64, device=dev).to(dt)
    run("colsum", lambda: _colsum(xc), 1.0 * xc.numel() * 2, rows=R, cols=xc.shape[1])
    g = torch.randn(R * Cc, device=dev).to(dt)
    run("sq_norm", lambda: ops.sq_norm(g), 1.0 * g.numel() * 2, n=g.numel())
    # convolution and pooling (NCHW)
    N_, Ci, H, Co = (32, 64, 56, 64) if cuda else (2, 4, 8, 4)
    xi = torch.randn(N_, Ci, H, H, device=dev)
    wc = torch.randn(Co, Ci, 3, 3, device=dev) * 0.05
    conv_bytes = 4.0 * (xi.numel() + N_ * Co * H * H)
    run("conv2d_fp32_direct", lambda: C.conv2d(xi, wc, None, (1, 1), (1, 1)), conv_bytes,
        flops=2.0 * N_ * Co * H * H * Ci * 9)
    xb, wb = xi.to(dt), wc.to(dt)
    run("conv2d_bf16_im2col_gemm", lambda: C.conv2d(xb, wb, None, (1, 1), (1, 1)), conv_bytes / 2,
        flops=2.0 * N_ * Co * H * H * Ci * 9)
    run("max_pool2d", lambda: C.max_pool2d(xi, (2, 2)), 4.0 * xi.numel() * 1.25)
    run("avg_pool2d", lambda: C.avg_pool2d(xi, (2, 2)), 4.0 * xi.numel() * 1.25)
    # MoE router: softmax, top-6 of 64, renormalise, counts, auxiliary loss
    n_r, E, k = (65536, 64, 6) if cuda else (128, 8, 2)
    lg = torch.randn(n_r, E, device=dev).to(dt if cuda else torch.float32)
    if cuda:
        run("moe_router", lambda: _RouterTopK.apply(lg, k, 0.01), 1.0 * n_r * E * 2 + n_r * k * 8, tokens=n_r)
    # vision filters on one 2048 x 2048 RGB image (uint8, HWC)
    hw = 2048 if cuda else 32
    img = torch.randint(0, 256, (hw, hw, 3), dtype=torch.uint8, device=dev)
    gray = torch.randint(0, 256, (hw, hw, 1), dtype=torch.uint8, device=dev)
    if cuda:
        px = float(hw * hw)
        run("vision_resize_bilinear_x0.5", lambda: VK.resize(img, hw // 2, hw // 2, True), px * 3 * 1.25)
        run("vision_to_gray", lambda: VK.to_gray(img), px * 4)
        run("vision_gaussian_5x5", lambda: VK.gaussian_blur(img, 5, 5, 1.0), px * 3 * 4)
        run("vision_median_3", lambda: VK.median(img, 3), px * 3 * 2)
        run("vision_bilateral_r2", lambda: VK.bilateral(img, 2, 25.0, 2.0), px * 3 * 2)
        run("vision_sobel", lambda: VK.deriv3(gray, 0), px * 2)
        run("vision_canny", lambda: VK.canny(gray, 50, 150), px * 2)
        run("vision_erode_3", lambda: VK.morph(gray, 3, False), px * 2)
        run("vision_clahe", lambda: VK.clahe_plane(gray[..., 0].contiguous(), 2.0, 8), px * 2)
        bw = (gray[..., 0] > 127).to(torch.uint8).contiguous()
        run("vision_connected_components", lambda: VK.connected_components(bw, 4), px * 5)
    return rows_out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all")
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    table = {"gemm": bench_gemm, "attn": bench_attn, "attn_kernel": bench_attn_kernel, "norm": bench_norm, "ce": bench_ce,
             "adamw": bench_adamw, "misc": bench_misc}
    for name, fn in table.items():
        if a.op in ("all", name):
            for r in fn(a.small):
                print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))


if __name__ == "__main__":
    main()
