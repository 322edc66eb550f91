"""Bandwidth-bound kernels and attention against fp32 torch references."""
import math

import pytest
import torch
import torch.nn.functional as F

from momijo_b200 import ops
from momijo_b200.ops import functional as fn

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _rand(*s, scale=1.0, grad=False):
    t = (torch.randn(*s, device="cuda") * scale).to(bf16)
    return t.requires_grad_(grad)


def _close(out, ref, tol=2e-2, fro=1e-2):
    """Max error relative to the largest reference entry, and the relative Frobenius error."""
    out, ref = out.float(), ref.float()
    err = ((out - ref).abs().max() / ref.abs().max().clamp_min(1e-6)).item()
    assert err < tol, f"relative max error {err}"
    ferr = ((out - ref).norm() / ref.norm().clamp_min(1e-6)).item()
    assert ferr < fro, f"relative Frobenius error {ferr}"


@pytest.mark.parametrize("C", [768, 1600, 2048, 4096, 5120, 8192, 136])
@pytest.mark.parametrize("mode", ["ln", "rms"])
@pytest.mark.parametrize("fused_res", [False, True])
@pytest.mark.parametrize("rows", [300, 20011])
def test_norm(C, mode, fused_res, rows):
    # 20011 rows: more tiles per CTA than the shared-memory ring has stages, and a ragged last tile
    torch.manual_seed(0)
    x, g, b = _rand(rows, C, grad=True), _rand(C, grad=True), _rand(C, grad=True)
    res = _rand(rows, C, grad=True) if fused_res else None
    if mode == "ln":
        out = ops.layer_norm(x, g, b, 1e-5, residual=res)
    else:
        out = ops.rms_norm(x, g, 1e-5, residual=res)
    y, r = out if fused_res else (out, None)
    xs = x.float() + (res.float() if fused_res else 0)
    xs = xs.to(bf16).float() if fused_res else xs
    xs = xs.detach().requires_grad_(True)
    gf, bfl = g.float().detach().requires_grad_(True), b.float().detach().requires_grad_(True)
    if mode == "ln":
        yr = F.layer_norm(xs, (C,), gf, bfl, 1e-5)
    else:
        yr = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
    _close(y, yr)
    dy = _rand(rows, C)
    loss = (y.float() * dy.float()).sum()
    if fused_res:
        dr = _rand(rows, C)
        loss = loss + (r.float() * dr.float()).sum()
        _close(r, xs)
    loss.backward()
    lr = (yr * dy.float()).sum()
    if fused_res:
        lr = lr + (xs * dr.float()).sum()
    lr.backward()
    _close(x.grad, xs.grad, 3e-2)
    if fused_res:
        _close(res.grad, xs.grad, 3e-2)
    _close(g.grad, gf.grad, 3e-2)
    if mode == "ln":
        _close(b.grad, bfl.grad, 3e-2)


def test_swiglu_and_activations():
    torch.manual_seed(1)
    gu = _rand(257, 2 * 1408, grad=True)
    y = ops.swiglu(gu)
    gr = gu.detach().float().requires_grad_(True)
    a, b = gr.chunk(2, -1)
    yr = F.silu(a) * b
    _close(y, yr)
    dy = _rand(257, 1408)
    y.backward(dy)
    yr.backward(dy.float())
    _close(gu.grad, gr.grad)
    for kind, ref in [("gelu", lambda t: F.gelu(t, approximate="tanh")), ("silu", F.silu),
                      ("relu", torch.relu), ("sigmoid", torch.sigmoid), ("tanh", torch.tanh),
                      ("leaky_relu", lambda t: F.leaky_relu(t, 0.01))]:
        x = _rand(64, 256, grad=True)
        y = ops.activation(x, kind)
        xr = x.detach().float().requires_grad_(True)
        yr = ref(xr)
        _close(y, yr)
        y.backward(torch.ones_like(y))
        yr.backward(torch.ones_like(yr))
        _close(x.grad, xr.grad)


def test_embedding():
    torch.manual_seed(2)
    V, C, B, T = 1000, 128, 4, 64
    wte, wpe = _rand(V, C, grad=True), _rand(T, C, grad=True)
    tok = torch.randint(0, V, (B, T), device="cuda")
    y = ops.embedding(tok, wte, wpe, T)
    wr, pr = wte.detach().float().requires_grad_(True), wpe.detach().float().requires_grad_(True)
    yr = F.embedding(tok, wr) + pr[:T]
    _close(y, yr)
    dy = _rand(B, T, C)
    y.backward(dy)
    yr.backward(dy.float())
    _close(wte.grad, wr.grad, 3e-2)
    _close(wpe.grad, pr.grad, 3e-2)


@pytest.mark.parametrize("V", [1000, 50257])
def test_cross_entropy(V):
    torch.manual_seed(3)
    n = 64
    Vp = ops.pad_vocab(V)
    buf = torch.full((n, Vp), 7.0, device="cuda", dtype=bf16)  # padding must be ignored
    logits = buf[:, :V]
    logits.copy_(_rand(n, V, scale=2.0))
    tgt = torch.randint(0, V, (n,), device="cuda")
    tgt[3] = -100
    loss, dl = ops.softmax_cross_entropy(logits, tgt)
    lr = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(lr, tgt, ignore_index=-100)   # mean over the rows that count
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    _close(dl, lr.grad, 3e-2)


def test_lm_head_ce():
    torch.manual_seed(4)
    M, C, V = 256, 128, 1000
    x, w = _rand(M, C, grad=True), _rand(ops.pad_vocab(V), C, scale=0.05, grad=True)
    tgt = torch.randint(0, V, (M,), device="cuda")
    loss = ops.lm_head_cross_entropy(x, w, tgt, V)
    loss.backward()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = F.cross_entropy((xr @ wr.t())[:, :V], tgt)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-2 * abs(ref.item())
    _close(x.grad, xr.grad, 4e-2)
    _close(w.grad, wr.grad, 4e-2)


def test_lm_head_ce_scaled_loss_reaches_main_grad():
    """(loss * s).backward() must scale the head's weight gradient too when that gradient is written straight
    into a flat main_grad buffer (autograd then never sees it), and ignored targets must not count."""
    torch.manual_seed(5)
    M, C, V = 256, 128, 1000
    x = _rand(M, C, grad=True)
    w = _rand(ops.pad_vocab(V), C, scale=0.05, grad=True)
    w.main_grad = torch.zeros_like(w)
    w._mg_fresh = True
    tgt = torch.randint(0, V, (M,), device="cuda")
    tgt[:17] = -100
    loss = ops.lm_head_cross_entropy(x, w, tgt, V)
    (loss * 0.25).backward()
    assert w.grad is None
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = F.cross_entropy((xr @ wr.t())[:, :V], tgt, ignore_index=-100)
    (ref * 0.25).backward()
    assert abs(loss.item() - ref.item()) < 1e-2 * abs(ref.item())
    _close(x.grad, xr.grad, 4e-2, 2e-2)
    _close(w.main_grad, wr.grad, 4e-2, 2e-2)


def test_adamw_and_sqnorm():
    torch.manual_seed(5)
    n = 100003
    g = _rand(n)
    w = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    p = torch.empty(n, device="cuda", dtype=bf16)
    wr = w.clone().requires_grad_(True)
    opt = torch.optim.AdamW([wr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ops.adamw_flat(g, w, m, v, p, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                       step=step)
        wr.grad = g.float()
        opt.step()
    assert (w - wr.detach()).abs().max().item() < 1e-4
    assert torch.equal(p, w.to(bf16))
    s = ops.sq_norm(g)
    assert abs(s.item() - g.float().pow(2).sum().item()) < 1e-3 * s.item()
    fi = torch.zeros(1, dtype=torch.int32, device="cuda")
    g2 = g.clone()
    g2[17] = float("inf")
    ops.sq_norm(g2, found_inf=fi)
    assert fi.item() == 1


def test_rope_roundtrip():
    torch.manual_seed(6)
    B, T, H, D = 2, 64, 4, 64
    x = _rand(B * T, H * D)
    tab = ops.rope_table(T, D, 10000.0, "cuda")
    y = x.clone()
    ops.rope_inplace(y, tab, 0, H, D, T, 1.0)
    yr = x.clone().cpu()
    fn.rope_inplace(yr, tab.cpu(), 0, H, D, T, 1.0)
    _close(y, yr.cuda())
    ops.rope_inplace(y, tab, 0, H, D, T, -1.0)
    _close(y, x)


def _attn_ref(q, k, v, causal):
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    k = k.repeat_interleave(Hq // Hkv, 1)
    v = v.repeat_interleave(Hq // Hkv, 1)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(D)
    if causal:
        s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return torch.softmax(s, -1) @ v


@pytest.mark.parametrize("B,T,Hq,Hkv,D,causal", [
    (2, 256, 4, 4, 64, True), (1, 384, 2, 2, 64, False), (2, 256, 8, 2, 128, True),
    (1, 200, 2, 2, 64, True), (1, 128, 4, 1, 128, False), (2, 1024, 12, 12, 64, True)])
def test_attention(B, T, Hq, Hkv, D, causal):
    torch.manual_seed(7)
    cols = (Hq + 2 * Hkv) * D
    qkv = _rand(B * T, cols, grad=True)
    out = ops.attention_packed(qkv, B, T, Hq, Hkv, D, causal=causal)
    x = qkv.detach().float().requires_grad_(True)
    q = x[:, :Hq * D].reshape(B, T, Hq, D).transpose(1, 2)
    k = x[:, Hq * D:(Hq + Hkv) * D].reshape(B, T, Hkv, D).transpose(1, 2)
    v = x[:, (Hq + Hkv) * D:].reshape(B, T, Hkv, D).transpose(1, 2)
    ref = _attn_ref(q, k, v, causal).transpose(1, 2).reshape(B * T, Hq * D)
    _close(out, ref)
    dy = _rand(B * T, Hq * D)
    out.backward(dy)
    ref.backward(dy.float())
    gq, rq = qkv.grad.float(), x.grad
    for name, sl in [("dq", slice(0, Hq * D)), ("dk", slice(Hq * D, (Hq + Hkv) * D)),
                     ("dv", slice((Hq + Hkv) * D, cols))]:
        err = ((gq[:, sl] - rq[:, sl]).abs().max() / rq[:, sl].abs().max()).item()
        assert err < 4e-2, f"{name} relative max error {err}"


def test_debug_bounds_build_records_bad_index(tmp_path):
    """The bounds-checked build records an out-of-range token id (and still clamps it); run in a child
    process because the library variant is chosen at import time."""
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import torch\n"
        "from momijo_b200 import _C, ops\n"
        "assert _C.DEBUG_BOUNDS\n"
        "w = torch.randn(64, 32, device='cuda').to(torch.bfloat16)\n"
        "tok = torch.tensor([[1, 2, 99, 3]], device='cuda')\n"
        "y = ops.embedding(tok, w)\n"
        "rec = _C.debug_bounds()\n"
        "e = [r for r in rec if r['unit'] == 'elementwise'][0]\n"
        "assert e['count'] > 0 and e['index'] == 99 and e['limit'] == 64, rec\n"
        "assert torch.equal(y.reshape(-1, 32)[2], w[63])\n"
        "assert all(r['count'] == 0 for r in _C.debug_bounds())\n"
        "print('BOUNDS_OK')\n")
    env = dict(os.environ, MOMIJO_DEBUG_BOUNDS="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert "BOUNDS_OK" in out.stdout, out.stdout + out.stderr


@pytest.mark.parametrize("n,E,k", [(1000, 64, 6), (257, 8, 2), (64, 160, 4)])
def test_moe_router_kernel_matches_torch(n, E, k):
    """Device router (softmax, top-k, renormalise, counts, auxiliary loss) and its backward against torch."""
    from momijo_b200.parallel.ep import _RouterTopK

    torch.manual_seed(9)
    coef = 0.01
    logits = (torch.randn(n, E, device="cuda") * 2).to(bf16).requires_grad_(True)
    w, idx, aux = _RouterTopK.apply(logits, k, coef)
    lr = logits.detach().float().requires_grad_(True)
    probs = torch.softmax(lr, -1)
    wr, ir = torch.topk(probs, k, dim=-1)
    wr = wr / wr.sum(-1, keepdim=True)
    f = torch.zeros(E, device="cuda").scatter_add_(0, ir.reshape(-1), torch.ones(ir.numel(), device="cuda")) / ir.numel()
    auxr = coef * E * (f * probs.mean(0)).sum()
    assert torch.equal(idx.long().sort(-1).values, ir.sort(-1).values)
    order = idx.long().argsort(-1)
    order_r = ir.argsort(-1)
    _close(w.gather(1, order), wr.gather(1, order_r), 1e-4, 1e-4)
    assert abs(aux.item() - auxr.item()) < 1e-5 * max(1.0, abs(auxr.item()))
    gw = torch.randn(n, k, device="cuda")
    # the same upstream gradient for the same (token, expert) pairs
    loss = (w.gather(1, order) * gw).sum() + 3.0 * aux
    loss.backward()
    loss_r = (wr.gather(1, order_r) * gw).sum() + 3.0 * auxr
    loss_r.backward()
    _close(logits.grad, lr.grad, 3e-2, 1e-2)
    # bitwise reproducible
    w2, idx2, aux2 = _RouterTopK.apply(logits.detach(), k, coef)
    assert torch.equal(w2, w.detach()) and torch.equal(idx2, idx) and aux2.item() == aux.item()


_CHAIN = r'''
import hashlib, torch
from momijo_b200 import ops
from momijo_b200.ops import functional as fn
bf16 = torch.bfloat16
torch.manual_seed(5)
R, C, F_ = 4096, 768, 3072
x = (torch.randn(R, C, device="cuda")).to(bf16).requires_grad_(True)
g, b = [torch.randn(C, device="cuda").to(bf16).requires_grad_(True) for _ in range(2)]
w1 = (torch.randn(F_, C, device="cuda") * 0.02).to(bf16).requires_grad_(True)
b1 = torch.zeros(F_, device="cuda", dtype=bf16, requires_grad=True)
w2 = (torch.randn(C, F_, device="cuda") * 0.02).to(bf16).requires_grad_(True)
b2 = torch.zeros(C, device="cuda", dtype=bf16, requires_grad=True)
outs = []
for it in range(3):   # the same chain three times: launches follow each other without a gap
    h = ops.layer_norm(x, g, b)
    y = fn.mlp_gelu(h, w1, b1, w2, b2, residual=x)
    z, r = ops.layer_norm(y, g, b, residual=x)
    (z.float().sum() * 1e-3 + r.float().mean()).backward()
    outs += [y, z, r]
outs += [x.grad, g.grad, b.grad, w1.grad, b1.grad, w2.grad, b2.grad]
torch.cuda.synchronize()
hsh = hashlib.sha256()
for t in outs:
    hsh.update(t.detach().float().cpu().numpy().tobytes())
print("CHAIN", hsh.hexdigest())
'''


def test_dependent_launch_gives_the_same_bits_as_plain_stream_order():
    """Norm -> GEMM(+GELU) -> GEMM -> norm forward and backward, three times back to back: kernels launched
    with programmatic stream serialization (each waits for its predecessor before its first global access)
    must produce exactly the bits of the same chain launched in plain stream order."""
    import os
    import subprocess
    import sys
    res = {}
    for pdl in ("1", "0"):
        env = dict(os.environ, MOMIJO_PDL=pdl)
        r = subprocess.run([sys.executable, "-c", _CHAIN], capture_output=True, text=True, env=env, timeout=300,
                           cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        res[pdl] = [l for l in r.stdout.splitlines() if l.startswith("CHAIN")][0]
    assert res["1"] == res["0"]
