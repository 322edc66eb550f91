"""tcgen05 GEMM against a plain fp32 torch reference: operand majors, ragged shapes, epilogues."""
import pytest
import torch

from momijo_b200.ops import gemm
from momijo_b200.ops.gemm import _gelu_tanh, _gelu_tanh_grad

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _rand(*s, scale=1.0):
    return (torch.randn(*s, device="cuda") * scale).to(bf16)


def _close(out, ref, tol=2e-2, fro=1e-2):
    """Max error relative to the largest reference entry, and the relative Frobenius error (bf16 rounding
    alone is about 3e-3 of the norm; a dropped K tail or a misplaced tile moves it by far more)."""
    out, ref = out.float(), ref.float()
    denom = ref.abs().max().clamp_min(1e-6)
    err = ((out - ref).abs().max() / denom).item()
    assert err < tol, f"relative max error {err}"
    ferr = ((out - ref).norm() / ref.norm().clamp_min(1e-6)).item()
    assert ferr < fro, f"relative Frobenius error {ferr}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 256), (384, 768, 768), (1000, 520, 328),
                                   (129, 72, 200), (2048, 2304, 768), (64, 64, 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_majors(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    Kp = K
    a = _rand(K, M) if a_mn else _rand(M, Kp)
    b = _rand(K, N) if b_mn else _rand(N, Kp)
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte aligned leading dimension")
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    A = (a.t() if a_mn else a).float()
    B = (b if b_mn else b.t()).float()
    _close(out, A @ B)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths(bn):
    torch.manual_seed(1)
    a, b = _rand(640, 512), _rand(768, 512)
    _close(gemm(a, b, bn=bn), a.float() @ b.float().t())


def test_gemm_epilogues():
    torch.manual_seed(2)
    M, N, K = 512, 1024, 384
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    bias, aux = _rand(N), _rand(M, N)
    ref = a.float() @ b.float().t()
    _close(gemm(a, b, bias=bias), ref + bias.float())
    act, pre = gemm(a, b, bias=bias, gelu=True)
    _close(pre, ref + bias.float())
    _close(act, _gelu_tanh(ref + bias.float()))
    _close(gemm(a, b, dgelu_aux=aux), ref * _gelu_tanh_grad(aux.float()))
    _close(gemm(a, b, add_aux=aux), ref + aux.float())
    _close(gemm(a, b, mul_aux=aux), ref * aux.float())
    _close(gemm(a, b, silu=True), torch.nn.functional.silu(ref))
    rs = torch.rand(M, device="cuda")
    _close(gemm(a, b, row_scale=rs), ref * rs[:, None])
    o32 = gemm(a, b, out_f32=True)
    assert o32.dtype == torch.float32
    _close(o32, ref, tol=1e-3)
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    gemm(a, b, out=acc, accumulate=True)
    _close(acc, ref + 1.0, tol=1e-3)
    accb = _rand(M, N)
    expect = ref + accb.float()
    gemm(a, b, out=accb, accumulate=True)
    _close(accb, expect)


def test_gemm_padded_vocab_view():
    """Output view with a wider leading dimension and a ragged N (LM head layout)."""
    torch.manual_seed(3)
    M, K, V, Vp = 256, 128, 1000, 1024
    x, w = _rand(M, K), _rand(V, K)
    logits = torch.zeros(M, Vp, device="cuda", dtype=bf16)
    gemm(x, w, out=logits[:, :V])
    _close(logits[:, :V], x.float() @ w.float().t())
    assert logits[:, V:].abs().max().item() == 0
    dx = gemm(logits[:, :V], w, b_mn=True)
    _close(dx, logits[:, :V].float() @ w.float())
    dw = gemm(logits[:, :V], x, a_mn=True, b_mn=True)
    _close(dw, logits[:, :V].float().t() @ x.float())


def test_gemm_deterministic():
    a, b = _rand(1024, 512), _rand(768, 512)
    assert torch.equal(gemm(a, b), gemm(a, b))


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 768), (1000, 520, 328), (2048, 2304, 768),
                                   (4096, 1024, 1536)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_cta_pair(M, N, K, a_mn, b_mn):
    """CTA-pair kernel (two SMs per 256 x 256 tile): same products as the one-SM kernel."""
    torch.manual_seed(3)
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=True)
    A = (a.t() if a_mn else a).float()
    B = (b if b_mn else b.t()).float()
    _close(out, A @ B)


def test_gemm_cta_pair_epilogues():
    torch.manual_seed(4)
    M, N, K = 1024, 1024, 384
    a, b = _rand(M, K), _rand(N, K, scale=0.05)
    bias, aux = _rand(N), _rand(M, N)
    ref = a.float() @ b.float().t()
    act, pre = gemm(a, b, bias=bias, gelu=True, pair=True)
    _close(pre, ref + bias.float())
    _close(act, _gelu_tanh(ref + bias.float()))
    _close(gemm(a, b, dgelu_aux=aux, pair=True), ref * _gelu_tanh_grad(aux.float()))
    _close(gemm(a, b, add_aux=aux, pair=True), ref + aux.float())
    o32 = gemm(a, b, out_f32=True, pair=True)
    _close(o32, ref, tol=1e-3)


@pytest.mark.parametrize("force", [None, (4, 128, False), (2, 256, True), (2, 256, "pair"), (5, 256, "pair")])
@pytest.mark.parametrize("M,N", [(768, 768), (3072, 768), (520, 1000)])
def test_gemm_split_k_weight_gradient(force, M, N):
    """dW = dy^T x with a long contraction: split-K slabs + reduction, on one-SM tiles and on CTA pairs."""
    from momijo_b200.ops import gemm as gemm_mod
    import sys
    mod = sys.modules["momijo_b200.ops.gemm"]
    torch.manual_seed(5)
    K = 8192
    dy, x = _rand(K, M, scale=0.1), _rand(K, N, scale=0.1)
    ref = dy.float().t() @ x.float()
    old = mod._SPLITK["force"]
    mod._SPLITK["force"] = force
    try:
        out = gemm(dy, x, a_mn=True, b_mn=True)
        _close(out, ref)
        acc = _rand(M, N)
        expect = ref + acc.float()
        gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True)
        _close(acc, expect)
    finally:
        mod._SPLITK["force"] = old
