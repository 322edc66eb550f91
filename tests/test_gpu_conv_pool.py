"""Convolution / pooling kernels against plain fp32 torch references (forward and every gradient)."""
import pytest
import torch
import torch.nn.functional as tF

from momijo_b200.ops import conv as cv

pytestmark = pytest.mark.gpu


def _close(a, b, tol, fro):
    a, b = a.float(), b.float()
    err = ((a - b).abs().max() / b.abs().max().clamp_min(1e-6)).item()
    ferr = ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
    assert err < tol and ferr < fro, (err, ferr)


def _ref(fn, tensors, dy):
    """fp32 CPU reference values and gradients."""
    ts = [t.detach().float().cpu().requires_grad_(True) for t in tensors]
    y = fn(*ts)
    y.backward(dy.float().cpu())
    return y, [t.grad for t in ts]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,C,H,W,OC,k,s,p,d,g", [
    (2, 3, 17, 19, 8, 3, 1, 1, 1, 1), (2, 8, 16, 16, 16, 3, 2, 1, 1, 1), (1, 4, 12, 12, 6, 5, 1, 2, 2, 2),
    (2, 6, 9, 9, 6, 3, 1, 1, 1, 6), (2, 16, 14, 14, 32, 3, 1, 1, 1, 1)])
def test_conv2d_forward_and_gradients(dtype, N, C, H, W, OC, k, s, p, d, g):
    torch.manual_seed(0)
    x = torch.randn(N, C, H, W, device="cuda").to(dtype).requires_grad_(True)
    w = (torch.randn(OC, C // g, k, k, device="cuda") * 0.2).to(dtype).requires_grad_(True)
    b = torch.randn(OC, device="cuda").to(dtype).requires_grad_(True)
    y = cv.conv2d(x, w, b, s, p, d, g)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr, (gx, gw, gb) = _ref(lambda a, c, e: tF.conv2d(a, c, e, s, p, d, g), (x, w, b), dy)
    tol, fro = (1e-4, 1e-5) if dtype == torch.float32 else (3e-2, 1e-2)
    _close(y, yr.cuda(), tol, fro)
    _close(x.grad, gx.cuda(), tol, fro)
    _close(w.grad, gw.cuda(), tol, fro)
    _close(b.grad, gb.cuda(), tol, fro)


def test_im2col_col2im_match_unfold_fold():
    torch.manual_seed(1)
    x = torch.randn(2, 5, 11, 13, device="cuda")
    cols = cv.im2col(x, (3, 2), (2, 1), (1, 0))
    ref = tF.unfold(x, (3, 2), padding=(1, 0), stride=(2, 1)).transpose(1, 2).reshape(-1, 5 * 6)
    assert torch.equal(cols, ref)
    back = cv.col2im(cols, x.shape, (3, 2), (2, 1), (1, 0))
    c = ref.reshape(2, -1, 30).transpose(1, 2)
    _close(back, tF.fold(c, (11, 13), (3, 2), padding=(1, 0), stride=(2, 1)), 1e-5, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,s,p", [(2, 2, 0), (3, 1, 1), (3, 2, 1)])
def test_pooling_and_deterministic_backward(dtype, k, s, p):
    torch.manual_seed(2)
    x = torch.randn(2, 4, 15, 14, device="cuda").to(dtype).requires_grad_(True)
    for fn, ref in ((lambda t: cv.max_pool2d(t, k, s, p), lambda t: tF.max_pool2d(t, k, s, p)),
                    (lambda t: cv.avg_pool2d(t, k, s, p), lambda t: tF.avg_pool2d(t, k, s, p, count_include_pad=False))):
        x.grad = None
        y = fn(x)
        dy = torch.randn_like(y)
        y.backward(dy)
        g1 = x.grad.clone()
        yr, (gx,) = _ref(ref, (x,), dy)
        tol, fro = (1e-5, 1e-6) if dtype == torch.float32 else (2e-2, 1e-2)
        _close(y, yr.cuda(), tol, fro)
        _close(g1, gx.cuda(), tol, fro)
        x.grad = None
        fn(x).backward(dy)
        assert torch.equal(g1, x.grad)     # overlapping windows, no atomics: bitwise reproducible
    y, idx = cv.max_pool2d(x, k, s, p, return_indices=True)
    yr, ir = tF.max_pool2d(x.detach().float(), k, s, p, return_indices=True)
    assert torch.equal(idx, ir)


def test_conv_transpose2d():
    torch.manual_seed(3)
    x = torch.randn(2, 6, 7, 9, device="cuda", requires_grad=True)
    w = (torch.randn(6, 4, 3, 3, device="cuda") * 0.2).requires_grad_(True)
    b = torch.randn(4, device="cuda", requires_grad=True)
    y = cv.conv_transpose2d(x, w, b, 2, 1)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr, (gx, gw, gb) = _ref(lambda a, c, e: tF.conv_transpose2d(a, c, e, 2, 1), (x, w, b), dy)
    _close(y, yr.cuda(), 1e-4, 1e-5)
    _close(x.grad, gx.cuda(), 1e-4, 1e-5)
    _close(w.grad, gw.cuda(), 1e-4, 1e-5)
    _close(b.grad, gb.cuda(), 1e-4, 1e-5)


def test_layers_use_native_kernels():
    from momijo_b200 import _C
    from momijo_b200.learn.nn.conv import Conv2d, MaxPool2d

    conv = Conv2d(3, 8, 3, pad=(1, 1)).cuda()
    pool = MaxPool2d(2, stride=(2, 2))
    before = _C.launches
    y = pool(conv(torch.randn(2, 3, 16, 16, device="cuda")))
    y.sum().backward()
    assert _C.launches - before >= 5
    assert conv.weight.grad is not None and y.shape == (2, 8, 8, 8)
