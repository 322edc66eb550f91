"""CUDA pixel kernels against the host restatement of the same arithmetic."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _img(h, w, c, seed=0):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.integers(0, 256, (h, w, c), dtype=np.uint8))


def _close(a, b, tol=0):
    d = (a.cpu().to(torch.int16) - b.cpu().to(torch.int16)).abs().max().item()
    assert d <= tol, d


def test_vision_kernels_match_host():
    from momijo_b200.vision import kernels as K
    src = _img(241, 317, 3)
    dev = src.cuda()
    _close(K.resize(dev, 100, 150, False), K.resize(src, 100, 150, False))
    _close(K.resize(dev, 480, 600, False), K.resize(src, 480, 600, False))
    _close(K.resize(dev, 100, 150, True), K.resize(src, 100, 150, True), 1)
    _close(K.resize(dev, 480, 600, True), K.resize(src, 480, 600, True), 1)
    _close(K.to_gray(dev, False), K.to_gray(src, False))
    _close(K.to_gray(dev, True), K.to_gray(src, True))
    _close(K.swap_rb(dev), K.swap_rb(src))
    _close(K.gaussian_blur(dev, 7, 5, 1.5), K.gaussian_blur(src, 7, 5, 1.5), 1)
    g, gd = K.to_gray(src), K.to_gray(dev)
    for mode in range(4):
        _close(K.deriv3(gd, mode), K.deriv3(g, mode), 1 if mode == 3 else 0)
    for k in (3, 5):
        _close(K.morph(dev, k, False), K.morph(src, k, False))
        _close(K.morph(dev, k, True), K.morph(src, k, True))
    import math
    t = math.radians(17.0)
    inv = [math.cos(t), math.sin(t), -20.0, -math.sin(t), math.cos(t), 35.0, 0, 0, 1]
    for border in (0, 1, 2):
        _close(K.warp(dev, inv, False, border, 7), K.warp(src, inv, False, border, 7))
    hinv = [1.0, 0.05, -3.0, 0.02, 0.98, 4.0, 1e-4, -2e-4, 1.0]
    _close(K.warp(dev, hinv, True, 0, 0), K.warp(src, hinv, True, 0, 0))
    assert torch.equal(K.histogram(gd).cpu(), K.histogram(g))
    lut = np.arange(255, -1, -1, dtype=np.uint8)
    _close(K.apply_lut(dev, lut), K.apply_lut(src, lut))
    other = _img(241, 317, 3, 1)
    for op in (K.OP_AND, K.OP_OR):
        _close(K.binary(dev, other.cuda(), op), K.binary(src, other, op))
    _close(K.binary(dev, None, K.OP_NOT), K.binary(src, None, K.OP_NOT))
    _close(K.binary(dev, other.cuda(), K.OP_WEIGHTED, 0.3, 0.6, 4.0), K.binary(src, other, K.OP_WEIGHTED, 0.3, 0.6, 4.0), 1)


def test_vision_pipeline_on_device():
    import momijo_b200.vision as V
    img = V.Image(_img(480, 640, 3)).cuda()
    g = V.Graph()
    g.append_resize(240, 320)
    g.append_rgb_to_gray()
    g.append_gaussian(5)
    out = V.run_graph(g, img)
    ref = V.run_graph(g, img.cpu(), V.KernelRegistry(V.BackendKind.CPUSIMD))
    assert out.device.type == "cuda" and out.shape == (240, 320, 1)
    _close(out.data, ref.data, 1)
    eq = V.equalize_hist(out)
    _close(eq.data, V.equalize_hist(ref).data, 0 if torch.equal(out.data.cpu(), ref.data) else 255)


def test_neighbourhood_and_region_kernels_match_host_transforms():
    """Median, bilateral, Canny (NMS + hysteresis), CLAHE and connected components: the CUDA kernels against
    the host implementations of the same transforms."""
    import momijo_b200.vision as V
    from momijo_b200.vision.transforms import filter as Fl, color as Cl, segmentation as Sg

    rng = np.random.default_rng(5)
    # a smooth image with structure (random noise alone makes every pixel an edge)
    yy, xx = np.mgrid[0:150, 0:201]
    base = (127 + 90 * np.sin(xx / 11.0) * np.cos(yy / 7.0)).astype(np.float32)
    img = np.clip(base[..., None] + rng.normal(0, 6, (150, 201, 3)), 0, 255).astype(np.uint8)
    host = V.Image(torch.from_numpy(img))
    dev = host.cuda()
    for k in (3, 5):
        _close(Fl.median_blur(dev, k).data, Fl.median_blur(host, k).data)
    _close(Fl.bilateral_filter(dev, 5, 30.0, 3.0).data, Fl.bilateral_filter(host, 5, 30.0, 3.0).data, 1)
    a, b = Fl.canny(dev, 60, 150).data.cpu(), Fl.canny(host, 60, 150).data
    assert a.shape == b.shape and (a != b).sum().item() == 0, (a != b).sum().item()
    assert 0 < (b > 0).sum().item() < b.numel() // 2
    _close(Cl.clahe_color_bgr(dev, 2.0, 8).data, Cl.clahe_color_bgr(host, 2.0, 8).data, 1)
    gray = V.Image(torch.from_numpy(img[..., :1].copy()))
    _close(Cl.clahe_color_bgr(gray.cuda(), 3.0, 4).data, Cl.clahe_color_bgr(gray, 3.0, 4).data, 1)
    bw = (rng.random((90, 120)) < 0.45).astype(np.uint8) * 255
    bimg = V.Image(torch.from_numpy(bw[..., None].copy()))
    for conn in (4, 8):
        n_d, l_d = Sg.connected_components(bimg.cuda(), conn)
        n_h, l_h = Sg.connected_components(bimg, conn)
        assert n_d == n_h and l_d == l_h
