"""Vision package on the host path: codecs round-trip, kernels against direct restatements, IR passes."""
import math
import os

import numpy as np
import pytest
import torch

import momijo_b200.vision as V
from momijo_b200.vision import kernels as K


def _img(h=37, w=53, c=3, seed=0):
    rng = np.random.default_rng(seed)
    return V.Image.from_numpy(rng.integers(0, 256, (h, w, c), dtype=np.uint8))


def test_codecs_roundtrip(tmp_path):
    img = _img()
    for ext in ("png", "ppm"):
        p = str(tmp_path / f"x.{ext}")
        assert V.write_image(p, img)
        ok, back = V.read_image_any(p)
        assert ok and np.array_equal(back.numpy(), img.numpy())
    gray = V.rgb_to_gray(img)
    p = str(tmp_path / "g.png")
    assert V.write_png(p, gray) and np.array_equal(V.read_png(p).numpy(), gray.numpy())
    smooth = V.gaussian_blur(V.resize(img, 96, 80), 7, 2.0)
    p = str(tmp_path / "s.jpg")
    assert V.write_image(p, smooth, quality=92)
    back = V.read_image(p)
    assert back.shape == smooth.shape
    assert np.abs(back.numpy().astype(int) - smooth.numpy().astype(int)).mean() < 3.0
    ok, bad = V.read_image_any(str(tmp_path / "missing.png"))
    assert not ok and bad.shape == (1, 1, 1)


def test_png_filters_decode():
    # every scanline filter type, written by hand
    import struct, zlib
    from momijo_b200.vision.io.png import _chunk, _SIG, decode_png
    rng = np.random.default_rng(1)
    a = rng.integers(0, 256, (5, 4, 3), dtype=np.uint8)
    rows = a.reshape(5, 12).astype(int)
    raw = bytearray()
    prev = np.zeros(12, dtype=int)
    for y, ft in enumerate([0, 1, 2, 3, 4]):
        cur = rows[y]
        out = np.zeros(12, dtype=int)
        for i in range(12):
            left = cur[i - 3] if i >= 3 else 0
            up = prev[i]
            ul = prev[i - 3] if i >= 3 else 0
            if ft == 0: pred = 0
            elif ft == 1: pred = left
            elif ft == 2: pred = up
            elif ft == 3: pred = (left + up) // 2
            else:
                p = left + up - ul
                pa, pb, pc = abs(p - left), abs(p - up), abs(p - ul)
                pred = left if (pa <= pb and pa <= pc) else (up if pb <= pc else ul)
            out[i] = (cur[i] - pred) & 255
        raw.append(ft)
        raw += bytes(int(v) for v in out)
        prev = cur
    png = _SIG + _chunk(b"IHDR", struct.pack(">IIBBBBB", 4, 5, 8, 2, 0, 0, 0)) + \
        _chunk(b"IDAT", zlib.compress(bytes(raw))) + _chunk(b"IEND", b"")
    assert np.array_equal(decode_png(png), a)


def test_resize_and_gray_formulas():
    img = _img()
    a = img.numpy()
    out = V.resize_nearest(img, 20, 31).numpy()
    for y in (0, 7, 19):
        for x in (0, 11, 30):
            sy, sx = min(int(y * (37 / 20)), 36), min(int(x * (53 / 31)), 52)
            assert np.array_equal(out[y, x], a[sy, sx])
    g = V.rgb_to_gray(img).numpy()[..., 0]
    ref = (a[..., 0].astype(int) * 299 + a[..., 1].astype(int) * 587 + a[..., 2].astype(int) * 114) // 1000
    assert np.array_equal(g, ref)
    assert np.array_equal(V.bgr_to_rgb(img).numpy(), a[..., ::-1])
    up = V.resize(img, 106, 74).numpy()
    assert up.shape == (74, 106, 3) and abs(up.mean() - a.mean()) < 3


def test_gaussian_and_morph_match_loops():
    img = _img(9, 11, 1)
    a = img.numpy()[..., 0].astype(float)
    taps = K.gaussian_taps(5, 1.1)
    tmp = np.zeros_like(a)
    for y in range(9):
        for x in range(11):
            tmp[y, x] = int(min(max(sum(taps[k + 2] * a[y, min(max(x + k, 0), 10)] for k in range(-2, 3)), 0), 255) + 0.5)
    ref = np.zeros_like(a)
    for y in range(9):
        for x in range(11):
            ref[y, x] = int(min(max(sum(taps[k + 2] * tmp[min(max(y + k, 0), 8), x] for k in range(-2, 3)), 0), 255) + 0.5)
    got = V.gaussian_blur(img, 5, 1.1).numpy()[..., 0]
    assert np.abs(got.astype(int) - ref.astype(int)).max() <= 1
    er = V.erode(img, 3).numpy()[..., 0]
    di = V.dilate(img, 3).numpy()[..., 0]
    ai = img.numpy()[..., 0]
    for y, x in ((0, 0), (4, 5), (8, 10)):
        win = ai[max(y - 1, 0):y + 2, max(x - 1, 0):x + 2]
        assert er[y, x] == win.min() and di[y, x] == win.max()


def test_warps_and_borders():
    img = _img(16, 20, 3)
    a = img.numpy()
    t = V.translate(img, 3, 2).numpy()
    assert np.array_equal(t[2:, 3:], a[:-2, :-3]) and t[:2].sum() == 0
    assert np.array_equal(V.translate(img, 3, 0, V.BORDER_REPLICATE()).numpy()[:, 0], a[:, 0])
    assert np.array_equal(V.flip(img, 1).numpy(), a[:, ::-1])
    assert np.array_equal(V.rotate90(img, 1).numpy(), np.rot90(a, 1))
    assert np.array_equal(V.rotate(img, 180).numpy(), np.rot90(a, 2))
    ident = V.perspective(img, [(0, 0), (19, 0), (19, 15), (0, 15)], [(0, 0), (19, 0), (19, 15), (0, 15)])
    assert np.array_equal(ident.numpy(), a)
    b = V.copy_make_border(img, 1, 2, 3, 4, V.BORDER_REFLECT())
    assert b.shape == (19, 27, 3)


def test_threshold_hist_equalize():
    img = V.rgb_to_gray(_img(40, 40, 3))
    h = V.histogram(img)
    assert sum(h) == 1600 and len(V.histogram(img, 16)) == 16
    tb = V.threshold_binary(img, 100).numpy()
    assert set(np.unique(tb)) <= {0, 255} and ((img.numpy() > 100) == (tb == 255)).all()
    assert set(np.unique(V.threshold_otsu(img).numpy())) <= {0, 255}
    assert V.adaptive_threshold(img, 255, 0, 11, 2).shape == img.shape
    eq = V.equalize_hist(img)
    assert eq.numpy().max() == 255
    assert V.plot_hist_u8(h).shape == (200, 256, 1)


def test_shapes_features_drawing():
    c = V.Image.new_hwc_u8(64, 64, 1)
    V.rectangle(c, 10, 10, 30, 30, [255], -1)
    V.circle(c, 48, 48, 8, [255], -1)
    n, labels = V.connected_components(c)
    assert n == 2
    cs = V.find_contours(c, external_only=True)
    assert V.len_contours(cs) == 2
    x, y, w, h = V.bounding_rect(cs[0])
    assert (x, y, w, h) == (10, 10, 21, 21)
    assert abs(V.contour_area(cs[0]) - 400) < 1e-6
    assert abs(V.arc_length([(0, 0), (3, 4)], False) - 5.0) < 1e-9
    edges = V.canny(c, 50, 150)
    assert edges.numpy().max() == 255
    circ = V.hough_circles(V.circle(V.Image.new_hwc_u8(64, 64, 1), 32, 32, 12, [255], 1), 1.0, 20, 100.0, 20.0, 8, 16)
    assert circ and abs(circ[0][0] - 32) <= 2 and abs(circ[0][2] - 12) <= 2
    lines = V.hough_lines_p(V.line(V.Image.new_hwc_u8(64, 64, 1), 5, 5, 60, 50, [255]), 1, math.pi / 180, 30, 10, 2)
    assert lines
    img = V.resize(_img(), 160, 160)
    k, d = V.orb_detect_and_compute(img, 100)
    assert V.len_keypoints(k) <= 100 and V.valid_descriptors(d)
    m = V.bf_match_hamming(d, d)
    assert all(a == b and dist == 0 for a, b, dist in m)
    assert len(V.top_k_matches(m, 5)) == 5
    canvas = V.draw_matches(img, k, img, k, m[:10])
    assert canvas.shape == (160, 320, 3)
    assert V.label_to_color(3) == (0, 0, 255)


def test_bitwise_and_blend():
    a, b = _img(8, 8, 3, 1), _img(8, 8, 3, 2)
    assert np.array_equal(V.bitwise_and(a, b).numpy(), a.numpy() & b.numpy())
    assert np.array_equal(V.bitwise_not(a).numpy(), ~a.numpy())
    w = V.add_weighted(a, 0.5, b, 0.5, 0).numpy().astype(int)
    assert np.abs(w - (a.numpy().astype(int) + b.numpy().astype(int)) / 2).max() <= 1


def test_ir_passes_and_executor():
    g = V.Graph()
    g.append_resize(64, 64)
    g.append_rgb_to_gray()
    g.append_rgb_to_gray()
    g.append_resize(32, 32)
    V.fuse_resizes(g)
    V.simplify_convert_color(g)
    assert [n.kind() for n in g.nodes()] == [V.OpKind.ConvertRGBToGray, V.OpKind.ResizeNearest]
    out = V.run_graph(g, _img(), V.KernelRegistry(V.BackendKind.CPUSIMD))
    assert out.shape == (32, 32, 1)


def test_image_accessors_and_alpha():
    img = V.Image.new_hwc_u8(4, 5, 4, 200)
    img.set_u8(1, 2, 3, 128)
    assert img.get_u8(1, 2, 3) == 128 and img.get_u8(9, 9, 0) == 0
    pm = img.premultiply_alpha()
    assert pm.meta().is_premultiplied() and pm.get_u8(1, 2, 0) == (200 * 128 + 127) // 255
    assert abs(pm.unpremultiply_alpha().get_u8(1, 2, 0) - 200) <= 1
    roi = img.roi(1, 1, 10, 10)
    assert roi.shape == (3, 4, 4)
    assert V.wait_key(0) == -1
