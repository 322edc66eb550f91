"""Smoothing filters, gradients, thresholds and Canny edges
(mirrors legacy/examples/vision/filters_threshold_edges.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(64, 64, 3, 20)
    V.rectangle(img, 16, 16, 48, 48, (220, 220, 220), -1)
    gray = V.bgr_to_gray(img)
    smooth = V.gaussian_blur(gray, 5, 5, 1.0)
    med = V.median_blur(gray, 3)
    gx, lap = V.sobel(gray, 1, 0), V.laplacian(gray)
    fixed, otsu = V.threshold_binary(gray, 128), V.threshold_otsu(gray)
    local = V.adaptive_threshold(gray, 255, 0, 11, 2)
    edges = V.canny(smooth, 40, 120)
    n_edge = int((edges.data > 0).sum())
    print("edge pixels:", n_edge, "white after otsu:", int((otsu.data > 0).sum()), med.shape, gx.shape, lap.shape, local.shape)
    assert bool((fixed.data == otsu.data).all()) and 80 < n_edge < 400
    return edges


if __name__ == "__main__":
    main()
