"""Probabilistic Hough segments and Hough circles on a synthetic drawing
(mirrors legacy/examples/vision/hough_detections.mojo)."""
import math

import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(96, 128, 1, 0)
    V.line(img, 10, 20, 110, 20, (255,), 1)
    V.line(img, 30, 30, 30, 90, (255,), 1)
    V.circle(img, 84, 62, 18, (255,), 1)
    segs = V.hough_lines_p(img, 1.0, math.pi / 180.0, 30, 30, 3)
    circles = V.hough_circles(img, dp=1.0, min_dist=20, param1=100.0, param2=12.0, min_r=10, max_r=30)
    canvas = V.draw_circles(V.draw_lines_p(V.gray_to_bgr(img), segs), circles)
    print("segments:", len(segs), "circles:", circles[:3], canvas.shape)
    assert len(segs) >= 2 and canvas.shape[2] == 3
    return canvas


if __name__ == "__main__":
    main()
