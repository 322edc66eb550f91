"""Draw shapes, blur, detect edges and contours, write a PNG (legacy/examples/vision/ has 12 demos of
this kind). Runs on the GPU kernels when the image is moved there with ``img.cuda()``."""
import os
import tempfile

import momijo.vision as V


def main(out_dir: str = None):
    img = V.Image.new_hwc_u8(128, 160, 3, 0)
    V.rectangle(img, 20, 20, 70, 90, (255, 255, 255), -1)
    V.circle(img, 115, 64, 25, (0, 255, 0), -1)
    V.put_text(img, "MOMIJO", 24, 118, scale=2, color=(255, 128, 0))
    gray = V.bgr_to_gray(V.gaussian_blur(img, 5, 1.2))
    edges = V.canny(gray, 40, 120)
    contours = V.find_contours(V.threshold_otsu(gray), external_only=True)
    canvas = V.draw_contours(img.clone(), contours, -1, (0, 0, 255), 1)
    out_dir = out_dir or tempfile.mkdtemp()
    path = os.path.join(out_dir, "contours.png")
    assert V.write_image(path, canvas)
    back = V.read_image(path)
    print("contours:", V.len_contours(contours), "edge pixels:", int((edges.numpy() > 0).sum()), "wrote", path, back.shape)
    return len(contours)


if __name__ == "__main__":
    main()
