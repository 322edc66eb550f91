"""Codecs and colour conversions: PNG / JPEG / PPM files, in-memory encode / decode, BGR <-> grey
(mirrors legacy/examples/vision/io_colors.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(24, 32, 3, 0)
    V.rectangle(img, 4, 4, 20, 16, (10, 200, 90), -1)
    assert V.write_png("a.png", img) and V.write_jpeg("a.jpg", img, 95) and V.write_ppm("a.ppm", img)
    png, jpg, ppm = V.read_png("a.png"), V.read_jpeg("a.jpg"), V.read_ppm("a.ppm")
    blob = V.encode_image(img, "png")
    again = V.decode_image(blob)
    gray = V.bgr_to_gray(img)
    err = (jpg.data.int() - img.data.int()).abs().float().mean().item()
    print("png exact:", bool((png.data == img.data).all()), "jpeg mean abs error:", round(err, 2), "png bytes:", len(blob), gray.shape)
    assert bool((png.data == img.data).all()) and bool((ppm.data == img.data).all()) and bool((again.data == img.data).all()) and err < 6.0
    return gray


if __name__ == "__main__":
    main()
