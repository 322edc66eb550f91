"""Resize (nearest / bilinear), crop, flips, quarter turns, free rotation, affine and perspective warps, borders
(mirrors legacy/examples/vision/resize_crop_rotate_flip.mojo, geometric_transforms.mojo and borders_and_roi.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(60, 80, 3, 0)
    V.rectangle(img, 10, 10, 40, 30, (255, 255, 255), -1)
    small = V.resize(img, 40, 30)
    near = V.resize(img, 160, 120, V.INTER_NEAREST())
    roi = V.crop(img, 5, 5, 30, 40)
    turned = V.rotate90(img, 1)
    mirrored = V.flip(img, 1)
    spun = V.rotate(img, 30.0)
    sheared = V.affine(img, [[1.0, 0.2, 0.0], [0.0, 1.0, 0.0]])
    framed = V.copy_make_border(img, 4, 4, 6, 6, V.BORDER_REFLECT())
    print(small.shape, near.shape, roi.shape, turned.shape, mirrored.shape, spun.shape, sheared.shape, framed.shape)
    assert tuple(small.shape[:2]) == (30, 40) and tuple(turned.shape[:2]) == (80, 60) and tuple(framed.shape[:2]) == (68, 92)
    assert int(mirrored.data[15, 80 - 1 - 20, 0]) == 255 and int(roi.data[10, 10, 0]) == 255
    return framed


if __name__ == "__main__":
    main()
