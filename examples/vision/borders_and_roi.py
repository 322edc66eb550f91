"""Border modes of copy_make_border and region-of-interest copies
(legacy/examples/vision/borders_and_roi.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(6, 8, 1, 0)
    for x in range(8):
        img.data[:, x, 0] = 10 * (x + 1)
    const = V.copy_make_border(img, 1, 1, 2, 2, V.BORDER_CONSTANT(), 7)
    repl = V.copy_make_border(img, 1, 1, 2, 2, V.BORDER_REPLICATE())
    refl = V.copy_make_border(img, 1, 1, 2, 2, V.BORDER_REFLECT())
    assert tuple(const.shape[:2]) == (8, 12)
    assert int(const.data[0, 0, 0]) == 7 and int(const.data[1, 2, 0]) == 10
    assert [int(v) for v in repl.data[3, :4, 0]] == [10, 10, 10, 20]
    assert int(refl.data[3, 1, 0]) in (10, 20) and int(refl.data[3, 0, 0]) in (20, 30)
    roi = V.crop(img, 1, 2, 3, 4)             # y, x, height, width
    assert tuple(roi.shape[:2]) == (3, 4) and int(roi.data[0, 0, 0]) == 30
    roi.data[:] = 255                         # a crop is a copy: the source keeps its pixels
    assert int(img.data[1, 2, 0]) == 30
    print(const.shape, repl.shape, refl.shape, roi.shape)
    return const


if __name__ == "__main__":
    main()
