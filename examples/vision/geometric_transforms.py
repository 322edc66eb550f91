"""Translation, rotation about the centre, affine and perspective warps, flips
(legacy/examples/vision/geometric_transforms.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(80, 100, 1, 0)
    V.rectangle(img, 30, 20, 60, 50, (255,), -1)
    moved = V.translate(img, 10, 5)
    assert int(moved.data[30, 50, 0]) == 255 and int(moved.data[22, 35, 0]) == 0
    half_turn = V.rotate(img, 180.0)
    assert int(half_turn.data[80 - 1 - 35, 100 - 1 - 45, 0]) == 255
    assert tuple(V.rotate90(img, 1).shape[:2]) == (100, 80)
    ident = V.affine(img, [[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]])
    assert int((ident.data != img.data).sum()) == 0
    scaled = V.affine(img, [[2.0, 0.0, 0.0], [0.0, 2.0, 0.0]])
    assert int(scaled.data[70, 90, 0]) == 255               # (45, 35) doubled
    persp = V.perspective(img, [[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]])
    assert int((persp.data != img.data).sum()) == 0
    assert int(V.flip(img, 0).data[80 - 1 - 35, 45, 0]) == 255
    print(moved.shape, half_turn.shape, scaled.shape)
    return moved


if __name__ == "__main__":
    main()
