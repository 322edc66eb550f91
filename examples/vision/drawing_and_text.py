"""Drawing primitives and bitmap text on an image
(legacy/examples/vision/drawing_and_text.mojo)."""
import momijo.vision as V


def main():
    img = V.Image.new_hwc_u8(120, 200, 3, 0)
    V.line(img, 10, 10, 190, 10, (255, 0, 0), 1)
    V.rectangle(img, 20, 30, 80, 70, (0, 255, 0), 2)
    V.rectangle(img, 100, 30, 140, 70, (0, 0, 255), -1)        # filled
    V.circle(img, 170, 50, 15, (255, 255, 0), -1)
    V.arrowed_line(img, 20, 100, 100, 100, (255, 255, 255), 1)
    V.fill_poly(img, [(120, 80), (160, 80), (140, 110)], (0, 255, 255))
    V.put_text(img, "momijo", 20, 90, 0, 1.0, (255, 255, 255))
    d = img.data
    assert [int(v) for v in d[10, 100]] == [255, 0, 0]            # on the line
    assert [int(v) for v in d[50, 120]] == [0, 0, 255]            # inside the filled rectangle
    assert [int(v) for v in d[50, 50]] == [0, 0, 0]               # inside the outlined rectangle
    assert [int(v) for v in d[50, 170]] == [255, 255, 0]          # centre of the disc
    assert int((d.sum(-1) > 0).sum()) > 2000
    V.write_image("drawing.png", img)
    back = V.read_image("drawing.png")
    assert tuple(back.shape) == tuple(img.shape) and int((back.data != d).sum()) == 0
    print("drawn pixels:", int((d.sum(-1) > 0).sum()))
    return img


if __name__ == "__main__":
    main()
