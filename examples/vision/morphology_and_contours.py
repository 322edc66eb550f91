"""Erode / dilate / open / close, connected components, contours with area and bounding box
(mirrors legacy/examples/vision/morphology_and_contours.mojo)."""
import momijo.vision as V


def main():
    bw = V.Image.new_hwc_u8(64, 64, 1, 0)
    V.rectangle(bw, 8, 8, 28, 28, (255,), -1)
    V.circle(bw, 46, 44, 9, (255,), -1)
    bw.data[2, 2, 0] = 255                                    # a speck that opening removes
    opened = V.morphology(bw, V.MORPH_OPEN(), 3)
    grown, shrunk = V.dilate(bw, 3), V.erode(bw, 3)
    n_before, _ = V.connected_components(bw)
    n_after, labels = V.connected_components(opened)
    contours = V.find_contours(opened, external_only=True)
    boxes = [V.bounding_rect(c) for c in contours]
    coloured = V.label_to_color_image(labels)
    print("components:", n_before, "->", n_after, "areas:", [V.contour_area(c) for c in contours], "boxes:", boxes, coloured.shape)
    assert n_before == n_after + 1 and len(contours) == 2 and int((grown.data > 0).sum()) > int((shrunk.data > 0).sum())
    return opened


if __name__ == "__main__":
    main()
