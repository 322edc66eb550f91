"""Weighted blends and masked bitwise operations (mirrors legacy/examples/vision/blending_bitwise.mojo)."""
import momijo.vision as V


def main():
    a = V.Image.new_hwc_u8(32, 32, 3, 200)
    b = V.Image.new_hwc_u8(32, 32, 3, 100)
    mask = V.Image.new_hwc_u8(32, 32, 1, 0)
    V.circle(mask, 16, 16, 8, (255,), -1)
    mix = V.add_weighted(a, 0.25, b, 0.75, 0.0)
    cut = V.bitwise_and(a, a, mask)
    inv = V.bitwise_not(a)
    either = V.bitwise_or(cut, b)
    print("blend value:", int(mix.data[0, 0, 0]), "kept pixels:", int((cut.data[..., 0] > 0).sum()), "inverse:", int(inv.data[0, 0, 0]), either.shape)
    assert int(mix.data[0, 0, 0]) == 125 and int(inv.data[0, 0, 0]) == 55 and int(cut.data[0, 0, 0]) == 0 and int(cut.data[16, 16, 0]) == 200
    return mix


if __name__ == "__main__":
    main()
