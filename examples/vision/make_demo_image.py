"""Synthesise the test card the other demos start from: gradient background, filled shapes, lines and text
(mirrors legacy/examples/vision/make_demo_image.mojo and drawing_and_text.mojo)."""
import torch

import momijo.vision as V


def make_card(h: int = 120, w: int = 160) -> "V.Image":
    ramp = torch.linspace(0, 200, w).to(torch.uint8).view(1, w, 1).expand(h, w, 3).contiguous()
    img = V.Image(ramp)
    V.rectangle(img, 10, 10, 60, 50, (255, 255, 255), -1)
    V.circle(img, 110, 40, 22, (0, 200, 255), -1)
    V.line(img, 0, h - 1, w - 1, 60, (255, 0, 0), 2)
    V.arrowed_line(img, 20, 100, 90, 80, (0, 255, 0), 1)
    V.put_text(img, "B200", 70, 105, scale=2, color=(255, 255, 0))
    return img


def main():
    img = make_card()
    assert V.write_image("card.png", img) and V.write_ppm("card.ppm", img)
    back = V.read_image("card.png")
    print("card", img.shape, "round trip equal:", bool((back.data == img.data).all()))
    assert bool((back.data == img.data).all()) and bool((V.read_ppm("card.ppm").data == img.data).all())
    return img


if __name__ == "__main__":
    main()
