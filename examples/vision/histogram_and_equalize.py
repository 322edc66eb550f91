"""Grey-level histogram, global equalisation, CLAHE on colour and a plotted histogram
(mirrors legacy/examples/vision/histogram_and_equalize.mojo)."""
import torch

import momijo.vision as V


def main():
    ramp = torch.linspace(60, 120, 64).to(torch.uint8).view(1, 64, 1).expand(48, 64, 1).contiguous()
    gray = V.Image(ramp)
    hist = V.histogram(gray)
    eq = V.equalize_hist(gray)
    colour = V.clahe_color_bgr(V.gray_to_bgr(gray), 2.0, 8)
    plot = V.plot_hist_u8(V.histogram(eq))
    spread_before = int(gray.data.max()) - int(gray.data.min())
    spread_after = int(eq.data.max()) - int(eq.data.min())
    print("levels used:", sum(1 for h in hist if h), "spread", spread_before, "->", spread_after, colour.shape, plot.shape)
    assert sum(hist) == 48 * 64 and spread_after > spread_before
    return eq


if __name__ == "__main__":
    main()
