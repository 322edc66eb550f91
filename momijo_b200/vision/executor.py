"""Run an IR graph on an image (legacy/src/momijo/vision/executor.mojo:75-113): optimise, then walk the
nodes in order through the kernel registry. With a CUDA registry every node is one launch on the
current stream and nothing synchronises until the caller reads the result."""
from __future__ import annotations

from .backend.registry import KernelRegistry, default_registry
from .image import ColorSpace, Image
from .ir import Graph, OpKind, optimize


def run_graph(g: Graph, img: Image, registry: KernelRegistry = None, do_optimize: bool = True) -> Image:
    reg = registry or default_registry()
    if do_optimize:
        g = optimize(g.copy())
    t = reg.place(img.ensure_packed_hwc_u8().data)
    meta = img.meta().copy()
    for n in g.nodes():
        k = n.kind()
        if k == OpKind.ResizeNearest:
            t = reg.run("resize_nearest", t, n.oh(), n.ow())
        elif k == OpKind.ResizeBilinear:
            t = reg.run("resize_bilinear", t, n.oh(), n.ow())
        elif k == OpKind.ConvertRGBToGray:
            if t.shape[2] >= 3:
                t = reg.run("rgb_to_gray", t)
                meta = meta.with_colorspace(ColorSpace("GRAY"))
        elif k == OpKind.GaussianBlur:
            t = reg.run("gaussian", t, n.oh())
        elif k == OpKind.Erode:
            t = reg.run("erode", t, n.oh())
        elif k == OpKind.Dilate:
            t = reg.run("dilate", t, n.oh())
        elif k == OpKind.SwapRB:
            t = reg.run("swap_rb", t)
        else:
            raise ValueError(f"unknown op kind {k}")
    return Image(t, meta)
