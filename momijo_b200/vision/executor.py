"""Run an IR graph on an image (legacy/src/momijo/vision/executor.mojo:75-113): optimise, then walk the
nodes in order through the kernel registry. With a CUDA registry every node is one launch on the
current stream and nothing synchronises until the caller reads the result."""
from __future__ import annotations

from .backend.registry import KernelRegistry, default_registry
from .image import ColorSpace, Image
from .ir import Graph, OpKind, OpNode, optimize


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


def run_graph_no_fuse(g: Graph, img: Image, registry: KernelRegistry = None) -> Image:
    """Every node as written, no fusion or simplification pass first
    (legacy/src/momijo/vision/executor.mojo:91-99)."""
    return run_graph(g, img, registry, do_optimize=False)


def run_single_op(kind, img: Image, oh: int = 0, ow: int = 0, registry: KernelRegistry = None) -> Image:
    """One op by kind; kinds that need no size ignore ``oh`` / ``ow``, unknown kinds pass the image through
    (legacy/src/momijo/vision/executor.mojo:103-113)."""
    try:
        kind = OpKind(kind)
    except ValueError:
        return img.clone()
    if kind == OpKind.ConvertRGBToGray and img.channels() != 3:
        return img.clone()
    g = Graph([OpNode(kind, oh, ow)])
    return run_graph(g, img, registry, do_optimize=False)
