"""Graph rewrites (legacy/src/momijo/vision/ir/fusion.mojo:42-107)."""
from __future__ import annotations

from .ir import Graph, OpKind, OpNode


def fuse_resizes(g: Graph) -> None:
    """Keep only the last nearest-resize, at its own position: nearest sampling of nearest sampling
    lands on the final grid, so the intermediate sizes never need to be materialised. (Exact when every
    intermediate size is a multiple of the previous one; the reference applies it unconditionally.)"""
    last = g.last_index_of_resize()
    if last < 0:
        return
    g.set_nodes([n for i, n in enumerate(g.nodes()) if n.kind() != OpKind.ResizeNearest or i == last])


def simplify_convert_color(g: Graph) -> None:
    """Drop a grey conversion that directly follows another one."""
    out, prev_gray = [], False
    for n in g.nodes():
        if n.kind() == OpKind.ConvertRGBToGray:
            if not prev_gray:
                out.append(n)
            prev_gray = True
        else:
            out.append(n)
            prev_gray = False
    g.set_nodes(out)


def hoist_gray_before_resize(g: Graph) -> None:
    """Grey conversion commutes with nearest resize; converting first makes the resize move a third of
    the bytes. (No counterpart in the reference's pass list.)"""
    nodes = g.nodes()
    changed = True
    while changed:
        changed = False
        for i in range(len(nodes) - 1):
            if nodes[i].kind() == OpKind.ResizeNearest and nodes[i + 1].kind() == OpKind.ConvertRGBToGray \
                    and nodes[i].oh() * nodes[i].ow() > 0:
                nodes[i], nodes[i + 1] = nodes[i + 1], nodes[i]
                changed = True
    g.set_nodes(nodes)


def optimize(g: Graph) -> Graph:
    fuse_resizes(g)
    simplify_convert_color(g)
    return g
