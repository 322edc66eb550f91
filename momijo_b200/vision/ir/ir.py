"""A small linear IR for image pipelines (legacy/src/momijo/vision/ir/ir.mojo:12-122). The reference
knows two ops, ``ResizeNearest`` and ``ConvertRGBToGray``; the same two keep their numeric ids here and
a few more pixel ops ride along so that a whole preprocessing chain can be queued on one stream."""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import List


class NodeId:
    def __init__(self, id: int):
        self._id = int(id)

    def id(self) -> int:
        return self._id


class OpKind(IntEnum):
    ResizeNearest = 0
    ConvertRGBToGray = 1
    ResizeBilinear = 2
    GaussianBlur = 3
    Erode = 4
    Dilate = 5
    SwapRB = 6


@dataclass
class OpNode:
    _kind: OpKind
    _oh: int = 0
    _ow: int = 0

    def kind(self) -> OpKind:
        return self._kind

    def oh(self) -> int:
        return self._oh

    def ow(self) -> int:
        return self._ow


class Graph:
    def __init__(self, nodes: List[OpNode] = None):
        self._nodes: List[OpNode] = list(nodes or [])

    def add_node(self, node: OpNode):
        self._nodes.append(node)

    def node_count(self) -> int:
        return len(self._nodes)

    def node_at(self, i: int) -> OpNode:
        return self._nodes[i]

    def nodes(self) -> List[OpNode]:
        return list(self._nodes)

    def clear(self):
        self._nodes = []

    def set_nodes(self, nodes: List[OpNode]):
        self._nodes = list(nodes)

    def append_resize(self, oh: int, ow: int):
        self.add_node(OpNode(OpKind.ResizeNearest, oh, ow))

    def append_resize_bilinear(self, oh: int, ow: int):
        self.add_node(OpNode(OpKind.ResizeBilinear, oh, ow))

    def append_rgb_to_gray(self):
        self.add_node(OpNode(OpKind.ConvertRGBToGray, 0, 0))

    def append_gaussian(self, ksize: int):
        self.add_node(OpNode(OpKind.GaussianBlur, ksize, ksize))

    def append_erode(self, ksize: int):
        self.add_node(OpNode(OpKind.Erode, ksize, ksize))

    def append_dilate(self, ksize: int):
        self.add_node(OpNode(OpKind.Dilate, ksize, ksize))

    def append_swap_rb(self):
        self.add_node(OpNode(OpKind.SwapRB, 0, 0))

    def last_index_of_resize(self) -> int:
        for i in range(len(self._nodes) - 1, -1, -1):
            if self._nodes[i]._kind == OpKind.ResizeNearest:
                return i
        return -1

    def copy(self) -> "Graph":
        return Graph(self._nodes)


def Graph_add_node(g: Graph, node: OpNode):
    g.add_node(node)
