from .fusion import fuse_resizes, hoist_gray_before_resize, optimize, simplify_convert_color  # noqa: F401
from .ir import Graph, Graph_add_node, NodeId, OpKind, OpNode  # noqa: F401
