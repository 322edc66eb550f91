"""``export_onnx_lite``: a small JSON graph of Linear / ReLU chains
(legacy/src/momijo/learn/api/onnx_lite.mojo:52-117)."""
from __future__ import annotations

import json

from ..nn.layers import Linear, ReLU, LeakyReLU, Sigmoid, Tanh


def emit_onnx_lite(layer, in_name: str):
    """-> (node_json, out_name)."""
    if isinstance(layer, Linear):
        out = in_name + "_fc"
        node = {"op": "Gemm", "input": in_name, "output": out, "transB": 1,
                "W": {"shape": list(layer.weight.shape), "data": layer.weight.detach().float().reshape(-1).tolist()},
                "B": {"shape": list(layer.bias_t.shape), "data": layer.bias_t.detach().float().reshape(-1).tolist()}}
    else:
        op = {ReLU: "Relu", LeakyReLU: "LeakyRelu", Sigmoid: "Sigmoid", Tanh: "Tanh"}.get(type(layer), type(layer).__name__)
        out = in_name + "_" + op.lower()
        node = {"op": op, "input": in_name, "output": out}
    return json.dumps(node, separators=(",", ":")), out


def export_onnx_lite(model, path: str | None = None, input_name: str = "input") -> str:
    layers = model.to_list() if hasattr(model, "to_list") else [model]
    nodes, cur = [], input_name
    for l in layers:
        n, cur = emit_onnx_lite(l, cur)
        nodes.append(n)
    doc = '{"format":"onnx-lite","version":1,"input":"%s","output":"%s","nodes":[%s]}' % (
        input_name, cur, ",".join(nodes))
    if path is not None:
        with open(path, "w") as f:
            f.write(doc)
    return doc
