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


def export_onnx_lite(model, path=None, input_name: str = "input", *ref_args) -> str:
    """``export_onnx_lite(model, path=None, input_name="input")``. The reference's forms
    ``(model, input_shape, input_name="x", output_name="y", opset=17)`` and the same with a ``path`` after the shape
    (legacy/src/momijo/learn/api/onnx_lite.mojo:52-94) are recognised by the list-valued second argument: the document
    then also carries ``opset``, the input shape and the requested output name."""
    if isinstance(path, (list, tuple)):
        shape, rest = list(path), [input_name] + list(ref_args) if input_name != "input" or ref_args else list(ref_args)
        out_path = None
        if rest and isinstance(rest[0], str) and (len(rest) >= 4 or "/" in rest[0] or rest[0].endswith(".json")):
            out_path, rest = rest[0], rest[1:]
        in_name = rest[0] if len(rest) > 0 else "x"
        out_name = rest[1] if len(rest) > 1 else "y"
        opset = rest[2] if len(rest) > 2 else 17
        body = export_onnx_lite(model, None, in_name)
        doc = body[:-1] + ',"opset":%d,"input_shape":%s,"output_name":"%s"}' % (opset, shape, out_name)
        if out_path is not None:
            with open(out_path, "w") as f:
                f.write(doc)
        return doc
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
