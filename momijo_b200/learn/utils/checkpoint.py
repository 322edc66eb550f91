"""MNP checkpoints (legacy/src/momijo/learn/utils/checkpoint.mojo).

Layout A, ``save_state_dict(model, P)`` (checkpoint.mojo:250-277):
  ``P.json``        header ``{"format":"MNP","version":1,"created_at":"1970-01-01T00:00:00Z",
                    "model_class":"Model","files":{"state":...,"blob":...},"blob_meta":{...}}``
  ``P.state.json``  the model's state JSON (dotted names -> tensor summaries)
  ``P.bin``         named by the reference but never written; here it holds the real
                    little-endian tensor data and the header gains ``blob_meta.total_elems`` /
                    ``dtype`` plus a ``"tensors"`` index and an ``"extra"`` object (optimizer /
                    scaler / RNG / step). A version-1 reader ignores the added keys because it
                    extracts fields by substring search.
Layout B, ``make_checkpoint`` / ``apply_checkpoint`` (checkpoint.mojo:19-154): header
``{"params":[{"type":"Linear","w":nW,"b":nB},...]}`` + one flat Float32 vector (weight then bias
per Linear / Conv2d layer in traversal order); apply copies by position.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Optional

import torch
import torch.nn as nn

from ... import _C

_DT = {torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16",
       torch.float64: "float64", torch.int64: "int64", torch.int32: "int32", torch.int8: "int8",
       torch.uint8: "uint8", torch.bool: "bool"}
_DT_INV = {v: k for k, v in _DT.items()}


def _now_iso8601() -> str:
    return "1970-01-01T00:00:00Z"  # deterministic, as in the reference (checkpoint.mojo:178-180)


def _escape_json_string(s: str) -> str:
    return s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n").replace("\t", "\\t")


def _header_path(base):
    return base + ".json"


def _state_path(base):
    return base + ".state.json"


def _blob_path(base):
    return base + ".bin"


def _write_text(p, s):
    try:
        with open(p, "w") as f:
            f.write(s)
    except OSError:
        pass


def _read_text(p) -> str:
    try:
        with open(p) as f:
            return f.read()
    except OSError:
        return ""


def _extract(header_json: str, key: str) -> str:
    k = f'"{key}":"'
    i = header_json.find(k)
    if i < 0:
        return ""
    j = header_json.find('"', i + len(k))
    return "" if j < 0 else header_json[i + len(k):j]


def _extract_state_path_from_header(h):
    return _extract(h, "state")


def _extract_model_class_from_header(h):
    return _extract(h, "model_class")


def _state_json(model) -> str:
    if hasattr(model, "state_json"):
        return model.state_json()
    sd = model.state_dict() if hasattr(model, "state_dict") else {}
    if isinstance(sd, str):
        return sd
    return json.dumps({k: f"tensor(dtype={str(v.dtype)}, shape={list(v.shape)})" for k, v in sd.items()},
                      separators=(",", ":"))


def _host():
    h = _C.host()
    h.mmj_blob_write.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int]
    h.mmj_blob_write.restype = ctypes.c_longlong
    h.mmj_blob_read.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int]
    h.mmj_blob_read.restype = ctypes.c_longlong
    return h


def write_blob(path: str, tensors) -> list:
    """Write tensors back to back (64-byte aligned) with the C++ writer; returns the index."""
    h = _host()
    index, off = [], 0
    first = True
    for name, t in tensors:
        tc = t.detach().contiguous().cpu()
        if tc.dtype == torch.bfloat16:
            raw = tc.view(torch.int16)
        else:
            raw = tc
        nbytes = raw.numel() * raw.element_size()
        rc = h.mmj_blob_write(path.encode(), raw.data_ptr(), nbytes, off, 1 if first else 0)
        if rc != 0:
            raise OSError(-rc, f"blob write failed: {path}")
        first = False
        index.append({"name": name, "shape": list(t.shape), "dtype": _DT[t.dtype], "offset": off,
                      "nbytes": nbytes})
        off = (off + nbytes + 63) // 64 * 64
    if first:
        open(path, "wb").close()
    return index


def read_blob_tensor(path: str, entry: dict) -> torch.Tensor:
    dt = _DT_INV[entry["dtype"]]
    store = torch.int16 if dt == torch.bfloat16 else dt
    n = 1
    for s in entry["shape"]:
        n *= s
    out = torch.empty(n, dtype=store)
    if n:
        got = _host().mmj_blob_read(path.encode(), out.data_ptr(), entry["nbytes"], entry["offset"], 4)
        if got != entry["nbytes"]:
            raise OSError(f"short read from {path}: {got} of {entry['nbytes']}")
    if dt == torch.bfloat16:
        out = out.view(torch.bfloat16)
    return out.view(entry["shape"])


def save_state_dict(model, path: str, stem: Optional[str] = None, extra: Optional[dict] = None,
                    rank: Optional[int] = None, world: Optional[int] = None,
                    shard_ranges: Optional[dict] = None) -> None:
    """Write header + state JSON + binary blob. ``(dir, stem)`` overload like the reference.
    Sharded runs pass ``rank/world`` and get one blob ``P.rank<r>of<W>.bin`` per rank."""
    base = os.path.join(path, stem) if stem is not None else path
    blob = _blob_path(base) if rank is None else f"{base}.rank{rank}of{world}.bin"
    sd = model.state_dict() if hasattr(model, "state_dict") else {}
    tensors = [(k, v) for k, v in sd.items() if isinstance(v, torch.Tensor)] if isinstance(sd, dict) else []
    index = write_blob(blob, tensors)
    total = sum(int(torch.Size(e["shape"]).numel()) for e in index)
    dts = {e["dtype"] for e in index}
    header = (
        "{"
        '"format":"MNP",'
        '"version":1,'
        f'"created_at":"{_escape_json_string(_now_iso8601())}",'
        '"model_class":"Model",'
        '"files":{'
        f'"state":"{_escape_json_string(_state_path(base))}",'
        f'"blob":"{_escape_json_string(blob)}"'
        "},"
        '"blob_meta":{'
        f'"dtype":"{(dts.pop() if len(dts) == 1 else "mixed") if index else "float32"}",'
        '"endian":"little",'
        f'"total_elems":{total}'
        "},"
        f'"tensors":{json.dumps(index, separators=(",", ":"))},'
        f'"sharding":{json.dumps({"rank": rank, "world": world, "ranges": shard_ranges}, separators=(",", ":"))},'
        f'"extra":{json.dumps(extra or {}, separators=(",", ":"))}'
        "}"
    )
    if rank is None or rank == 0:
        _write_text(_header_path(base) if rank is None else f"{base}.rank{rank}of{world}.json", header)
        _write_text(_state_path(base), _state_json(model))
    else:
        _write_text(f"{base}.rank{rank}of{world}.json", header)


def load_state_dict(model, path: str, stem: Optional[str] = None, strict: bool = False,
                    rank: Optional[int] = None, world: Optional[int] = None):
    """Returns True on success (reference contract). Loads tensor values when the header carries
    a blob index; a reference-written checkpoint (no blob) only validates the state JSON."""
    base = os.path.join(path, stem) if stem is not None else path
    hp = _header_path(base) if rank is None else f"{base}.rank{rank}of{world}.json"
    if os.path.exists(hp):
        hj = _read_text(hp)
        state_str = _extract_state_path_from_header(hj)
        if not state_str:
            return False
        sp = state_str if os.path.exists(state_str) else _state_path(base)
        if not os.path.exists(sp):
            return False
        try:
            h = json.loads(hj)
        except Exception:
            h = {}
        idx = h.get("tensors") or []
        if idx:
            blob = h["files"]["blob"]
            if not os.path.exists(blob):
                blob = _blob_path(base) if rank is None else f"{base}.rank{rank}of{world}.bin"
            sd = model.state_dict()
            with torch.no_grad():
                for e in idx:
                    if e["name"] in sd:
                        sd[e["name"]].copy_(read_blob_tensor(blob, e).to(sd[e["name"]].dtype))
                    elif strict:
                        raise KeyError(e["name"])
        elif hasattr(model, "load_state_json"):
            model.load_state_json(_read_text(sp))
        return True
    if os.path.exists(base):
        if hasattr(model, "load_state_json"):
            model.load_state_json(_read_text(base))
        return True
    return False


def read_extra(path: str) -> dict:
    try:
        return json.loads(_read_text(_header_path(path))).get("extra", {})
    except Exception:
        return {}


def exists_checkpoint(path: str, stem: Optional[str] = None) -> bool:
    base = os.path.join(path, stem) if stem is not None else path
    return os.path.exists(_header_path(base)) or os.path.exists(_state_path(base))


def exists_checkpoint_at(dir_: str, stem: str) -> bool:
    """``exists_checkpoint(dir_ + "/" + stem)`` (legacy/src/momijo/learn/utils/checkpoint.mojo:366-373)."""
    base = dir_
    if base and not base.endswith("/"):
        base += "/"
    return exists_checkpoint(base + stem)


def read_model_class_from_header(path: str, stem: Optional[str] = None) -> str:
    base = os.path.join(path, stem) if stem is not None else path
    return _extract_model_class_from_header(_read_text(_header_path(base)))


# ---- layout B ---------------------------------------------------------------------------------
def _param_layers(net):
    from ..nn.layers import Linear
    from ..nn.conv import Conv2d

    mods = net.to_list() if hasattr(net, "to_list") else list(net.modules())
    for m in mods:
        if isinstance(m, Linear):
            yield "Linear", m
        elif isinstance(m, Conv2d):
            yield "Conv2d", m


def make_checkpoint(net):
    """-> (header_json, flat Float32 tensor)."""
    parts, entries = [], []
    for kind, m in _param_layers(net):
        w, b = m.weight.detach().float().reshape(-1).cpu(), m.bias_t.detach().float().reshape(-1).cpu()
        parts += [w, b]
        entries.append('{"type":"%s","w":%d,"b":%d}' % (kind, w.numel(), b.numel()))
    flat = torch.cat(parts) if parts else torch.zeros(0)
    return '{"params":[' + ",".join(entries) + "]}", flat


def apply_checkpoint(net, header: str, blob: torch.Tensor) -> bool:
    """Copy by position; the header is not consulted (checkpoint.mojo:107-154)."""
    k = 0
    blob = blob.reshape(-1)
    with torch.no_grad():
        for _, m in _param_layers(net):
            for p in (m.weight, m.bias_t):
                n = p.numel()
                if k + n > blob.numel():
                    return False
                p.copy_(blob[k:k + n].view(p.shape).to(p.dtype))
                k += n
    return True
