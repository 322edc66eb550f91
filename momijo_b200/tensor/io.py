"""Text I/O for tensors: CSV / JSON / XML for f64, f32 and int, plus ``save_npz_f64``
(legacy/src/momijo/tensor/io.mojo:194-791)."""
from __future__ import annotations

import io as _io
import json
import re
import zipfile
from dataclasses import dataclass

import numpy as np
import torch

from .tensor import _raw, _wrap


@dataclass
class CsvOptions:
    delimiter: str = ","
    has_header: bool = False
    precision: int = 17
    newline: str = "\n"


def _fmt(v, dt, prec):
    if dt == torch.int64:
        return str(int(v))
    return repr(float(v)) if prec >= 17 else f"{float(v):.{prec}g}"


def _write_csv(x, path, dt, opts, header=None):
    """``opts`` is a ``CsvOptions`` or, in the reference's call form ``write_csv_f64(x, path, delim, header)``
    (legacy/src/momijo/tensor/io.mojo:710-713), the delimiter string followed by the header names."""
    if isinstance(opts, str):
        opts = CsvOptions(delimiter=opts)
    opts = opts or CsvOptions()
    r = _raw(x).to(dt).cpu()
    r2 = r.reshape(1, -1) if r.dim() <= 1 else r.reshape(r.shape[0], -1)
    with open(path, "w") as f:
        if header:
            f.write(opts.delimiter.join(str(h) for h in header) + opts.newline)
        elif opts.has_header:
            f.write(opts.delimiter.join(f"c{i}" for i in range(r2.shape[1])) + opts.newline)
        for row in r2.tolist():
            f.write(opts.delimiter.join(_fmt(v, dt, opts.precision) for v in row) + opts.newline)
    return True


def _read_csv(path, dt, opts):
    opts = opts or CsvOptions()
    rows = []
    with open(path) as f:
        lines = [l.strip() for l in f if l.strip()]
    if opts.has_header and lines:
        lines = lines[1:]
    for l in lines:
        rows.append([float(v) if dt != torch.int64 else int(float(v)) for v in l.split(opts.delimiter)])
    return _wrap(torch.tensor(rows, dtype=dt))


def write_csv_f64(x, path, opts=None, header=None): return _write_csv(x, path, torch.float64, opts, header)
def write_csv_f32(x, path, opts=None, header=None): return _write_csv(x, path, torch.float32, opts, header)
def write_csv_int(x, path, opts=None, header=None): return _write_csv(x, path, torch.int64, opts, header)
def read_csv_f64(path, opts=None): return _read_csv(path, torch.float64, opts)
def read_csv_f32(path, opts=None): return _read_csv(path, torch.float32, opts)
def read_csv_int(path, opts=None): return _read_csv(path, torch.int64, opts)


def _write_json(x, path, dt, pretty=False):
    r = _raw(x).to(dt).cpu()
    with open(path, "w") as f:
        json.dump({"shape": list(r.shape), "dtype": str(dt).replace("torch.", ""), "data": r.reshape(-1).tolist()}, f,
                  indent=2 if pretty else None)
    return True


def _read_json(path, dt):
    with open(path) as f:
        d = json.load(f)
    return _wrap(torch.tensor(d["data"], dtype=dt).reshape(d["shape"]))


def write_json_f64(x, path, pretty=True): return _write_json(x, path, torch.float64, pretty)
def write_json_f32(x, path, pretty=True): return _write_json(x, path, torch.float32, pretty)
def write_json_int(x, path, pretty=True): return _write_json(x, path, torch.int64, pretty)
def read_json_f64(path): return _read_json(path, torch.float64)
def read_json_f32(path): return _read_json(path, torch.float32)
def read_json_int(path): return _read_json(path, torch.int64)


def _write_xml(x, path, dt, root_tag="tensor", row_tag="row", item_tag="v"):
    """One root element carrying dtype and shape with the values as text. With non-default tags the reference's nested
    layout ``<root><row><v>..</v>..</row>..</root>`` is written instead (legacy/src/momijo/tensor/io.mojo:729-733)."""
    r = _raw(x).to(dt).cpu()
    if (root_tag, row_tag, item_tag) != ("tensor", "row", "v"):
        with open(path, "w") as f:
            f.write(tensor_to_xml_numbers(_wrap(r), None, root_tag, row_tag, item_tag))
        return True
    name = str(dt).replace("torch.", "")
    body = " ".join(_fmt(v, dt, 17) for v in r.reshape(-1).tolist())
    with open(path, "w") as f:
        f.write(f'<tensor dtype="{name}" shape="{",".join(map(str, r.shape))}">{body}</tensor>\n')
    return True


def _read_xml(path, dt, row_tag="row", item_tag="v"):
    with open(path) as f:
        s = f.read()
    m = re.search(r'<tensor[^>]*shape="([^"]*)"[^>]*>(.*?)</tensor>', s, re.S)
    if not m or f"<{item_tag}>" in s:
        return _wrap(_raw(xml_numbers_to_tensor_with(s, None, row_tag, item_tag)).to(dt))
    shape = [int(v) for v in m.group(1).split(",") if v]
    vals = [float(v) if dt != torch.int64 else int(float(v)) for v in m.group(2).split()]
    return _wrap(torch.tensor(vals, dtype=dt).reshape(shape))


def write_xml_f64(x, path, root_tag="tensor", row_tag="row", item_tag="v"): return _write_xml(x, path, torch.float64, root_tag, row_tag, item_tag)  # noqa: E501
def write_xml_f32(x, path, root_tag="tensor", row_tag="row", item_tag="v"): return _write_xml(x, path, torch.float32, root_tag, row_tag, item_tag)  # noqa: E501
def write_xml_int(x, path, root_tag="tensor", row_tag="row", item_tag="v"): return _write_xml(x, path, torch.int64, root_tag, row_tag, item_tag)  # noqa: E501
def read_xml_f64(path, row_tag="row", item_tag="v"): return _read_xml(path, torch.float64, row_tag, item_tag)
def read_xml_f32(path, row_tag="row", item_tag="v"): return _read_xml(path, torch.float32, row_tag, item_tag)
def read_xml_int(path, row_tag="row", item_tag="v"): return _read_xml(path, torch.int64, row_tag, item_tag)


def save_npz_f64(path, **arrays):
    """NumPy ``.npz`` archive of float64 arrays."""
    np.savez(path, **{k: _raw(v).double().cpu().numpy() for k, v in arrays.items()})
    return True


def load_npz(path):
    with np.load(path) as z:
        return {k: _wrap(torch.from_numpy(z[k])) for k in z.files}


def save_npy(path, x):
    np.save(path, _raw(x).cpu().numpy())
    return True


def load_npy(path):
    return _wrap(torch.from_numpy(np.load(path)))


# ---- converter-parameterised text forms (legacy/src/momijo/tensor/io.mojo:247-680). ``from_f64`` / ``to_f64`` are
# the element converters of the reference's generic functions; any callable (or None) works here.
def _conv_in(vals, from_f64):
    return [from_f64(float(v)) for v in vals] if from_f64 is not None else [float(v) for v in vals]


def _conv_out(x, to_f64):
    r = _raw(x).cpu()
    flat = r.reshape(-1).tolist()
    return r, ([to_f64(v) for v in flat] if to_f64 is not None else [float(v) for v in flat])


def csv_to_tensor_with(text: str, from_f64=None, opts: CsvOptions = None):
    """Rows of delimiter-separated numbers -> 2-D tensor (ragged rows are padded with zeros)."""
    opts = opts or CsvOptions()
    lines = [l.strip() for l in text.splitlines() if l.strip()]
    if opts.has_header and lines:
        lines = lines[1:]
    rows = [_conv_in([c for c in l.split(opts.delimiter) if c.strip() != ""], from_f64) for l in lines]
    width = max((len(r) for r in rows), default=0)
    rows = [r + [0] * (width - len(r)) for r in rows]
    return _wrap(torch.tensor(rows) if rows else torch.zeros(0, 0))


def tensor_to_csv(x, to_f64=None, delim: str = ",", header=None) -> str:
    r, flat = _conv_out(x, to_f64)
    cols = r.shape[-1] if r.dim() >= 1 else 1
    rows = [flat[i:i + cols] for i in range(0, len(flat), max(cols, 1))]
    out = [delim.join(header)] if header else []
    out += [delim.join(repr(v) for v in row) for row in rows]
    return "\n".join(out) + ("\n" if out else "")


def json_numbers_to_tensor_with(text: str, from_f64=None):
    """A JSON array of numbers (nested arrays give the shape)."""
    try:
        data = json.loads(text)
    except ValueError:
        return _wrap(torch.zeros(0))
    t = torch.tensor(data, dtype=torch.float64)
    return _wrap(torch.tensor(_conv_in(t.reshape(-1).tolist(), from_f64)).reshape(t.shape))


def tensor_to_json_array(x, to_f64=None, pretty: bool = True) -> str:
    r, flat = _conv_out(x, to_f64)
    nested = torch.tensor(flat, dtype=torch.float64).reshape(r.shape).tolist() if flat else []
    return json.dumps(nested, indent=2 if pretty else None)


def xml_numbers_to_tensor_with(text: str, from_f64=None, row_tag: str = "row", item_tag: str = "v"):
    rows = re.findall(rf"<{row_tag}[^>]*>(.*?)</{row_tag}>", text, re.S)
    if not rows:
        rows = [text]
    data = [_conv_in(re.findall(rf"<{item_tag}[^>]*>\s*([^<\s]+)\s*</{item_tag}>", r), from_f64) for r in rows]
    width = max((len(r) for r in data), default=0)
    data = [r + [0] * (width - len(r)) for r in data]
    return _wrap(torch.tensor(data) if data and width else torch.zeros(0, 0))


def tensor_to_xml_numbers(x, to_f64=None, root_tag: str = "tensor", row_tag: str = "row", item_tag: str = "v") -> str:
    r, flat = _conv_out(x, to_f64)
    cols = r.shape[-1] if r.dim() >= 1 else 1
    rows = [flat[i:i + cols] for i in range(0, len(flat), max(cols, 1))]
    body = "".join(f"<{row_tag}>" + "".join(f"<{item_tag}>{v!r}</{item_tag}>" for v in row) + f"</{row_tag}>"
                   for row in rows)
    return f"<{root_tag}>{body}</{root_tag}>"


def _read(path: str) -> str:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return ""


def _write(path: str, text: str) -> bool:
    try:
        with open(path, "w") as f:
            f.write(text)
        return True
    except OSError:
        return False


def read_csv_with(path, from_f64=None, opts: CsvOptions = None): return csv_to_tensor_with(_read(path), from_f64, opts)   # noqa: E704,E501
def write_csv(x, to_f64, path, delim=",", header=None): return _write(path, tensor_to_csv(x, to_f64, delim, header))     # noqa: E704,E501
def read_json_numbers_with(path, from_f64=None): return json_numbers_to_tensor_with(_read(path), from_f64)              # noqa: E704,E501
def write_json_numbers(x, to_f64, path, pretty=True): return _write(path, tensor_to_json_array(x, to_f64, pretty))      # noqa: E704,E501


def read_xml_numbers_with(path, from_f64=None, row_tag="row", item_tag="v"):
    return xml_numbers_to_tensor_with(_read(path), from_f64, row_tag, item_tag)


def write_xml_numbers(x, to_f64, path, root_tag="tensor", row_tag="row", item_tag="v"):
    return _write(path, tensor_to_xml_numbers(x, to_f64, root_tag, row_tag, item_tag))
