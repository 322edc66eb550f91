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


def _write_csv(x, path, dt, opts):
    opts = opts or CsvOptions()
    r = _raw(x).to(dt).cpu()
    r2 = r.reshape(1, -1) if r.dim() <= 1 else r.reshape(r.shape[0], -1)
    with open(path, "w") as f:
        if opts.has_header:
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


def write_csv_f64(x, path, opts=None): return _write_csv(x, path, torch.float64, opts)
def write_csv_f32(x, path, opts=None): return _write_csv(x, path, torch.float32, opts)
def write_csv_int(x, path, opts=None): return _write_csv(x, path, torch.int64, opts)
def read_csv_f64(path, opts=None): return _read_csv(path, torch.float64, opts)
def read_csv_f32(path, opts=None): return _read_csv(path, torch.float32, opts)
def read_csv_int(path, opts=None): return _read_csv(path, torch.int64, opts)


def _write_json(x, path, dt):
    r = _raw(x).to(dt).cpu()
    with open(path, "w") as f:
        json.dump({"shape": list(r.shape), "dtype": str(dt).replace("torch.", ""), "data": r.reshape(-1).tolist()}, f)
    return True


def _read_json(path, dt):
    with open(path) as f:
        d = json.load(f)
    return _wrap(torch.tensor(d["data"], dtype=dt).reshape(d["shape"]))


def write_json_f64(x, path): return _write_json(x, path, torch.float64)
def write_json_f32(x, path): return _write_json(x, path, torch.float32)
def write_json_int(x, path): return _write_json(x, path, torch.int64)
def read_json_f64(path): return _read_json(path, torch.float64)
def read_json_f32(path): return _read_json(path, torch.float32)
def read_json_int(path): return _read_json(path, torch.int64)


def _write_xml(x, path, dt):
    r = _raw(x).to(dt).cpu()
    name = str(dt).replace("torch.", "")
    body = " ".join(_fmt(v, dt, 17) for v in r.reshape(-1).tolist())
    with open(path, "w") as f:
        f.write(f'<tensor dtype="{name}" shape="{",".join(map(str, r.shape))}">{body}</tensor>\n')
    return True


def _read_xml(path, dt):
    with open(path) as f:
        s = f.read()
    m = re.search(r'<tensor[^>]*shape="([^"]*)"[^>]*>(.*?)</tensor>', s, re.S)
    if not m:
        raise ValueError("not a tensor XML file")
    shape = [int(v) for v in m.group(1).split(",") if v]
    vals = [float(v) if dt != torch.int64 else int(float(v)) for v in m.group(2).split()]
    return _wrap(torch.tensor(vals, dtype=dt).reshape(shape))


def write_xml_f64(x, path): return _write_xml(x, path, torch.float64)
def write_xml_f32(x, path): return _write_xml(x, path, torch.float32)
def write_xml_int(x, path): return _write_xml(x, path, torch.int64)
def read_xml_f64(path): return _read_xml(path, torch.float64)
def read_xml_f32(path): return _read_xml(path, torch.float32)
def read_xml_int(path): return _read_xml(path, torch.int64)


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
