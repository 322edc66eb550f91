"""String forms of lists, dicts and tensors (legacy/src/momijo/tensor/printing.mojo:13-61,
legacy/src/momijo/tensor/cast.mojo:5197-5310)."""
import torch


def list_to_string(xs) -> str:
    return "[" + ", ".join(str(x) for x in xs) + "]"


def dict_to_string(d) -> str:
    return "{" + ", ".join(f"{k}: {v}" for k, v in d.items()) + "}"


def _fmt(v):
    if isinstance(v, bool):
        return "True" if v else "False"
    if isinstance(v, float):
        return f"{v:.6g}" if v == v else "nan"
    return str(v)


def _nd(x, max_items=6):
    if not isinstance(x, list):
        return _fmt(x)
    if len(x) > 2 * max_items:
        parts = [_nd(v, max_items) for v in x[:max_items]] + ["..."] + [_nd(v, max_items) for v in x[-max_items:]]
    else:
        parts = [_nd(v, max_items) for v in x]
    return "[" + ", ".join(parts) + "]"


def tensor_to_string(t) -> str:
    r = t.as_subclass(torch.Tensor) if isinstance(t, torch.Tensor) else torch.as_tensor(t)
    dt = str(r.dtype).replace("torch.", "")
    body = _nd(r.detach().cpu().tolist() if r.dtype != torch.bfloat16 else r.detach().float().cpu().tolist())
    return f"Tensor(shape={list(r.shape)}, dtype={dt}, data={body})"


# names of the reference (legacy/src/momijo/tensor/printing.mojo:13-61)
def to_string_list(xs) -> str: return list_to_string(xs)          # noqa: E704
def to_string_dict(d) -> str: return dict_to_string(d)            # noqa: E704
def to_string_tensor(t) -> str: return tensor_to_string(t)        # noqa: E704


to_string_inttensor = to_string_tensor


def ravel(x) -> list:
    """Flat Python list of a tensor's elements (row-major)."""
    from .tensor import _raw
    return _raw(x).reshape(-1).tolist()
