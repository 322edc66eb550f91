"""Collate helpers (legacy/src/momijo/learn/data/collate.mojo:19-69)."""
import torch


def pad_int_sequences(seqs, pad_value: int = 0, max_len: int | None = None):
    L = max_len if max_len is not None else max((len(s) for s in seqs), default=0)
    out = torch.full((len(seqs), L), pad_value, dtype=torch.int64)
    lens = []
    for i, s in enumerate(seqs):
        n = min(len(s), L)
        if n:
            out[i, :n] = torch.as_tensor(list(s[:n]), dtype=torch.int64)
        lens.append(n)
    return out, lens


def collate_stack(items):
    return torch.stack([torch.as_tensor(x) for x in items], 0)


def collate_pairs(items):
    xs, ys = zip(*items)
    return collate_stack(xs), collate_stack(ys)


def collate_identity(items):
    return list(items)


COLLATE_FNS = {0: collate_identity, 1: collate_stack, 2: collate_pairs}
