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


def stack_int_labels(labels):
    """[n] int64 tensor of class labels (legacy/src/momijo/learn/data/collate.mojo:48-49)."""
    return torch.as_tensor([int(v) for v in labels], dtype=torch.int64)


def _seq_of(x):
    return x.reshape(-1).tolist() if isinstance(x, torch.Tensor) else list(x)


def collate_pairs_varlen(batch):
    """Batch of items with ``.x`` (an int sequence) and ``.y`` (a label), or ``(x, y)`` tuples ->
    (zero-padded [B, maxlen] int64, [B] int64) (legacy/src/momijo/learn/data/collate.mojo:53-64)."""
    seqs, labs = [], []
    for item in batch:
        x, y = (item.x, item.y) if hasattr(item, "x") and hasattr(item, "y") else item
        seqs.append(_seq_of(x))
        labs.append(int(y))
    return pad_int_sequences(seqs, 0)[0], stack_int_labels(labs)


def collate_varlen_by(batch, get_seq, get_label):
    """Same with caller-supplied extractors (legacy/src/momijo/learn/data/collate.mojo:69-84)."""
    seqs = [_seq_of(get_seq(item)) for item in batch]
    labs = [int(get_label(item)) for item in batch]
    return pad_int_sequences(seqs, 0)[0], stack_int_labels(labs)
