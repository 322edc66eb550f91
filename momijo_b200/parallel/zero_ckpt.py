"""Checkpoint / resume of ``ShardedDataParallel``: the optimizer state (fp32 master weights, AdamW
moments, step count) in the MNP layout, one blob per rank, readable by a run of any other world size.

The state is stored per parameter, not per flat buffer: a rank writes, for every parameter, the
piece of ``master`` / ``m`` / ``v`` that falls into its shards, named ``master::<param>`` and so on,
and records the piece's range inside the flattened parameter in the header's ``sharding.ranges``
(files ``<base>.rank<r>of<W>.json|.bin``, the reference's per-rank naming; one rank writes
``<base>.json|.bin``). A reader looks up, for every piece it owns under its own layout, the
overlapping pieces of all the writers: bucket padding, shard boundaries and the world size may all
differ between the two runs.

Reference: the MNP header / blob format, legacy/src/momijo/learn/utils/checkpoint.mojo:208-373;
``ZeroStage1.state_dict`` (legacy/src/momijo/learn/distributed/sharding.mojo:176-184) carries only
``world_size`` and ``rank``, which is why the tensors live in the blob and the ranges in the header.
"""
from __future__ import annotations

import glob
import json
import os
import re
from collections import OrderedDict
from typing import Dict, Iterator, List, Tuple

import torch

KINDS = ("master", "m", "v")


def _names(engine) -> Dict[int, str]:
    return {id(p): n for n, p in engine.module.named_parameters()}


def owned_pieces(engine) -> Iterator[Tuple[str, int, int, int]]:
    """``(name, lo, hi, at)``: this rank holds the optimizer state of elements ``[lo, hi)`` of the flattened
    parameter ``name`` at index ``at`` of its ``master`` / ``m`` / ``v`` arrays."""
    names = _names(engine)
    if engine.world == 1:
        lay = engine.flat.layout
        for p, off in zip(lay.params, lay.offsets):
            yield names[id(p)], 0, p.numel(), off
        return
    R = engine.rank
    for b in engine.buckets:
        s_lo, s_hi = R * b.shard, (R + 1) * b.shard
        for p, o in zip(b.params, b.offsets):
            lo, hi = max(o, s_lo), min(o + p.numel(), s_hi)
            if lo < hi:
                yield names[id(p)], lo - o, hi - o, b.moff + lo - s_lo


class _State:
    """What ``learn.utils.checkpoint.save_state_dict`` needs from a model: a dict of tensors."""

    def __init__(self, tensors):
        self._t = tensors

    def state_dict(self):
        return self._t


def flat_pieces(engine) -> Iterator[Tuple[str, int, int, int]]:
    """The pieces of an engine that keeps the whole optimizer state in one ``FlatParams`` layout (bucketed data
    parallel, single rank): every parameter in full."""
    names = _names(engine)
    lay = engine.flat.layout
    for p, off in zip(lay.params, lay.offsets):
        yield names[id(p)], 0, p.numel(), off


def _collect(engine, pieces):
    state = {"master": engine.master, "m": engine.m, "v": engine.v}
    tensors, ranges = OrderedDict(), {}
    for name, lo, hi, at in pieces:
        ranges[name] = [lo, hi]
        for k in KINDS:
            tensors[f"{k}::{name}"] = state[k][at:at + hi - lo]
    return tensors, ranges


def save_replicated(engine, base: str, extra: dict | None = None) -> None:
    """One writer: an engine whose ranks all hold the same full optimizer state (``DistributedDataParallel``)."""
    from ..learn.utils.checkpoint import save_state_dict

    tensors, ranges = _collect(engine, flat_pieces(engine))
    meta = {"engine": type(engine).__name__, "world": 1, "step_count": engine.step_count, "lr": engine.optim.lr}
    meta.update(extra or {})
    d = os.path.dirname(base)
    if d:
        os.makedirs(d, exist_ok=True)
    if engine.master.is_cuda:
        torch.cuda.synchronize()
    save_state_dict(_State(tensors), base, extra=meta, shard_ranges=ranges)


def save(engine, base: str, extra: dict | None = None) -> None:
    """Write this rank's part of the optimizer state. Every rank calls it with the same ``base``."""
    from ..learn.utils.checkpoint import save_state_dict

    tensors, ranges = _collect(engine, owned_pieces(engine))
    meta = {"engine": "ShardedDataParallel", "stage": engine.stage, "world": engine.world,
            "step_count": engine.step_count, "lr": engine.lr,
            "betas": list(engine.optim.betas), "eps": engine.optim.eps, "weight_decay": engine.optim.weight_decay}
    meta.update(extra or {})
    d = os.path.dirname(base)
    if d:
        os.makedirs(d, exist_ok=True)
    if engine.is_cuda_engine():
        torch.cuda.synchronize()
    if engine.world == 1:
        save_state_dict(_State(tensors), base, extra=meta, shard_ranges=ranges)
    else:
        save_state_dict(_State(tensors), base, extra=meta, rank=engine.rank, world=engine.world,
                        shard_ranges=ranges)
        engine.comm.host_barrier()


def _writer_headers(base: str) -> List[Tuple[dict, str]]:
    """Headers (parsed) and blob paths of every rank that wrote ``base``."""
    out = []
    by_world: Dict[int, List[Tuple[int, str]]] = {}
    for f in glob.glob(glob.escape(base) + ".rank*of*.json"):
        m = re.search(r"\.rank(\d+)of(\d+)\.json$", f)
        if m:
            by_world.setdefault(int(m.group(2)), []).append((int(m.group(1)), f))
    if by_world:
        # several world sizes may have written to the same base over time: the newest complete set wins
        complete = {w: sorted(fs) for w, fs in by_world.items() if len(fs) == w}
        if not complete:
            w, fs = next(iter(by_world.items()))
            raise FileNotFoundError(f"{base}: found {len(fs)} of {w} rank files")
        world = max(complete, key=lambda w: max(os.path.getmtime(f) for _, f in complete[w]))
        single = base + ".json"
        if os.path.exists(single) and os.path.getmtime(single) > max(os.path.getmtime(f) for _, f in complete[world]):
            out.append((json.load(open(single)), base + ".bin"))
            return out
        for _, f in complete[world]:
            out.append((json.load(open(f)), f[:-len(".json")] + ".bin"))
    elif os.path.exists(base + ".json"):
        out.append((json.load(open(base + ".json")), base + ".bin"))
    else:
        raise FileNotFoundError(f"no checkpoint at {base}")
    return out


def load(engine, base: str) -> dict:
    """Restore the optimizer state from a checkpoint written by any world size, republish the bf16 parameters
    from the restored master weights and return the checkpoint's ``extra`` dict. Collective over the ranks."""
    extra = read_into(engine, base, owned_pieces(engine))
    engine.step_count = int(extra.get("step_count", engine.step_count))
    if "lr" in extra:
        engine.lr = float(extra["lr"])
    engine.republish_from_master()
    return extra


def read_into(engine, base: str, pieces) -> dict:
    """Fill ``engine.master / m / v`` at the given pieces from whatever ranks wrote ``base``; returns ``extra``."""
    from ..learn.utils.checkpoint import read_blob_tensor

    writers = _writer_headers(base)
    index = []   # per writer: name -> (range, {kind: entry})
    for h, blob in writers:
        ranges = (h.get("sharding") or {}).get("ranges") or {}
        ent = {e["name"]: e for e in h.get("tensors", [])}
        index.append((ranges, ent, blob))
    state = {"master": engine.master, "m": engine.m, "v": engine.v}
    cache: Dict[Tuple[int, str], torch.Tensor] = {}
    with torch.no_grad():
        for name, lo, hi, at in pieces:
            covered = 0
            for wi, (ranges, ent, blob) in enumerate(index):
                if name not in ranges:
                    continue
                olo, ohi = ranges[name]
                a, b = max(lo, olo), min(hi, ohi)
                if a >= b:
                    continue
                for k in KINDS:
                    key = (wi, f"{k}::{name}")
                    t = cache.get(key)
                    if t is None:
                        t = read_blob_tensor(blob, ent[key[1]]).reshape(-1)
                        cache[key] = t
                    state[k][at + a - lo:at + b - lo].copy_(t[a - olo:b - olo])
                covered += b - a
            if covered != hi - lo:
                raise KeyError(f"{base}: elements [{lo}, {hi}) of {name} are covered {covered} times over")
            cache = {k_: v_ for k_, v_ in cache.items() if not k_[1].endswith("::" + name)}
    return writers[0][0].get("extra", {})
