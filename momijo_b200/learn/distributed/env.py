"""Rank / world discovery from the environment (legacy/src/momijo/learn/distributed/env.mojo:15-82).
The reference's getenv shim always returns None; this reads RANK / WORLD_SIZE / LOCAL_RANK /
MASTER_ADDR / MASTER_PORT as the shim was meant to."""
import os


def getenv_compat(name: str, default=None):
    return os.environ.get(name, default)


def get_rank_world():
    """-> (rank, world, ok): ok is False when the launcher variables are absent."""
    r, w = os.environ.get("RANK"), os.environ.get("WORLD_SIZE")
    if r is None or w is None:
        return 0, 1, False
    try:
        return int(r), int(w), True
    except ValueError:
        return 0, 1, False


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def get_master():
    return os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ.get("MASTER_PORT", "29500"))
