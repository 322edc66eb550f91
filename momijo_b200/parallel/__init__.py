"""Process groups, peer-memory runtime and the parallel wrappers (DDP / ZeRO / TP / EP / PP)."""
from .flat import FlatParams, FlatLayout  # noqa: F401
from .zero import ShardedDataParallel, AdamWConfig, default_units  # noqa: F401
from .engine import HybridEngine, mark_replicated  # noqa: F401
from .ddp import DistributedDataParallel  # noqa: F401
from .cp import context_parallel_attention, shard_sequence  # noqa: F401
