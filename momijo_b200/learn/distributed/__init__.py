"""Distributed API (``momijo.learn.distributed``): the reference facade plus the parallel wrappers."""
from .env import get_rank_world, getenv_compat, get_local_rank  # noqa: F401
from .collective import (  # noqa: F401
    ReduceOp, get_world_size, get_rank, allreduce, allreduce_sum, allreduce_sum_f64, broadcast,
    barrier, reduce, reduce_f64, reduce_list_int, reduce_list_f64, all_gather, reduce_scatter,
    all_to_all, send, recv, isend, irecv, is_distributed,
)
from .ddp import ProcessGroup, init_process_group, destroy_process_group, DDPLinear  # noqa: F401
from .strategies import DataParallel, DistributedDataParallel  # noqa: F401
from .sharding import ShardRange, partition_1d, ZeroStage1  # noqa: F401
from ...parallel.zero import ShardedDataParallel, AdamWConfig  # noqa: F401
