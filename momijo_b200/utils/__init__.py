"""Timing, clock sampling and misc helpers."""
from .clocks import ClockSampler  # noqa: F401
from .timing import cuda_time_ms, max_over_ranks  # noqa: F401
from .elastic import (DictStore, FailureDetector, Heartbeat, RankFailure, guarded_step, partition_1d,  # noqa: F401
                      reshard_flat, run_elastic)
