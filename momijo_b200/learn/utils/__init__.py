"""Utilities (``momijo.learn.utils``)."""
from . import checkpoint, checkpoint_fileio, tensor_bytes, fileio_stub, randomness, profiling, summary, prune  # noqa: F401
from .checkpoint import (  # noqa: F401
    make_checkpoint, apply_checkpoint, save_state_dict, load_state_dict, exists_checkpoint,
    read_model_class_from_header,
)
from .checkpoint_fileio import save_checkpoint_files, load_checkpoint_files  # noqa: F401
from .tensor_bytes import pack_f64, unpack_f64, pack_f64_to_bytes, unpack_bytes_to_f64  # noqa: F401
from .randomness import SplitMix64, Xoshiro256ss, RNG, SeedBundle, seed_all, derived_rngs  # noqa: F401
from .profiling import Timer, ScopedTimer, LapStats, LabelProfiler, ScopedSection, SMA, TrainingLoopProfiler  # noqa: F401
from .summary import Summarizer, model_summary  # noqa: F401
from .prune import PruneState, tensor_sparsity  # noqa: F401
