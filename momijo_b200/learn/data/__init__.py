"""Data loading (``momijo.learn.data``)."""
from .dataset import (  # noqa: F401
    Dataset, TupleDataset, TensorDataset, IterableDataset, IndexSliceDataset, IndexListDataset,
    ZipDataset, EnumerateDataset, lcg_shuffle, LCG32, shuffle_inplace, make_arange, clamp_index,
    make_random_index_partition, IndexAdapter, make_index_slice, make_index_list, make_zip, make_enumerate,
)
from .dataloader import (  # noqa: F401
    DataLoader, DataLoaderOptions, BatchIter, IndexIter, RNG32, make_dataloaders_from_png,
)
from .sampler import RandomSampler, SequentialSampler, DistributedSampler, _assert_dist_shapes_equal  # noqa: F401
from .pipeline import Pipeline, PipelineIter  # noqa: F401
from .collate import (  # noqa: F401
    pad_int_sequences, collate_stack, collate_pairs, collate_identity, stack_int_labels, collate_pairs_varlen,
    collate_varlen_by,
)
from .pair import Pair  # noqa: F401
from .image import ImageFolderDataset, list_dirs_sorted, list_dirs_sorted_paths, list_pngs_sorted  # noqa: F401
