"""Data loading (``momijo.learn.data``)."""
from .dataset import (  # noqa: F401
    Dataset, TupleDataset, TensorDataset, IterableDataset, IndexSliceDataset, IndexListDataset,
    ZipDataset, EnumerateDataset, lcg_shuffle,
)
from .dataloader import DataLoader, DataLoaderOptions  # noqa: F401
from .sampler import RandomSampler, SequentialSampler, DistributedSampler, _assert_dist_shapes_equal  # noqa: F401
from .pipeline import Pipeline, PipelineIter  # noqa: F401
from .collate import pad_int_sequences, collate_stack, collate_pairs, collate_identity  # noqa: F401
from .pair import Pair  # noqa: F401
from .image import ImageFolderDataset  # noqa: F401
