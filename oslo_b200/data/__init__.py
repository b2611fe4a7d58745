from .blending import DatasetBlender  # noqa: F401
from .datasets import DatasetForCausalLM  # noqa: F401
from .indexing import (IndexedCachedDataset, IndexedDataset, IndexedDatasetBuilder,  # noqa: F401
                       MMapIndex, MmapIndex, MMapIndexedDataset, MMapIndexedDatasetBuilder, NumpyUtils, PathUtils)
from .loaders import InfiniteDataLoader  # noqa: F401
from .preprocess import DatasetBinarizer, DatasetEncoder, DatasetPreprocessor  # noqa: F401
from .samplers import DatasetFromSampler, DistributedProxySampler  # noqa: F401
