"""Megatron / NeMo style datasets: memory-mapped token files, GPT sample index, weighted blending, C++ index helpers."""
from nanotron_b200.data.nemo_dataset.blendable_dataset import BlendableDataset, MemoryEfficientBlendableDataset  # noqa: F401
from nanotron_b200.data.nemo_dataset.dataset_utils import get_datasets_weights_and_num_samples, get_train_valid_test_split_  # noqa: F401
from nanotron_b200.data.nemo_dataset.indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder, make_builder, make_indexed_dataset  # noqa: F401


def __getattr__(name):
    # GPTDataset and the builders import the logging / distributed stack: resolved lazily so that the light pieces above
    # (and the C++ helpers) can be used on their own.
    if name in ("GPTDataset", "build_dataset", "build_train_valid_test_datasets", "get_indexed_dataset", "permute", "SubsetSplitLog"):
        from nanotron_b200.data.nemo_dataset import gpt_dataset

        return getattr(gpt_dataset, name)
    raise AttributeError(name)
