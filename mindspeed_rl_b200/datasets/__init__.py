"""Datasets: indexed ``.bin/.idx`` files, chat templates, preprocessing handlers, prompt loaders."""
from .indexed_dataset import (CombinedDataset, IndexedDataset, IndexedDatasetBuilder,
                              get_packed_indexed_dataset)
from .prompt_dataset import (BaseDataset, PromptDataset, build_train_valid_test_datasets,
                             get_train_valid_test_split)
from .dataloader import InfiniteLoader, PretrainingSampler, PromptDataLoader, PromptSampler
from .data_handler import build_dataset, get_dataset_handler
from .templates import Template, get_model_template
from .synthetic import SyntheticPromptLoader

__all__ = ["IndexedDataset", "IndexedDatasetBuilder", "CombinedDataset", "get_packed_indexed_dataset",
           "BaseDataset", "PromptDataset", "build_train_valid_test_datasets", "get_train_valid_test_split",
           "PromptDataLoader", "PromptSampler", "PretrainingSampler", "InfiniteLoader",
           "get_dataset_handler", "build_dataset", "Template", "get_model_template",
           "SyntheticPromptLoader"]
