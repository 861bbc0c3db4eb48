"""Contract of a rollout engine as the workers use it.

Reference: ``mindspeed_rl/models/base/base_inference_engine.py:6-125`` (``BaseInferEngine``).  The
in-tree ``LLMEngine`` implements it; an external engine can be plugged in by implementing the same
five calls.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, List, Sequence


class BaseInferEngine(ABC):
    def __init__(self, tokenizer_name_or_path: str = "", train_tensor_parallel_size: int = 1,
                 train_pipeline_parallel_size: int = 1, train_expert_parallel_size: int = 1,
                 infer_tensor_parallel_size: int = 1, infer_pipeline_parallel_size: int = 1,
                 infer_expert_parallel_size: int = 1, max_num_seqs: int = 1, max_model_len: int = 2048,
                 dtype: str = "bfloat16", gpu_memory_utilization: float = 0.5, trust_remote_code: bool = True):
        self.tokenizer_name_or_path = tokenizer_name_or_path
        self.train_tensor_parallel_size = train_tensor_parallel_size
        self.train_pipeline_parallel_size = train_pipeline_parallel_size
        self.train_expert_parallel_size = train_expert_parallel_size
        self.infer_tensor_parallel_size = infer_tensor_parallel_size
        self.infer_pipeline_parallel_size = infer_pipeline_parallel_size
        self.infer_expert_parallel_size = infer_expert_parallel_size
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.dtype = dtype
        self.gpu_memory_utilization = gpu_memory_utilization
        self.trust_remote_code = trust_remote_code

    @abstractmethod
    def init_cache_engine(self) -> None:
        """Allocate the KV cache (start of a rollout phase)."""

    @abstractmethod
    def free_cache_engine(self) -> None:
        """Release the KV cache (end of a rollout phase)."""

    @abstractmethod
    def offload_model_weights(self) -> None:
        """Drop the engine's view of the weights so that the trainer owns the memory again."""

    @abstractmethod
    def sync_model_weights(self, params: Any, load_format: str = "megatron") -> None:
        """Bind the current training weights (resharded if needed) into the engine."""

    @abstractmethod
    def generate_sequences(self, idx_list: Sequence[Sequence[int]], **kwargs) -> List[Any]:
        """Generate for a list of prompt token lists."""
