"""Engine options.  Names, meanings and defaults are the reference's ``EngineConfig`` (config.h:66-81):
``model_path``, ``max_num_batched_tokens`` (4096), ``max_num_seqs`` (256), ``max_chunk_tokens`` (1024, 0 = no
cap), ``max_model_len`` (4096), ``gpu_memory_utilization`` (0.90), ``num_kv_blocks`` (-1 = size from free
memory), ``enforce_eager`` (false = decode steps replay CUDA graphs), ``dtype`` and ``seed``.
``tensor_parallel_size`` exists only so that a value other than 1 is refused: this engine runs on one GPU.
Added here: ``block_size`` (tokens per cache page; the reference fixes 16 in sequence.h:28; the default here is 32,
because a TMA box is one page of one head and boxes of 32 rows come out a few percent faster than boxes of 16),
``pipeline_depth`` (steps in flight: 2 as the reference's ``kDepth``, engine/llm_engine.h:51, or 1 to wait for
every step's samples before the next step is scheduled) and ``enable_prefix_caching`` (requests share the cache pages
of a common prefix; always on in the reference, engine/block_manager.cpp:71-143; off by default here) and
``use_ref_kernels`` (every part uses its plain twin kernels: the general attention kernel, library products with separate
norm and activation kernels; for comparing the fast kernels with, inside the whole engine) and ``native_cache_manager``
(the cache manager in C++, as the reference's block manager is, engine/block_manager.cpp; false = its plain twin in
Python, which the tests compare it with) and ``native_scheduler`` (the scheduler and the requests in C++ as well, as
the reference's are, engine/scheduler.cpp; it needs the cache manager in C++; false = its plain twin in Python).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {name!r}") from None


@dataclass
class EngineConfig:
    model_path: str = ""
    max_num_batched_tokens: int = 4096
    max_num_seqs: int = 256
    max_chunk_tokens: int = 1024
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.90
    num_kv_blocks: int = -1
    tensor_parallel_size: int = 1
    enforce_eager: bool = False
    dtype: object = "bfloat16"
    seed: int = 0
    block_size: int = 32
    pipeline_depth: int = 2
    enable_prefix_caching: bool = False
    use_ref_kernels: bool = False
    native_cache_manager: bool = True
    native_scheduler: bool = True
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        if self.tensor_parallel_size != 1:
            raise ValueError("tensor_parallel_size must be 1: this engine runs on one GPU")
        if self.block_size <= 0 or self.block_size % 16:
            raise ValueError(f"block_size must be a positive multiple of 16, got {self.block_size}")
        if self.max_num_batched_tokens <= 0 or self.max_num_seqs <= 0 or self.max_model_len <= 0:
            raise ValueError("max_num_batched_tokens, max_num_seqs and max_model_len must be positive")
        if self.pipeline_depth not in (1, 2):
            raise ValueError("pipeline_depth must be 1 or 2")
        if self.max_chunk_tokens < 0:
            raise ValueError("max_chunk_tokens must be >= 0 (0 = no cap)")
