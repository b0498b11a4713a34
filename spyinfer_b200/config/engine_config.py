"""Engine options, with the names of spymaster2h/spyinfer's ``Config`` (src/config.hpp:17-27)
and of the keys its ``LLMEngine`` accepts (src/engine/llm_engine.cpp:11-16) where it has them.

Differences from the reference, which reads only some of its own fields:
``max_num_batched_tokens`` and ``max_num_seqs`` are honoured here (the token budget of a
step and the number of live requests), and ``chunk_size`` (not in the reference, which runs a prompt whole) caps
one request's prompt portion in a step; ``num_kvcache_blocks`` may be left out, and is then
derived from free device memory and ``gpu_memory_utilization``; ``kvcache_block_size``
defaults to 16 tokens rather than 4.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineConfig:
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    chunk_size: Optional[int] = None  # most prompt tokens of ONE request in a step; None: the token budget alone cuts prompts
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    kvcache_block_size: int = 16
    num_kvcache_blocks: Optional[int] = None
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    use_cuda_graphs: bool = True
    graph_step_tokens: int = 384      # steps of other shapes than decode steps are replayed from CUDA graphs up to this many tokens (0: never)
    lookahead_decode: bool = True     # launch the next decode step before the last one's tokens are read (see LLMEngine.step)

    def __post_init__(self):
        if self.dtype not in _DTYPES:
            raise ValueError(f"dtype {self.dtype!r}: choose bfloat16 or float32")
        self.dtype = _DTYPES[self.dtype]
        for name in ("max_num_batched_tokens", "max_num_seqs", "max_model_len", "kvcache_block_size"):
            v = getattr(self, name)
            if not isinstance(v, int) or v <= 0:
                raise ValueError(f"{name} must be a positive integer, found {v!r}")
        if self.chunk_size is not None and (not isinstance(self.chunk_size, int) or self.chunk_size <= 0):
            raise ValueError(f"chunk_size must be a positive integer or None, found {self.chunk_size!r}")
        if self.num_kvcache_blocks is not None and self.num_kvcache_blocks <= 0:
            raise ValueError(f"num_kvcache_blocks must be positive, found {self.num_kvcache_blocks!r}")
        if not isinstance(self.graph_step_tokens, int) or self.graph_step_tokens < 0:
            raise ValueError(f"graph_step_tokens must be a non-negative integer, found {self.graph_step_tokens!r}")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must lie in (0, 1]")

    def clamp_to_model(self, max_position: int) -> None:
        """``max_model_len`` never exceeds what the model's positions allow (src/config.hpp:12)."""
        self.max_model_len = min(self.max_model_len, int(max_position))
