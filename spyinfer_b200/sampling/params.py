"""Per-request sampling options.

The reference samples greedily only (argmax on the host, spymaster2h/spyinfer
src/engine/model_runner.cpp:120-134) and stops at ``eos_token_id`` or ``max_model_len``
(:148).  Here: ``temperature`` 0 is that greedy choice; a positive temperature draws from
``softmax(logits / temperature)`` with a per-request ``seed``, among the ``top_k`` most
likely tokens only if that is given (0: among all); ``max_new_tokens`` and ``ignore_eos``
bound the generation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0
    top_k: int = 0
    max_new_tokens: Optional[int] = None
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError(f"temperature must not be negative, found {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must not be negative (0 means all tokens), found {self.top_k}")
        if self.max_new_tokens is not None and self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be positive, found {self.max_new_tokens}")
