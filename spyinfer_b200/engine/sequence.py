"""The host-side record of one request, as the scheduler sees it.

Counterpart of the reference's ``Sequence`` (spymaster2h/spyinfer src/engine/sequence.hpp:8-32):
id, status, tokens; ``num_computed`` plays the part of its ``token_pos`` (how many tokens
already have keys and values in the cache).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class Sequence:
    id: int
    tokens: List[int]
    num_prompt_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed: int = 0
    finish_reason: Optional[str] = None
    num_preemptions: int = 0

    def __len__(self) -> int:
        return len(self.tokens)

    @property
    def remaining(self) -> int:
        """Tokens that have not been run yet (1 while decoding)."""
        return len(self.tokens) - self.num_computed

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.num_prompt_tokens

    @property
    def output_tokens(self) -> List[int]:
        return self.tokens[self.num_prompt_tokens:]
