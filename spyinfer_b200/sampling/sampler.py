"""Chooses the next token of every row of a step's logits, on the device.

One kernel launch for the whole batch; only the token ids cross to the host.  A row's token
depends on its logits, its request's seed and the number of tokens the request has drawn so
far, not on the batch: a request preempted and recomputed draws the same tokens again.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from .params import SamplingParams


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], draws: Sequence[int]) -> torch.Tensor:
        """``logits [R, V]`` float32 on the device; ``draws[r]`` is how many tokens row r's
        request has generated before this one.  Returns int32 ``[R]`` on the device."""
        R = logits.shape[0]
        tokens = torch.empty(R, dtype=torch.int32, device=logits.device)
        if all(p.temperature == 0.0 for p in params):
            return kernels.sample(logits, tokens)
        t = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(logits.device, non_blocking=True)
        s = torch.tensor([p.seed for p in params], dtype=torch.int64).to(logits.device, non_blocking=True)
        d = torch.tensor(list(draws), dtype=torch.int64).to(logits.device, non_blocking=True)
        k = None
        if any(p.top_k > 0 and p.temperature > 0.0 for p in params):
            k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(logits.device, non_blocking=True)
        return kernels.sample(logits, tokens, t, s, d, k)
