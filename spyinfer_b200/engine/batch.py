"""The batch of one step: for every request in it, its next tokens; flat arrays on the device.

One step may hold portions of prompts beside single decoded tokens, cut anywhere.  The
arrays (all int32):

* ``token_ids[T]``, ``positions[T]`` (absolute position of each token in its request),
  ``seq_of_token[T]`` (index of its request in this batch);
* ``q_start[S + 1]`` (where each request's tokens begin), ``ctx_len[S]`` (the request's length
  after this step), ``state_slot[S]``;
* one block table ``[S, width]`` per cache group;
* ``logit_rows[R]``: the tokens whose logits are wanted.

The reference builds the same kind of flat batch in its scheduler (spymaster2h/spyinfer
src/engine/scheduler.hpp:15-24, scheduler.cpp:52-119) and derives positions in the runner
(src/engine/model_runner.cpp:61-84); it re-allocates the device copies every step
(src/utils/context.cpp:49-78).  Here one pinned staging buffer and one device buffer are
reused, and a step is one host-to-device copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and which of them want logits
    (indices into ``tokens``)."""

    request: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepBatch:
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    q_start: torch.Tensor
    ctx_len: torch.Tensor
    state_slot: torch.Tensor
    logit_rows: torch.Tensor
    block_tables: List[torch.Tensor]
    status: torch.Tensor
    # host copies, for parts that plan their launches on the host
    host_positions: np.ndarray = None
    host_q_start: np.ndarray = None
    host_ctx_len: np.ndarray = None
    host_state_slot: np.ndarray = None
    max_q_len: int = 0
    max_ctx_len: int = 0
    #: every request of the batch brings exactly one token (a decode step): parts may then take kernels made for that
    one_token_each: bool = False
    #: how many requests at the head of the batch bring exactly one token while later ones bring more (0 when the batch is
    #: not laid out that way): an attention part may run those through its kernel for decoding and the rest through the
    #: one for prompt portions
    one_token_head: int = 0
    extras: Dict[str, object] = field(default_factory=dict)


class BatchStager:
    """Owns the pinned host buffer and the device buffer that every step's arrays live in."""

    def __init__(self, device, max_tokens: int, max_seqs: int, table_width: int, num_groups: int):
        self.device = device
        self.max_tokens, self.max_seqs, self.width, self.num_groups = max_tokens, max_seqs, table_width, num_groups
        n = 4 * max_tokens + 3 * max_seqs + 1 + num_groups * max_seqs * table_width + 8
        self.capacity = n
        self.host = torch.empty(n, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(n, dtype=torch.int32, device=device)
        self.status = kernels.status_word(device)
        self._copied = torch.cuda.Event()
        self._copy_pending = False

    def stage(self, token_ids: np.ndarray, positions: np.ndarray, seq_of_token: np.ndarray, q_start: np.ndarray, ctx_len: np.ndarray,
              state_slot: np.ndarray, logit_rows: np.ndarray, tables: List[np.ndarray], pad_tokens: int = 0, pad_seqs: int = 0) -> StepBatch:
        """Copies the arrays to the device (one transfer) and returns views of the device buffer.

        ``pad_tokens``/``pad_seqs``: lay the arrays out for at least this many tokens/requests
        (fixed offsets for a captured graph); the padding is not part of the batch."""
        T, S, R = len(token_ids), len(ctx_len), len(logit_rows)
        if T > self.max_tokens or S > self.max_seqs:
            raise ValueError(f"a step of {T} tokens / {S} requests exceeds the limits {self.max_tokens} / {self.max_seqs}")
        Tc, Sc = max(T, pad_tokens), max(S, pad_seqs)
        if self._copy_pending:  # the last step's transfer must have read the pinned buffer before it is rewritten
            self._copied.synchronize()
        h, off, spans = self.host_np, 0, []
        for arr, cap in ((token_ids, Tc), (positions, Tc), (seq_of_token, Tc), (logit_rows, Tc), (q_start, Sc + 1), (ctx_len, Sc), (state_slot, Sc)):
            h[off:off + len(arr)] = arr
            spans.append((off, len(arr)))
            off += cap
        widths = []
        for t in tables:
            w = t.shape[1]
            h[off:off + S * w] = t.reshape(-1)
            spans.append((off, S * w))
            widths.append(w)
            off += Sc * w
        self.dev[:off].copy_(self.host[:off], non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        d = self.dev
        v = [d[o:o + n] for o, n in spans]
        return StepBatch(
            num_tokens=T, num_seqs=S, token_ids=v[0], positions=v[1], seq_of_token=v[2], logit_rows=v[3], q_start=v[4], ctx_len=v[5],
            state_slot=v[6], block_tables=[v[7 + i].view(S, widths[i]) for i in range(len(tables))], status=self.status,
            host_positions=positions, host_q_start=q_start, host_ctx_len=ctx_len, host_state_slot=state_slot,
            max_q_len=int(np.max(q_start[1:] - q_start[:-1])) if S else 0, max_ctx_len=int(ctx_len.max()) if S else 0,
            one_token_each=bool(S > 0 and T == S and int(np.min(q_start[1:] - q_start[:-1])) == 1))
