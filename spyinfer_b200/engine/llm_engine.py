"""The request-level interface, in the manner of the reference's ``LLMEngine``
(spymaster2h/spyinfer src/engine/llm_engine.hpp:21-47): ``add_request``, ``step``,
``is_request_finished``, ``remove_request``, ``get_output_tokens``,
``has_unfinished_requests``.  Requests are token ids in and token ids out; text is outside
this engine.  Engine options are keyword arguments with the names of the reference's
parameter map (src/engine/llm_engine.cpp:11-16): ``max_num_batched_tokens``,
``max_num_seqs``, ``max_model_len``, ``kvcache_block_size``, ``num_kvcache_blocks``,
``backend_type`` (only "cuda" exists here), plus ``dtype``.

    engine = LLMEngine("/path/to/model", dtype="bfloat16", max_num_seqs=64)
    rid = engine.add_request([1, 2, 3], SamplingParams(max_new_tokens=16))
    while not engine.is_request_finished(rid):
        engine.step()
    tokens = engine.get_output_tokens(rid)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence as Seq, Tuple, Union

import torch

from ..cache import OutOfPages
from ..config import ArchitectureConfig, EngineConfig, load_model_config
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .model import Model
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import Sequence, SequenceStatus


PLACEHOLDER = -1     # stands in a request's tokens for a token that has been sampled on the device and not read yet


@dataclass
class _InFlight:
    """A step whose sampled tokens are still on the device."""

    seqs: List[Sequence]
    places: List[int]        # where in each request's tokens the sampled token goes
    tokens: torch.Tensor     # int32 [len(seqs)] on the device
    pending: object          # the queued copy of the tokens to the host (ModelRunner.start_read)


def _known(tokens: List[int]) -> List[int]:
    n = len(tokens)
    while n > 0 and tokens[n - 1] == PLACEHOLDER:
        n -= 1
    return tokens[:n]


class LLMEngine:
    def __init__(self, model_path: Optional[str] = None, *, model_config: Optional[ArchitectureConfig] = None, seed: int = 0,
                 weight_std: float = 0.02, norm_std: float = 0.05, backend_type: str = "cuda", **params):
        """``model_path``: a folder with config.json and safetensors.  Without it, ``model_config``
        and ``seed`` make a model with random weights on the device."""
        if backend_type != "cuda":
            raise ValueError(f"backend_type {backend_type!r}: this engine runs on CUDA only (the reference's \"cpu\" backend has no "
                             "counterpart here)")
        if (model_path is None) == (model_config is None):
            raise ValueError("give either model_path or model_config")
        from ..kernels import require_cuda
        require_cuda()
        self.config = EngineConfig(**params)
        self.model_config = load_model_config(model_path) if model_path is not None else model_config
        spec = self.model_config.to_spec()
        self.config.clamp_to_model(spec.max_position)
        dtype = torch.bfloat16 if self.config.dtype == "bfloat16" else torch.float32
        self.model = Model(spec, dtype, self.config.device, self.config.max_model_len)
        if model_path is not None:
            self.model.load(model_path)
        else:
            self.model.init_random(seed, weight_std, norm_std)
        self.runner = ModelRunner(self.model, self.config)
        self.scheduler = Scheduler(self.config, self.runner.cache)
        self.sampler = Sampler(self.config.device)
        self.eos_token_id = spec.eos_token_id
        self._sequences: Dict[int, Sequence] = {}
        self._next_id = 0
        self._inflight: Optional[_InFlight] = None

    # ---- requests ----------------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Seq[int], sampling_params: Optional[SamplingParams] = None) -> int:
        if len(prompt_token_ids) == 0:
            raise ValueError("a request needs at least one prompt token")
        vocab = self.model.spec.vocab_size
        for t in prompt_token_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        sp = sampling_params or SamplingParams()
        seq = Sequence(self._next_id, [int(t) for t in prompt_token_ids], len(prompt_token_ids), sp)
        self.scheduler.check_fits(seq, sp.max_new_tokens or 1)
        self._next_id += 1
        self._sequences[seq.id] = seq
        self.scheduler.add_sequence(seq)
        return seq.id

    def is_request_finished(self, request_id: int) -> bool:
        seq = self._sequences.get(request_id)
        return True if seq is None else seq.status == SequenceStatus.FINISHED

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    def get_output_tokens(self, request_id: int) -> List[int]:
        """Every token of the request, prompt first (as the reference returns them)."""
        seq = self._sequences.get(request_id)
        return _known(seq.tokens) if seq is not None else []

    def get_generated_tokens(self, request_id: int) -> List[int]:
        seq = self._sequences.get(request_id)
        return _known(seq.tokens)[seq.num_prompt_tokens:] if seq is not None else []

    def finish_reason(self, request_id: int) -> Optional[str]:
        seq = self._sequences.get(request_id)
        return seq.finish_reason if seq is not None else None

    def remove_request(self, request_id: int) -> None:
        seq = self._sequences.pop(request_id, None)
        if seq is not None and seq.status != SequenceStatus.FINISHED:
            if seq in self.scheduler.waiting:
                self.scheduler.waiting.remove(seq)
            self.scheduler.finish(seq, "removed")

    # ---- one step ------------------------------------------------------------------------------
    def step(self) -> List[Tuple[int, Optional[int], bool]]:
        """Schedules and runs one batch.  Returns ``(request id, new token, finished)`` for the
        tokens that became known in this call.  A request that the scheduler had to end because it
        could not go on even alone (``finish_reason`` ``"out_of_pages"``) appears once as
        ``(request id, None, True)``.

        With ``lookahead_decode`` (the default) a step in which every request decodes is launched
        and left in flight: its tokens are read, and returned, by the next call, AFTER that call has
        launched the following decode step for the same requests, whose token ids it takes on the
        device from the sampler's output.  The device then never waits for the host between decode
        steps.  The following step is launched only when its batch is certain: nothing is waiting, no
        request of the step in flight ends by ``max_new_tokens`` or ``max_model_len``, pages are
        free; a request that ends by its end-of-sequence token has then run one token too many,
        which is dropped.  Everything else (prompts, mixed steps, a changed set of requests) is
        read before the next step is decided, as without the option."""
        prev, self._inflight = self._inflight, None
        results: List[Tuple[int, int, bool]] = []
        if prev is not None:
            ahead = self._look_ahead(prev)
            results = self._absorb(prev, self.runner.finish_read(prev.pending))
            if ahead is not None:
                self._inflight = ahead
                return results
        portions = self.scheduler.schedule()
        for seq in self.scheduler.ended_without_token:
            del seq.tokens[len(_known(seq.tokens)):]
            results.append((seq.id, None, True))
        self.scheduler.ended_without_token.clear()
        if not portions:
            return results
        entries = [StepEntry(p.seq.id, p.seq.tokens[p.start:p.start + p.num_tokens], [p.num_tokens - 1] if p.samples else [])
                   for p in portions]
        logits = self.runner.step(entries)
        for p in portions:
            p.seq.num_computed = p.start + p.num_tokens
        sampled = [p.seq for p in portions if p.samples]
        if not sampled:
            return results
        flight = self._sample(sampled, logits)
        if self.config.lookahead_decode and all(p.num_tokens == 1 and p.samples for p in portions):
            self._inflight = flight
            return results
        return results + self._absorb(flight, self.runner.finish_read(flight.pending))

    def _sample(self, seqs: List[Sequence], logits: torch.Tensor) -> "_InFlight":
        """Samples the next token of every request on the device; each request gets a placeholder
        where the token will go once it has been read."""
        tokens = self.sampler.sample(logits, [s.sampling for s in seqs], [s.num_generated for s in seqs])
        places = []
        for s in seqs:
            places.append(len(s.tokens))
            s.tokens.append(PLACEHOLDER)
        return _InFlight(seqs, places, tokens, self.runner.start_read(tokens))   # the copy is queued now, ahead of any step launched later

    def _ends_at(self, seq: Sequence, place: int, token: Optional[int]) -> Optional[str]:
        """Why the request ends with the token at ``place`` (None: it goes on); ``token`` None: not known yet."""
        if token is not None and token == self.eos_token_id and not seq.sampling.ignore_eos:
            return "eos"
        if seq.sampling.max_new_tokens is not None and place + 1 - seq.num_prompt_tokens >= seq.sampling.max_new_tokens:
            return "max_new_tokens"
        if place + 1 >= self.config.max_model_len:
            return "max_model_len"
        if place + 1 > self.scheduler.most_tokens_alone():
            return "out_of_pages"                          # the pool could not hold the token's keys even if the request were alone
        return None

    def _absorb(self, flight: "_InFlight", tokens: List[int]) -> List[Tuple[int, int, bool]]:
        """The tokens of a step have been read: they take their places, requests that end are finished."""
        results = []
        for seq, place, tok in zip(flight.seqs, flight.places, tokens):
            if seq.status == SequenceStatus.FINISHED:
                continue                                   # it ended while this step was in flight: the token is dropped
            tok = int(tok)
            seq.tokens[place] = tok
            reason = self._ends_at(seq, place, tok)
            if reason is not None:
                del seq.tokens[place + 1:]                 # the placeholder of a step launched ahead
                self.scheduler.finish(seq, reason)
            results.append((seq.id, tok, reason is not None))
        return results

    def _look_ahead(self, prev: "_InFlight") -> Optional["_InFlight"]:
        """Launches the decode step that follows the one in flight, if its batch is certain."""
        sch = self.scheduler
        if not self.config.lookahead_decode or sch.waiting or len(sch.running) != len(prev.seqs):
            return None
        for seq, place in zip(prev.seqs, prev.places):
            if seq.status != SequenceStatus.RUNNING or place != len(seq.tokens) - 1 or self._ends_at(seq, place, None) is not None:
                return None
        if {id(s) for s in sch.running} != {id(s) for s in prev.seqs}:
            return None
        try:
            logits = self.runner.step([StepEntry(seq.id, [0], [0]) for seq in prev.seqs], tokens_from=prev.tokens)
        except OutOfPages:
            return None                                    # the scheduler decides who gives way, once the tokens are known
        for seq in prev.seqs:
            seq.num_computed = len(seq.tokens)
        return self._sample(prev.seqs, logits)

    def step_raw(self, entries: Seq[StepEntry]):
        """One batch straight through the step function, outside the scheduler: ``entries`` are
        ``StepEntry(request, tokens, want)`` (any hashable request name; a request lives until
        ``release_raw``).  Returns the float32 logits at the wanted places as a NumPy array
        ``[wanted, vocab]``, or None when nothing is wanted.  Meant for tests and for comparing
        with other engines; requests made here are unknown to ``step()``."""
        if self._inflight is not None:
            raise RuntimeError("step_raw: a scheduled step is still in flight; call drain() first")
        logits = self.runner.step(list(entries))
        self.runner.check_status()
        return None if logits is None else logits.float().cpu().numpy()

    def release_raw(self, request) -> None:
        """Gives back what a request of ``step_raw`` holds."""
        self.runner.finish(request)

    def drain(self) -> List[Tuple[int, int, bool]]:
        """Reads the step in flight, if there is one, without launching another."""
        prev, self._inflight = self._inflight, None
        return self._absorb(prev, self.runner.finish_read(prev.pending)) if prev is not None else []

    # ---- whole generations -----------------------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> List[List[int]]:
        """Runs the prompts to their ends with continuous batching; returns the generated tokens
        of each, in the order given."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        while any(not self.is_request_finished(i) for i in ids):
            self.step()
        self.drain()
        out = [self.get_generated_tokens(i) for i in ids]
        for i in ids:
            self.remove_request(i)
        return out

    def stats(self) -> Dict[str, int]:
        return {"steps": self.runner.steps, "tokens_run": self.runner.tokens_run, "preemptions": self.scheduler.num_preemptions,
                "free_pages": self.runner.cache.min_free_pages(), "free_slots": self.runner.cache.num_free_slots()}
