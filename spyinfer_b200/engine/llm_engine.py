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

from typing import Dict, List, Optional, Sequence as Seq, Tuple, Union

import torch

from ..config import ArchitectureConfig, EngineConfig, load_model_config
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .model import Model
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import Sequence, SequenceStatus


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
        return list(seq.tokens) if seq is not None else []

    def get_generated_tokens(self, request_id: int) -> List[int]:
        seq = self._sequences.get(request_id)
        return seq.output_tokens if seq is not None else []

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
    def step(self) -> List[Tuple[int, int, bool]]:
        """Schedules and runs one batch.  Returns ``(request id, new token, finished)`` for every
        request that produced a token in this step."""
        portions = self.scheduler.schedule()
        if not portions:
            return []
        entries = [StepEntry(p.seq.id, p.seq.tokens[p.start:p.start + p.num_tokens], [p.num_tokens - 1] if p.samples else [])
                   for p in portions]
        logits = self.runner.step(entries)
        for p in portions:
            p.seq.num_computed = p.start + p.num_tokens
        sampled = [p.seq for p in portions if p.samples]
        if not sampled:
            return []
        tokens = self.runner.read_tokens(self.sampler.sample(logits, [s.sampling for s in sampled], [s.num_generated for s in sampled]))
        results = []
        for seq, tok in zip(sampled, tokens):
            seq.tokens.append(int(tok))
            reason = None
            if tok == self.eos_token_id and not seq.sampling.ignore_eos:
                reason = "eos"
            elif seq.sampling.max_new_tokens is not None and seq.num_generated >= seq.sampling.max_new_tokens:
                reason = "max_new_tokens"
            elif len(seq) >= self.config.max_model_len:
                reason = "max_model_len"
            if reason is not None:
                self.scheduler.finish(seq, reason)
            results.append((seq.id, int(tok), reason is not None))
        return results

    # ---- whole generations -----------------------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], sampling_params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> List[List[int]]:
        """Runs the prompts to their ends with continuous batching; returns the generated tokens
        of each, in the order given."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        while any(not self.is_request_finished(i) for i in ids):
            self.step()
        out = [self.get_generated_tokens(i) for i in ids]
        for i in ids:
            self.remove_request(i)
        return out

    def stats(self) -> Dict[str, int]:
        return {"steps": self.runner.steps, "tokens_run": self.runner.tokens_run, "preemptions": self.scheduler.num_preemptions,
                "free_pages": self.runner.cache.min_free_pages(), "free_slots": self.runner.cache.num_free_slots()}
