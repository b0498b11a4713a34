"""A model built from a ``ModelSpec``: embedding, layers in run order, final norm, head.

The model owns its parts and their weights; it does not own the cache.  ``forward`` runs
exactly the tokens of one ``StepBatch`` and returns 32-bit logits at the wanted rows
(the reference norms and projects every row: spymaster2h/spyinfer
src/models/qwen3.hpp:283-301; only the wanted rows are computed here).
"""
from __future__ import annotations

import warnings
from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec
from ..csrc import build
from ..parts import BuildContext, build_block, build_part
from ..weights.loader import LazyTensors, WeightDecl, open_checkpoint
from ..weights.random_init import random_tensor


class _Layer:
    """A layer's parts by role, built from the spec, and the block arrangement over them."""

    def __init__(self, spec, ctx):
        self.prefix = spec.weight_prefix
        self.by_role = {role: build_part(part, ctx) for role, part in spec.roles().items()}
        self.block = build_block(spec.block, self.by_role)
        self.mixer = self.by_role.get("mixer")          # the part that owns the layer's cache, if the layer has one
        self.feed_forward = self.by_role.get("feed_forward")

    def parts(self):
        return list(self.by_role.values())


def _prefixed(part, prefix: str) -> List[WeightDecl]:
    return [WeightDecl(prefix + d.name, d.shape, d.init, d.integer) for d in part.weight_decls()]


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, max_model_len: int):
        spec.validate()
        self.spec = spec
        self.ctx = BuildContext(dtype=dtype, device=torch.device(device) if device is not None else None,
                                max_model_len=min(max_model_len, spec.max_position))
        self.embedding = build_part(spec.embedding, self.ctx)
        self.layers = [_Layer(ls, self.ctx) for ls in spec.layers]
        self.final_norm = build_part(spec.final_norm, self.ctx)
        self.head = build_part(spec.head, self.ctx)

    # ---- weights ---------------------------------------------------------------------------
    def weight_decls(self) -> List[WeightDecl]:
        decls = _prefixed(self.embedding, "")
        for layer in self.layers:
            for part in layer.parts():
                decls += _prefixed(part, layer.prefix)
        decls += _prefixed(self.final_norm, "") + _prefixed(self.head, "")
        return decls

    def ignorable_tensors(self) -> List[str]:
        return list(getattr(self.head, "ignorable", []))

    def bind(self, tensors) -> None:
        """``tensors``: every declared tensor by its full name, on the device: a dictionary, or a
        ``LazyTensors`` that makes each tensor when its part is bound.  The parts are bound one
        after the other and each gets only its own tensors, so with the latter the model never
        holds a part's stored tensors and the fused layouts made from them for more than one
        part at a time."""
        def sub(part, prefix):
            return {d.name: tensors[prefix + d.name] for d in part.weight_decls()}

        self.embedding.bind(sub(self.embedding, ""))
        for layer in self.layers:
            for part in layer.parts():
                part.bind(sub(part, layer.prefix))
        self.final_norm.bind(sub(self.final_norm, ""))
        head_names = {d.name for d in self.head.weight_decls()} | {getattr(self.head, "weight_name", None)} - {None}
        self.head.bind({n: tensors[n] for n in head_names if n in tensors})
        # every product learns which weight the step reads after its own (the hint is a weight's address, nothing else)
        chain = [lin for e in self.spec.run_order for part in self.layers[e.layer].parts() for lin in part.linears()] + self.head.linears()
        for lin, following in zip(chain, chain[1:]):
            lin.next_weight = following.weight
        build.ensure_built(self.kernel_modules())

    def load(self, model_dir: str) -> None:
        tensors = open_checkpoint(model_dir, self.weight_decls(), self.ctx.device, self.ignorable_tensors())
        try:
            if self.ctx.dtype == torch.bfloat16:
                shapes = {d.name: d.shape for d in self.weight_decls()}
                wide = [n for n, t in tensors.stored_dtypes.items() if len(shapes[n]) == 2 and t in (torch.float32, torch.float16)]
                if wide:
                    # a tensor stored in 32-bit stays so, and a 32-bit matrix cannot go to the bfloat16 tensor-core product
                    warnings.warn(f"{model_dir}: {len(wide)} matrices are stored in 32-bit (or 16-bit float, which is widened), the first being "
                                  f"{wide[0]!r}; they stay 32-bit and are multiplied by the CUDA-core kernel, which is far slower than "
                                  "the bfloat16 tensor-core one. Store the checkpoint in bfloat16 for speed.", stacklevel=2)
            self.bind(tensors)
        finally:
            tensors.close()

    def init_random(self, seed: int, std: float = 0.02, norm_std: float = 0.05) -> None:
        """Seeded random weights made on the device, tensor by tensor as the parts are bound (no host copy)."""
        decls = {d.name: d for d in self.weight_decls()}
        self.bind(LazyTensors(list(decls), lambda name: random_tensor(decls[name], seed, std, norm_std, self.ctx.device)))

    def kernel_modules(self) -> List[str]:
        mods: List[str] = []
        for part in [self.embedding, self.final_norm, self.head] + [p for l in self.layers for p in l.parts()]:
            mods += part.modules()
        return list(dict.fromkeys(mods))

    def graph_safe(self) -> bool:
        """Every part and every block arrangement says that its launches do not depend on a batch's content."""
        parts = [self.embedding, self.final_norm, self.head] + [p for l in self.layers for p in l.parts()]
        nested = [p.position for p in parts if getattr(p, "position", None) is not None]
        return all(p.graph_safe for p in parts + nested) and all(l.block.graph_safe for l in self.layers)

    # ---- cache needs -------------------------------------------------------------------------
    def cache_needs(self):
        """Per run-order entry: its mixer's need, and the entry whose cache it reads instead."""
        needs = [self.layers[e.layer].mixer.cache_need() if self.layers[e.layer].mixer is not None else None for e in self.spec.run_order]
        return needs, [e.cache_of for e in self.spec.run_order]

    # ---- one step ------------------------------------------------------------------------------
    def forward(self, batch, cache_manager) -> Optional[torch.Tensor]:
        hidden = self.embedding.forward(batch.token_ids, batch.status)
        delta = None
        for i, entry in enumerate(self.spec.run_order):
            view = cache_manager.view(i)
            if view.kind == "paged":
                view.block_table = batch.block_tables[view.group]
            hidden, delta = self.layers[entry.layer].block.forward(hidden, delta, batch, view)
        if batch.logit_rows.shape[0] == 0:
            return None
        x = self.final_norm.forward_add(hidden, delta, rows=batch.logit_rows)
        return self.head.forward(x)


def declared_weights(spec: ModelSpec) -> List[WeightDecl]:
    """The tensors a model of this description needs (no device, no kernels)."""
    return Model(spec, torch.bfloat16, None, spec.max_position).weight_decls()
