"""``y = x @ W^T (+ b)`` for weights stored ``[out, in]``, as every projection of the model is.

The kernel is chosen by storage types and shape: bfloat16 activations with bfloat16 weights
go to the tcgen05 tensor-core kernel when it takes the shape, everything else (the float32
path, 32-bit weights, odd shapes) to the 32-bit CUDA-core kernel.  The choice depends on the
weight's shape only, never on the number of rows, so a token's result does not depend on the
batch it is in.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import kernels


def _prefetch_cap() -> int:
    """Most bytes of the following product's weights that a product asks to be brought into L2
    (``SPYINFER_L2_PREFETCH_MB`` in the environment, 0 turns the hint off)."""
    try:
        return max(0, int(float(os.environ.get("SPYINFER_L2_PREFETCH_MB", "16")) * (1 << 20)))
    except ValueError:
        return 16 << 20


class Linear:
    #: the weight of the product that runs next in a step (set by the model once all parts are bound):
    #: a decoding product asks for the start of it to be brought into L2 while the short kernels
    #: between the two products run
    next_weight: Optional[torch.Tensor] = None
    #: False where the next product follows at once (nothing short runs in between, so there is no idle memory to use)
    hint_next: bool = True

    def __init__(self, weight: torch.Tensor, activation_dtype: torch.dtype, bias: Optional[torch.Tensor] = None):
        """``bias`` ``[out]`` (optional) is added by a pass of its own after the product; such a product
        always hands over a summed result (``defer`` is ignored) and takes no fused epilogue."""
        if weight.dim() != 2:
            raise ValueError(f"a linear weight is [out, in], found shape {tuple(weight.shape)}")
        if bias is not None and tuple(bias.shape) != (weight.shape[0],):
            raise ValueError(f"a bias of shape {tuple(bias.shape)} does not fit a weight of shape {tuple(weight.shape)}")
        self.weight, self.bias = weight, bias
        self.out_features, self.in_features = weight.shape
        self.fast = (activation_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                     and kernels.tensor_core_gemm_takes(self.out_features, self.in_features))
        self.prefetch_bytes = _prefetch_cap()

    def modules(self) -> List[str]:
        return (["gemm_tcgen05"] if self.fast else ["gemm_simt"]) + (["swiglu"] if self.bias is not None else [])

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None, epilogue: Optional[str] = None, defer: bool = False) -> torch.Tensor:
        """``epilogue="swiglu"`` (tensor-core kernel only; the weight's rows must alternate gate
        and up rows) returns ``silu(gate) * up``.  ``defer=True`` allows the result to come back
        as a stack ``[splits, rows, out]`` of float32 partial products that the consumer sums."""
        if self.bias is not None:
            if epilogue is not None:
                raise ValueError("a product with a bias takes no fused epilogue")
            defer = False
        y = self._product(x, out_dtype, epilogue, defer)
        return kernels.add_bias(y, self.bias) if self.bias is not None else y

    def _product(self, x, out_dtype, epilogue, defer):
        if self.fast:
            hint = self.next_weight if self.hint_next and x.shape[0] <= 256 and self.prefetch_bytes > 0 else None
            return kernels.gemm_tcgen05(x, self.weight, out_dtype=out_dtype or x.dtype, epilogue=epilogue, defer=defer,
                                        prefetch=hint, prefetch_bytes=self.prefetch_bytes)
        if epilogue is not None:
            raise ValueError("only the tensor-core product has fused epilogues")
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        return kernels.gemm_simt(x, self.weight, out)
