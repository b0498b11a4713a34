"""``y = x @ W^T`` for weights stored ``[out, in]``, as every projection of the model is.

The kernel is chosen by storage types and shape: bfloat16 activations with bfloat16 weights
go to the tcgen05 tensor-core kernel when it takes the shape, everything else (the float32
path, 32-bit weights, odd shapes) to the 32-bit CUDA-core kernel.  The choice depends on the
weight's shape only, never on the number of rows, so a token's result does not depend on the
batch it is in.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, activation_dtype: torch.dtype):
        if weight.dim() != 2:
            raise ValueError(f"a linear weight is [out, in], found shape {tuple(weight.shape)}")
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self.fast = (activation_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                     and kernels.tensor_core_gemm_takes(self.out_features, self.in_features))

    def modules(self) -> List[str]:
        return ["gemm_tcgen05"] if self.fast else ["gemm_simt"]

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None, epilogue: Optional[str] = None, defer: bool = False) -> torch.Tensor:
        """``epilogue="swiglu"`` (tensor-core kernel only; the weight's rows must alternate gate
        and up rows) returns ``silu(gate) * up``.  ``defer=True`` allows the result to come back
        as a stack ``[splits, rows, out]`` of float32 partial products that the consumer sums."""
        if self.fast:
            return kernels.gemm_tcgen05(x, self.weight, out_dtype=out_dtype or x.dtype, epilogue=epilogue, defer=defer)
        if epilogue is not None:
            raise ValueError("only the tensor-core product has fused epilogues")
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        return kernels.gemm_simt(x, self.weight, out)
