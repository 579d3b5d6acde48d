"""y = x W^T (+ bias) (+ residual): the one place that picks a matrix-product kernel.

float32 weights run on CUDA cores with float32 fused multiply-adds (the true 32-bit path).
bfloat16 weights run on the tensor-core kernels; the plain kernel stays reachable through
``force_simple`` for tests that compare the two.
"""
from __future__ import annotations

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None):
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self.force_simple = False

    def forward(self, a: torch.Tensor, out_dtype: torch.dtype | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` (float32 [rows, out_features]) is added to in place and returned."""
        if residual is not None:
            out = residual
        else:
            out = torch.empty((a.shape[0], self.out_features), dtype=out_dtype or a.dtype, device=a.device)
        if self.weight.dtype == torch.bfloat16 and not self.force_simple and kernels.has_tensor_core_gemm():
            kernels.gemm_bf16(a, self.weight, out, bias=self.bias, residual=residual)
        else:
            kernels.gemm_simple(a, self.weight, out, bias=self.bias, residual=residual)
        return out
