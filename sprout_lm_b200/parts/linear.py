"""y = x W^T (+ bias) (+ residual): the one place that picks a matrix-product kernel.

float32 weights run on CUDA cores with float32 fused multiply-adds (the true 32-bit path).
bfloat16 weights run on the tcgen05 tensor-core kernel: weight rows on the MMA's M axis for a
handful of tokens (decode), tokens on M for many (prefill).
"""
from __future__ import annotations

import torch

from .. import kernels

SM_COUNT = 148


def small_batch_split_k(out_features: int, in_features: int, tokens: int, residual: bool) -> int:
    """How many CTAs share the K range of a small-batch product into a float32 residual:
    enough to put a CTA on most SMs when the matrix has few 128-row tiles."""
    if not residual or tokens > 256:
        return 1
    tiles = -(-out_features // 128)
    k_blocks = -(-in_features // 64)
    return max(1, min(k_blocks, SM_COUNT // tiles))


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, status: torch.Tensor):
        self.weight = weight
        self.bias = bias
        self.status = status
        self.out_features, self.in_features = weight.shape
        if weight.dtype == torch.bfloat16 and self.in_features % 8:
            raise ValueError(f"a bfloat16 matrix needs an inner size that is a multiple of 8 (got {self.in_features}): "
                             "its rows must start on 16-byte boundaries")

    def split_k(self, tokens: int, residual: bool) -> int:
        return small_batch_split_k(self.out_features, self.in_features, tokens, residual)

    def forward_swiglu(self, a: torch.Tensor) -> torch.Tensor:
        """silu(gate) * up of a fused, interleaved gate/up matrix: fused into the product's epilogue
        on the tensor-core path, a separate kernel on the 32-bit path."""
        half = self.out_features // 2
        out = torch.empty((a.shape[0], half), dtype=a.dtype, device=a.device)
        if self.weight.dtype == torch.bfloat16:
            kernels.gemm_bf16(a, self.weight, out, self.status, swiglu=True)
        else:
            kernels.swiglu(self.forward(a), out)
        return out

    def forward(self, a: torch.Tensor, out_dtype: torch.dtype | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` (float32 [rows, out_features]) is added to in place and returned."""
        if residual is not None:
            out = residual
        else:
            out = torch.empty((a.shape[0], self.out_features), dtype=out_dtype or a.dtype, device=a.device)
        if self.weight.dtype == torch.bfloat16:
            kernels.gemm_bf16(a, self.weight, out, self.status, bias=self.bias, residual=residual,
                              split_k=self.split_k(a.shape[0], residual is not None))
        else:
            kernels.gemm_simple(a, self.weight, out, bias=self.bias, residual=residual)
        return out
