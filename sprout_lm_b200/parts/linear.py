"""y = x W^T (+ bias) (+ residual): the one place that picks a matrix-product kernel.

float32 weights run on CUDA cores with float32 fused multiply-adds (the true 32-bit path).
bfloat16 weights run on the tcgen05 tensor-core kernel: weight rows on the MMA's M axis for a
handful of tokens (decode), tokens on M for many (prefill).  Up to 16 tokens through a small
matrix into a float32 sum take the light `mma.sync` kernel instead, which can also fold the
RMSNorm before the product in (csrc/linear_decode.cu).
"""
from __future__ import annotations

import os

import torch

from .. import kernels

SMALL_BATCH_TOKENS = 16     # up to this many tokens small layers take the light small-batch kernels (two tiles of the MMA's 8 columns)


def small_batch_enabled() -> bool:
    """SPROUT_SMALL_BATCH=0 keeps the tcgen05 products and the separate norm for every batch size."""
    return os.environ.get("SPROUT_SMALL_BATCH", "1") != "0"


def small_batch_split_k(out_features: int, in_features: int, tokens: int, residual: bool, sms: int) -> int:
    """How many CTAs share the K range of a small-batch product into a float32 residual:
    enough to put a CTA on most of the device's ``sms`` SMs when the matrix has few 128-row tiles."""
    if not residual or tokens > 256:
        return 1
    tiles = -(-out_features // 128)
    k_blocks = -(-in_features // 64)
    return max(1, min(k_blocks, sms // tiles))


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, status: torch.Tensor):
        self.weight = weight
        self.bias = bias
        self.status = status
        self.out_features, self.in_features = weight.shape
        self.sms = kernels.sm_count(weight.device) if weight.is_cuda else 0
        if weight.dtype == torch.bfloat16 and self.in_features % 8:
            raise ValueError(f"a bfloat16 matrix needs an inner size that is a multiple of 8 (got {self.in_features}): "
                             "its rows must start on 16-byte boundaries")
        # A handful of tokens through a small matrix: the light kernel (csrc/linear_decode.cu)
        self.small_tokens = 0
        if weight.dtype == torch.bfloat16 and weight.is_cuda and small_batch_enabled():
            for tokens in (SMALL_BATCH_TOKENS, 8):       # two tiles of 8 tokens where the pieces leave room, else one
                if kernels.linear_decode_supported(tokens, self.out_features, self.in_features):
                    self.small_tokens = tokens
                    break

    def split_k(self, tokens: int, residual: bool) -> int:
        return small_batch_split_k(self.out_features, self.in_features, tokens, residual, self.sms)

    def forward_swiglu(self, a: torch.Tensor, block: int) -> torch.Tensor:
        """silu(gate) * up of a fused gate/up matrix whose rows interleave the two in blocks of
        ``block``: fused into the product's epilogue on the tensor-core path (block 8), a separate
        kernel on the 32-bit path (any block)."""
        half = self.out_features // 2
        out = torch.empty((a.shape[0], half), dtype=a.dtype, device=a.device)
        if self.weight.dtype == torch.bfloat16:
            if block != 8:
                raise ValueError("the tensor-core SwiGLU epilogue reads gate and up rows interleaved in blocks of 8")
            kernels.gemm_bf16(a, self.weight, out, self.status, swiglu=True)
        else:
            kernels.swiglu(self.forward(a), out, block)
        return out

    def accumulate(self, a: torch.Tensor, acc: torch.Tensor) -> None:
        """acc (float32 [rows, out_features]) += a W^T, no bias: into a residual stream or a zeroed
        workspace.  bfloat16 weights only."""
        if a.shape[0] <= self.small_tokens:
            kernels.linear_decode(self.weight, acc, self.status, a=a)
        else:
            kernels.gemm_bf16(a, self.weight, acc, self.status, residual=acc, split_k=self.split_k(a.shape[0], True))

    def accumulate_unscaled(self, norm, x: torch.Tensor, acc: torch.Tensor) -> bool:
        """acc += bfloat16(x * gain) W^T: the product of the norm's output without its scale, for a
        consumer that multiplies row m's sums by 1 / rms(x[m]) itself (decode attention does).  The
        norm then costs no kernel of its own.  False (nothing done) when the sizes or the norm are not
        the kernel's."""
        tokens = x.shape[0]
        if self.weight.dtype != torch.bfloat16 or getattr(norm, "fused_kind", None) != "rmsnorm" or tokens > 256:
            return False
        split = self.split_k(tokens, True)
        if not kernels.gemm_bf16_unscaled_supported(tokens, self.out_features, self.in_features, split):
            return False
        # every CTA converts the tokens' columns of its own K range: with one k-block of 64 columns per
        # CTA (the 0.5B layer) that is cheaper than a norm kernel before the product, with 14 (the 7B
        # layer: 229 KB of rows read and converted per CTA) it is not (0.755 against 0.721 ms per
        # step of 4 layers at 64 tokens)
        if -(-(-(-self.in_features // 64)) // split) > 4:
            return False
        kernels.gemm_bf16_unscaled(x, norm.gain, self.weight, acc, self.status, split_k=split)
        return True

    def accumulate_normed(self, norm, x: torch.Tensor, acc: torch.Tensor) -> bool:
        """acc += rmsnorm(x) W^T in one kernel, for a few tokens of a small layer; False (nothing
        done) when the sizes or the norm are not the kernel's."""
        if x.shape[0] > self.small_tokens or getattr(norm, "fused_kind", None) != "rmsnorm":
            return False
        kernels.linear_decode(self.weight, acc, self.status, norm=(x, norm.gain, norm.eps))
        return True

    def forward(self, a: torch.Tensor, out_dtype: torch.dtype | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``residual`` (float32 [rows, out_features]) is added to in place and returned."""
        if residual is not None:
            out = residual
        else:
            out = torch.empty((a.shape[0], self.out_features), dtype=out_dtype or a.dtype, device=a.device)
        if self.weight.dtype == torch.bfloat16:
            if residual is not None and self.bias is None and a.shape[0] <= self.small_tokens:
                kernels.linear_decode(self.weight, out, self.status, a=a)
                return out
            kernels.gemm_bf16(a, self.weight, out, self.status, bias=self.bias, residual=residual,
                              split_k=self.split_k(a.shape[0], residual is not None))
        else:
            kernels.gemm_simple(a, self.weight, out, bias=self.bias, residual=residual)
        return out
