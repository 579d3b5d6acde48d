"""Learned RMSNorm: out = fround(x / sqrt(mean(x^2) + eps)) * gain (src/qwen.ts:72-77)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    fused_kind = "rmsnorm"       # a consumer that has this norm's arithmetic in its own kernel may take gain and eps

    def __init__(self, prefix: str, size: int, eps: float, name: str = "norm"):
        if eps <= 0:
            raise ValueError("rmsnorm: eps must be positive")
        self.size, self.eps = int(size), float(eps)
        self.tensor_name = f"{prefix}{name}.weight"
        self.gain = None
        self.out_dtype = None

    def tensor_decls(self):
        return [TensorDecl(self.tensor_name, (self.size,), "gain")]

    def load(self, source: WeightSource):
        self.gain = source.vector(self.tensor_name)
        self.out_dtype = source.runtime.dtype

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        count = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((count, self.size), dtype=self.out_dtype, device=x.device)
        kernels.rmsnorm(x, self.gain, out, self.eps, rows)
        return out
