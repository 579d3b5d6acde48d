"""Rotary position encoding with half-split pairs (d, d + head_dim/2), angle =
position / theta**(2d / head_dim) (src/qwen.ts:81-92).

The angles are computed in float64 on the host for every position up to ``max_positions``
and kept as float32 cosine and sine tables; the kernel that rotates q and k reads them.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part


@register_part("position", "rope_half_split")
class HalfSplitRotary(Part):
    def __init__(self, prefix: str, head_dim: int, theta: float, max_positions: int):
        if head_dim % 2:
            raise ValueError("rotary position encoding needs an even head_dim")
        if theta <= 0 or max_positions <= 0:
            raise ValueError("rotary position encoding needs positive theta and max_positions")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)

    def angles(self) -> np.ndarray:
        d = np.arange(self.head_dim // 2, dtype=np.float64)
        inv = self.theta ** (2.0 * d / self.head_dim)
        return np.arange(self.max_positions, dtype=np.float64)[:, None] / inv[None, :]

    interleaved = False          # pairs (d, d + head_dim / 2)

    def rotary_tables(self, runtime):
        """The tables depend on (head_dim, theta, max_positions) alone: all layers of a model share
        one copy on the device."""
        def build():
            angle = self.angles()
            cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(runtime.device)
            sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(runtime.device)
            return cos.contiguous(), sin.contiguous()
        shared = getattr(runtime, "shared", None)
        return shared(("rope_half_split", self.head_dim, self.theta, self.max_positions), build) if shared else build()


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k are used as projected."""

    def __init__(self, prefix: str = "", **_):
        pass

    def rotary_tables(self, runtime):
        return None
