"""SwiGLU feed-forward: x += W_down (silu(W_gate h) * W_up h), no biases (src/qwen.ts:196-200).

Gate and up are one fused product.  On the tensor-core path its weight rows interleave the two
in blocks of 8 (rows 16b..16b+7 are gate rows 8b..8b+7, rows 16b+8..16b+15 the matching up
rows), so that the product's epilogue sees a gate value and its up value side by side; that needs
an intermediate size that is a multiple of 8.  The 32-bit path has no such epilogue: it keeps the
gate rows first and the up rows after them, and takes any intermediate size.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part
from .linear import Linear, small_batch_enabled

INTERLEAVE = 8
FUSED_TOKENS = 16         # the one-kernel decode form takes up to this many tokens (two tiles of the MMA's 8 columns)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = INTERLEAVE) -> torch.Tensor:
    inter, hidden = gate.shape
    blocks = inter // block
    return torch.stack([gate.reshape(blocks, block, hidden), up.reshape(blocks, block, hidden)],
                       dim=1).reshape(2 * inter, hidden).contiguous()


@register_part("feed_forward", "swiglu_mlp")
class SwiGLUMLP(Part):
    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: dict | None = None):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("swiglu_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.block = INTERLEAVE            # rows of gate, then as many of up, and so on (set at load)
        names = names or {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.gate_up = self.down = None
        self._fused_tokens = 0            # up to this many tokens the one-kernel decode form runs

    def tensor_decls(self):
        return [TensorDecl(self.names["gate"] + ".weight", (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["up"] + ".weight", (self.intermediate_size, self.hidden_size)),
                TensorDecl(self.names["down"] + ".weight", (self.hidden_size, self.intermediate_size))]

    def load(self, source: WeightSource):
        if source.runtime.dtype == torch.bfloat16:
            if self.intermediate_size % INTERLEAVE:
                raise ValueError(f"swiglu_mlp: on the bfloat16 path intermediate_size must be a multiple of {INTERLEAVE} "
                                 f"(got {self.intermediate_size}): the tensor-core epilogue pairs gate and up rows in "
                                 f"blocks of {INTERLEAVE}; the float32 path takes any size")
            self.block = INTERLEAVE
        else:
            self.block = self.intermediate_size
        fused = interleave_gate_up(source.raw(self.names["gate"] + ".weight"), source.raw(self.names["up"] + ".weight"),
                                   self.block)
        self.gate_up = Linear(source.to_device_matrix(fused), None, source.runtime.status)
        self.down = Linear(source.matrix(self.names["down"] + ".weight"), None, source.runtime.status)
        # Small layers decode in one kernel that also takes the norm before the feed-forward
        # (csrc/ffn_decode.cu).
        if self.gate_up.weight.dtype == torch.bfloat16 and small_batch_enabled():
            for tokens in (FUSED_TOKENS, 8):             # two tiles of 8 tokens where the layer's shares leave room, else one
                if kernels.ffn_decode_supported(tokens, self.hidden_size, self.intermediate_size):
                    self._fused_tokens = tokens
                    break

    def forward(self, h, x, ctx=None):
        self.down.forward(self.gate_up.forward_swiglu(h, self.block), residual=x)

    def forward_with_norm(self, norm, x, ctx=None) -> bool:
        """x += feed_forward(norm(x)) in one kernel, if this layer and this batch allow it: an
        RMSNorm before it, a few tokens, a layer that fits.  False means nothing was done and the
        caller runs the norm and ``forward``."""
        tokens = x.shape[0]
        if getattr(norm, "fused_kind", None) != "rmsnorm" or tokens > self._fused_tokens:
            return False
        kernels.ffn_decode(x, norm.gain, norm.eps, self.gate_up.weight, self.down.weight, self.gate_up.status)
        return True
