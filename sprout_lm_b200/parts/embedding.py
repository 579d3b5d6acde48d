"""Token embedding (a row copy, no scaling: src/qwen.ts:162-163) and the output head
(logits = W h, no bias; W is the embedding matrix itself when tied: src/qwen.ts:152,203)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorDecl, WeightSource, register_part
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, name: str = "embed_tokens"):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.tensor_name = f"{prefix}{name}.weight"
        self.table = None
        self.runtime = None

    def tensor_decls(self):
        return [TensorDecl(self.tensor_name, (self.vocab_size, self.hidden_size))]

    def load(self, source: WeightSource):
        self.table = source.matrix(self.tensor_name)
        self.runtime = source.runtime

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = torch.empty((token_ids.numel(), self.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embed(self.table, token_ids, x, self.runtime.status)
        return x


@register_part("head", "lm_head")
class LMHead(Part):
    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: str | None = None,
                 name: str = "lm_head"):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.tensor_name = f"{prefix}{tied_to or name}.weight"
        self.tied = tied_to is not None
        self.linear = None

    def tensor_decls(self):
        return [] if self.tied else [TensorDecl(self.tensor_name, (self.vocab_size, self.hidden_size))]

    def load(self, source: WeightSource):
        self.linear = Linear(source.matrix(self.tensor_name), None, source.runtime.status)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.linear.forward(h, out_dtype=torch.float32)
