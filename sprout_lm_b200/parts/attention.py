"""Grouped-query attention over the paged cache (src/qwen.ts:166-195).

q, k, v = W h + b in one fused product; q and k are rotated by the token's position
(after the bias, before caching: the cache holds rotated keys and unrotated values); query head
h reads key/value head h // (heads // kv_heads); the score is the dot divided by
sqrt(head_dim); the mask is causal; the output projection has no bias unless ``out_bias``.
"""
from __future__ import annotations

import os

import torch

from .. import kernels
from ..config.specs import PartSpec
from .base import CacheSpec, CacheView, Part, TensorDecl, WeightSource, build_part, register_part
from .linear import Linear

# SPROUT_UNSCALED_PRODUCT=0: decode steps of more tokens than the small-batch kernels take run the norm
# before attention as a kernel of its own (else its scale is applied inside the attention kernel)
UNSCALED_PRODUCT = os.environ.get("SPROUT_UNSCALED_PRODUCT", "1") != "0"


@register_part("mixer", "gqa_attention")
class PagedGQAttention(Part):
    def __init__(self, prefix: str, hidden_size: int, heads: int, kv_heads: int, head_dim: int,
                 position: PartSpec, qkv_bias: bool = True, out_bias: bool = False, names: dict | None = None):
        if heads % kv_heads:
            raise ValueError(f"attention: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if head_dim <= 0 or head_dim % 2 or head_dim > 256:
            raise ValueError(f"attention: head_dim must be even and at most 256 (got {head_dim})")
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = hidden_size, heads, kv_heads, head_dim
        self.qkv_bias, self.out_bias = qkv_bias, out_bias
        names = names or {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}
        self.names = {key: prefix + value for key, value in names.items()}
        self.position = build_part("position", position)
        self.qkv = self.out = None
        self.tables = None
        self.interleaved = False
        self.runtime = None

    # ---- what it keeps
    def cache_spec(self):
        return CacheSpec(kv_heads=self.kv_heads, head_dim=self.head_dim, kind="full")

    def state_spec(self):
        return None

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        """How the decode step's attention is laid out: with the whole context in one CTA's shared
        memory (and room for how many keys), or divided among CTAs (and how): it follows the
        contexts' length, not only the block tables' width."""
        if self.heads // self.kv_heads > 16:
            return None
        return kernels.decode_attention_plan(requests, self.heads, self.kv_heads, self.head_dim, page_tokens, max_keys,
                                             planned_context)

    # ---- weights
    def tensor_decls(self):
        q_width, kv_width = self.heads * self.head_dim, self.kv_heads * self.head_dim
        decls = [TensorDecl(self.names["q"] + ".weight", (q_width, self.hidden_size)),
                 TensorDecl(self.names["k"] + ".weight", (kv_width, self.hidden_size)),
                 TensorDecl(self.names["v"] + ".weight", (kv_width, self.hidden_size)),
                 TensorDecl(self.names["o"] + ".weight", (self.hidden_size, q_width))]
        if self.qkv_bias:
            decls += [TensorDecl(self.names["q"] + ".bias", (q_width,), "bias"),
                      TensorDecl(self.names["k"] + ".bias", (kv_width,), "bias"),
                      TensorDecl(self.names["v"] + ".bias", (kv_width,), "bias")]
        if self.out_bias:
            decls.append(TensorDecl(self.names["o"] + ".bias", (self.hidden_size,), "bias"))
        return decls

    def load(self, source: WeightSource):
        self.runtime = source.runtime
        if source.runtime.dtype == torch.bfloat16 and self.head_dim % 16:
            raise ValueError(f"attention: on the bfloat16 path head_dim must be a multiple of 16 (got {self.head_dim}): "
                             "the tensor-core kernels are written for head sizes in steps of 16; the float32 path "
                             "takes any even head size up to 256")
        fused = torch.cat([source.raw(self.names[key] + ".weight") for key in ("q", "k", "v")], dim=0)
        bias = None
        if self.qkv_bias:
            bias = torch.cat([source.raw(self.names[key] + ".bias").to(torch.float32) for key in ("q", "k", "v")])
            bias = bias.to(source.runtime.device)
        self.qkv = Linear(source.to_device_matrix(fused), bias, source.runtime.status)
        out_bias = source.vector(self.names["o"] + ".bias") if self.out_bias else None
        self.out = Linear(source.matrix(self.names["o"] + ".weight"), out_bias, source.runtime.status)
        self.tables = self.position.rotary_tables(source.runtime)
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        if self.tables is not None:
            cos, sin = self.tables
            if cos.shape != sin.shape or cos.dim() != 2 or not 0 < cos.shape[1] <= self.head_dim // 2:
                raise ValueError("attention: the position part's tables must be [max_positions, rotary_dim / 2] with "
                                 f"rotary_dim <= head_dim (got {tuple(cos.shape)} for head_dim {self.head_dim})")

    # ---- the step
    SPLIT_TOKENS = 256          # up to this many tokens the q/k/v product is split along K

    def _workspace(self):
        """A zeroed float32 buffer [SPLIT_TOKENS, width] that split-K products accumulate into;
        the rotary kernel reads it and sets it back to zero, so one buffer per model (its runtime)
        and width serves every layer and every step.  A step that fails in between leaves sums
        behind: the runtime zeroes its workspaces then (``Runtime.reset_workspaces``)."""
        return self.runtime.workspace(("qkv_sums", self.qkv.out_features), (self.SPLIT_TOKENS, self.qkv.out_features))

    def forward_with_norm(self, norm, x, ctx, cache: CacheView, state=None) -> bool:
        """The mixer with the norm before it folded into the q/k/v product, when the batch and the
        layer are small enough for that kernel; False means nothing was done."""
        if self.qkv.weight.dtype != torch.bfloat16 or getattr(norm, "fused_kind", None) != "rmsnorm":
            return False
        if x.shape[0] > self.qkv.small_tokens and not (UNSCALED_PRODUCT and self._decodes_fused(x.shape[0], ctx, cache)):
            return False
        self.forward(None, x, ctx, cache, state, norm=norm)
        return True

    def _decodes_fused(self, tokens, ctx, cache) -> bool:
        """One token per request, the projection's tail inside the attention kernel: then that kernel
        can also apply the norm's scale, and the q/k/v product takes the rows as they are."""
        return tokens <= self.SPLIT_TOKENS and ctx.max_q_len == 1 and cache.write and \
            kernels.decode_fusable(tokens, self.heads, self.kv_heads, self.head_dim, cache.block_table.shape[1] * cache.page_tokens)

    def forward(self, h, x, ctx, cache: CacheView, state=None, norm=None):
        cos, sin = self.tables if self.tables is not None else (None, None)
        tokens = x.shape[0]
        dtype = self.qkv.weight.dtype
        if dtype == torch.bfloat16 and tokens <= self.SPLIT_TOKENS:
            # few tokens: the product is a stream of weights, and a CTA streams only about 1/148 of
            # the memory bandwidth; split K so that every SM streams a share, accumulate in float32
            # and let the rotary kernel add the bias, rotate, convert and clear
            acc = self._workspace()[:tokens]
            scale = None              # (rows before the norm, eps): the attention kernel applies the norm's scale
            if norm is not None and tokens > self.qkv.small_tokens and self.qkv.accumulate_unscaled(norm, x, acc):
                scale = (x, norm.eps)
            elif norm is None or not self.qkv.accumulate_normed(norm, x, acc):
                self.qkv.accumulate(h if h is not None else norm.forward(x), acc)
            attended = torch.empty((tokens, self.heads * self.head_dim), dtype=dtype, device=x.device)
            max_keys = cache.block_table.shape[1] * cache.page_tokens
            if ctx.max_q_len == 1 and cache.write and kernels.decode_fusable(tokens, self.heads, self.kv_heads,
                                                                             self.head_dim, max_keys):
                # one token per request: bias, rotation and the cache append happen inside the attention kernel
                planned = ctx.planned_context or ctx.max_context
                plan = kernels.decode_attention_plan(tokens, self.heads, self.kv_heads, self.head_dim, cache.page_tokens,
                                                     max_keys, planned)
                if plan[0] == "resident":
                    kernels.attention_decode_resident(cache.k, cache.v, cache.block_table, ctx.context_lens, attended,
                                                      self.heads, self.kv_heads, self.head_dim, self.runtime.status, plan[1],
                                                      acc=acc, bias=self.qkv.bias, cos_table=cos, sin_table=sin,
                                                      interleaved=self.interleaved, norm_x=scale)
                else:
                    kernels.attention_decode_fused(acc, self.qkv.bias, cos, sin, cache.k, cache.v, cache.block_table,
                                                   ctx.context_lens, attended, self.heads, self.kv_heads, self.head_dim,
                                                   self.runtime.status, live_keys=planned, interleaved=self.interleaved,
                                                   norm_x=scale)
                self.out.forward(attended, residual=x)
                return
            if scale is not None:
                raise RuntimeError("attention: sums without the norm's scale can only go to the fused decode kernels")
            qkv = torch.empty((tokens, self.qkv.out_features), dtype=dtype, device=x.device)
            kernels.rope_append(qkv, ctx.positions, ctx.seq_of_token, cache.block_table, cos, sin, cache.k, cache.v,
                                self.heads, self.kv_heads, self.head_dim, cache.page_tokens, cache.write,
                                self.runtime.status, acc=acc, bias=self.qkv.bias, interleaved=self.interleaved)
        else:
            qkv = self.qkv.forward(h)
            kernels.rope_append(qkv, ctx.positions, ctx.seq_of_token, cache.block_table, cos, sin, cache.k, cache.v,
                                self.heads, self.kv_heads, self.head_dim, cache.page_tokens, cache.write,
                                self.runtime.status, interleaved=self.interleaved)
        q = qkv[:, :self.heads * self.head_dim]
        attended = torch.empty((tokens, self.heads * self.head_dim), dtype=qkv.dtype, device=qkv.device)
        kernels.paged_attention(q, cache, ctx, attended, self.heads, self.kv_heads, self.head_dim,
                                self.runtime.status)
        self.out.forward(attended, residual=x)
