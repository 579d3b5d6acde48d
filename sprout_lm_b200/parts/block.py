"""Arrangements of a layer's parts.  ``pre_norm``: x += mixer(norm_0(x)); x += ffn(norm_1(x))
(src/qwen.ts:164-200)."""
from __future__ import annotations

from ..config.specs import LayerSpec
from .base import Part, build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    def __init__(self, prefix: str, layer: LayerSpec):
        if len(layer.norms) != 2:
            raise ValueError("a pre_norm block has two norms")
        self.norms = [build_part("norm", spec, prefix) for spec in layer.norms]
        self.mixer = build_part("mixer", layer.mixer, prefix)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, prefix)

    def parts(self):
        return [*self.norms, self.mixer, self.feed_forward]

    def tensor_decls(self):
        return [decl for part in self.parts() for decl in part.tensor_decls()]

    def load(self, source):
        for part in self.parts():
            part.load(source)

    def forward(self, x, ctx, cache, state):
        # a mixer or a feed-forward may offer to take the norm before it into its own kernel
        fused = getattr(self.mixer, "forward_with_norm", None)
        if fused is None or not fused(self.norms[0], x, ctx, cache, state):
            self.mixer.forward(self.norms[0].forward(x), x, ctx, cache, state)
        fused = getattr(self.feed_forward, "forward_with_norm", None)
        if fused is None or not fused(self.norms[1], x, ctx):
            self.feed_forward.forward(self.norms[1].forward(x), x, ctx)


def build_block(layer: LayerSpec):
    from .base import _REGISTRY
    from ..config.specs import ConfigError
    try:
        cls = _REGISTRY["block"][layer.block]
    except KeyError:
        raise ConfigError(f"no block arrangement {layer.block!r} is registered") from None
    return cls(prefix=layer.prefix, layer=layer)
