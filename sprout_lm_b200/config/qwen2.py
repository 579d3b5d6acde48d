"""Typed configuration of the Qwen2 dense decoder, read from its config.json keys.

The checks are those of the reference's parser (src/qwen.ts:14-40): every key
is required, nothing has a default, and options that would change the
arithmetic (sliding window, scaled or multimodal rotary embedding, quantised
checkpoints, another activation) are refused before any weight is read.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .specs import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec

_INT_KEYS = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "vocab_size", "max_position_embeddings")
_FLOAT_KEYS = ("rms_norm_eps", "rope_theta")
_REFUSED_WHEN_SET = ("use_sliding_window", "rope_scaling", "quantization_config", "use_mrope")


def _is_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def parse_eos_ids(value, vocab_size: int) -> tuple[int, ...]:
    """An id or a non-empty list of ids, each inside the vocabulary; duplicates dropped
    (src/qwen.ts:36-40)."""
    ids = value if isinstance(value, list) else [value]
    if not ids or any(not _is_int(i) or i < 0 or i >= vocab_size for i in ids):
        raise ConfigError("Invalid EOS token IDs.")
    return tuple(dict.fromkeys(ids))


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...]

    architecture = "Qwen2ForCausalLM"
    model_type = "qwen2"

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen2Config":
        if not isinstance(raw, Mapping):
            raise ConfigError("Invalid Qwen config.")
        if raw.get("model_type") != "qwen2" or raw.get("hidden_act") != "silu":
            raise ConfigError("Only Qwen2 with SiLU is supported.")
        if any(raw.get(key) for key in _REFUSED_WHEN_SET):
            raise ConfigError("Sliding window, scaled/multimodal RoPE and quantized checkpoints are not supported.")
        for key in _INT_KEYS:
            if not _is_int(raw.get(key)) or raw[key] <= 0:
                raise ConfigError(f"Invalid model config: {key}.")
        for key in _FLOAT_KEYS:
            value = raw.get(key)
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value <= 0:
                raise ConfigError(f"Invalid model config: {key}.")
        if not isinstance(raw.get("tie_word_embeddings"), bool):
            raise ConfigError("tie_word_embeddings must be boolean.")
        heads, kv_heads, hidden = raw["num_attention_heads"], raw["num_key_value_heads"], raw["hidden_size"]
        if hidden % heads or (hidden // heads) % 2 or heads % kv_heads \
                or ("head_dim" in raw and raw["head_dim"] is not None and raw["head_dim"] != hidden // heads):
            raise ConfigError("Unsupported Qwen head dimensions.")
        eos = parse_eos_ids(raw.get("eos_token_id"), raw["vocab_size"])
        return cls(hidden_size=hidden, intermediate_size=raw["intermediate_size"],
                   num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=heads,
                   num_key_value_heads=kv_heads, vocab_size=raw["vocab_size"],
                   max_position_embeddings=raw["max_position_embeddings"],
                   rms_norm_eps=float(raw["rms_norm_eps"]), rope_theta=float(raw["rope_theta"]),
                   tie_word_embeddings=raw["tie_word_embeddings"], eos_token_ids=eos)

    def to_dict(self) -> dict:
        """The config.json that ``from_dict`` reads back to the same configuration."""
        eos = list(self.eos_token_ids)
        return {
            "architectures": [self.architecture], "model_type": self.model_type, "hidden_act": "silu",
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta, "tie_word_embeddings": self.tie_word_embeddings,
            "eos_token_id": eos[0] if len(eos) == 1 else eos,
            "use_sliding_window": False, "rope_scaling": None,
        }

    def with_eos(self, eos_token_id) -> "Qwen2Config":
        """generation_config.json's eos_token_id replaces config.json's (src/qwen.ts:124-128)."""
        from dataclasses import replace
        return replace(self, eos_token_ids=parse_eos_ids(eos_token_id, self.vocab_size))

    def model_spec(self) -> ModelSpec:
        """Layer by layer: pre-norm block, GQA attention with QKV bias and half-split rotary
        positions, SwiGLU feed-forward, learned RMSNorm (src/qwen.ts:164-203)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rope_half_split", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                                "max_positions": self.max_position_embeddings})
        layers = []
        for index in range(self.num_hidden_layers):
            prefix = f"model.layers.{index}."
            mixer = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "heads": self.num_attention_heads,
                "kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "qkv_bias": True, "out_bias": False, "position": position,
                "names": {"q": "self_attn.q_proj", "k": "self_attn.k_proj",
                          "v": "self_attn.v_proj", "o": "self_attn.o_proj"}})
            ffn = PartSpec("swiglu_mlp", {
                "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "names": {"gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}})
            norms = (PartSpec("rmsnorm", {**norm.params, "name": "input_layernorm"}),
                     PartSpec("rmsnorm", {**norm.params, "name": "post_attention_layernorm"}))
            layers.append(LayerSpec("pre_norm", prefix, mixer, ffn, norms))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                                   "name": "model.embed_tokens"}),
            layers=tuple(layers),
            order=tuple(LayerCall(layer=i, cache=i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {**norm.params, "name": "model.norm"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                      "tied_to": "model.embed_tokens" if self.tie_word_embeddings else None,
                                      "name": "lm_head"}),
            eos_token_ids=self.eos_token_ids,
            ignorable_tensors=("lm_head.weight",) if self.tie_word_embeddings else ())
