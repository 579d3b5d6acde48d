"""Plain, slow Qwen2 decoder for tests: whole sequences, no cache, no paging.

This file is the oracle that the engine is compared with.  It shares no code
with the package: it has its own reader for model folders and one function per
part of the architecture.  Storage is float32 and every sum is accumulated in
float64 and rounded to float32 when stored, which is how the reference's CPU
runner computes (JavaScript numbers are doubles, its arrays are Float32Array).

The reference's model code is TypeScript for Node and cannot be imported or
compiled in a Python/CUDA environment, so this implementation rests on the
reference's formulas (cited per function as ``file:line`` inside the reference
project).  It is anchored by the reference's own fixture
``test/fixtures/qwen-tiny`` (logits computed independently by the reference's
authors), which ``tests/test_plain_reference.py`` checks when that folder can
be found.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

F32 = np.float32
F64 = np.float64


# ----------------------------------------------------------------------------
# model folder reading (independent of the package's loader)
# ----------------------------------------------------------------------------

def read_safetensors(path) -> dict[str, np.ndarray]:
    """All tensors of one safetensors file, widened to float32.

    Container layout as in src/safetensors.ts:26-66 (8-byte little-endian
    header length, JSON header, data); BF16 widened by a 16-bit shift as in
    src/safetensors.ts:93.
    """
    raw = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + header_len].decode("utf-8"))
    data = memoryview(raw)[8 + header_len:]
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        buf = data[begin:end]
        if entry["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(F32)
        elif entry["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(F32)
        elif entry["dtype"] == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(F32)
        else:
            raise ValueError(f"unsupported dtype {entry['dtype']} for {name}")
        out[name] = arr.reshape(entry["shape"])
    return out


def read_model_folder(directory):
    """(config dict, tensors) of a folder with config.json and model.safetensors."""
    directory = Path(directory)
    config = json.loads((directory / "config.json").read_text())
    return config, read_safetensors(directory / "model.safetensors")


# ----------------------------------------------------------------------------
# one function per part
# ----------------------------------------------------------------------------

def embed(table: np.ndarray, tokens) -> np.ndarray:
    """Row copy, no scaling, no position added (src/qwen.ts:162-163)."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F32)


def linear(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None = None) -> np.ndarray:
    """y = W.x + b with W stored [out, in]; float64 sum, float32 store (src/qwen.ts:59-70)."""
    y = x.astype(F64) @ weight.astype(F64).T
    if bias is not None:
        y = y + bias.astype(F64)
    return y.astype(F32)


def rms_norm(x: np.ndarray, gain: np.ndarray, eps: float) -> np.ndarray:
    """scale = 1/sqrt(mean(x^2) + eps); out = fround(x*scale) * gain (src/qwen.ts:72-77).

    eps is added to the mean inside the root; the normalised value is rounded
    to float32 before it is multiplied by the learned gain (no ``1 +``).
    """
    x64 = x.astype(F64)
    scale = 1.0 / np.sqrt((x64 * x64).sum(axis=-1, keepdims=True) / x.shape[-1] + eps)
    normed = (x64 * scale).astype(F32)
    return (normed.astype(F64) * gain.astype(F64)).astype(F32)


def rope_half_split(x: np.ndarray, positions, head_dim: int, theta: float) -> np.ndarray:
    """Rotate pairs (d, d + head_dim/2) of every head (src/qwen.ts:81-92).

    ``x`` is [tokens, heads*head_dim]; angle = position / theta**(2d/head_dim),
    computed in float64.
    """
    tokens = x.shape[0]
    half = head_dim // 2
    heads = x.shape[1] // head_dim
    pos = np.asarray(positions, dtype=F64).reshape(tokens, 1, 1)
    d = np.arange(half, dtype=F64).reshape(1, 1, half)
    angle = pos / theta ** (2.0 * d / head_dim)
    cos, sin = np.cos(angle), np.sin(angle)
    xs = x.astype(F64).reshape(tokens, heads, head_dim)
    a, b = xs[..., :half], xs[..., half:]
    out = np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)
    return out.reshape(tokens, heads * head_dim).astype(F32)


def causal_gqa_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray,
                         heads: int, kv_heads: int, head_dim: int) -> np.ndarray:
    """Attention of every position over positions 0..itself (src/qwen.ts:175-193).

    Query head h reads key/value head floor(h / (heads/kv_heads)); the score is
    the dot divided by sqrt(head_dim); scores, exponentials and probabilities
    are each rounded to float32 between the stages; sums are float64.
    """
    tokens = q.shape[0]
    group = heads // kv_heads
    out = np.zeros((tokens, heads * head_dim), dtype=F32)
    root = np.sqrt(F64(head_dim))
    for h in range(heads):
        g = h // group
        qh = q[:, h * head_dim:(h + 1) * head_dim].astype(F64)
        kh = k[:, g * head_dim:(g + 1) * head_dim].astype(F64)
        vh = v[:, g * head_dim:(g + 1) * head_dim].astype(F64)
        for t in range(tokens):
            scores = ((kh[:t + 1] @ qh[t]) / root).astype(F32)
            e = np.exp(scores.astype(F64) - F64(scores.max())).astype(F32)
            p = (e.astype(F64) / e.astype(F64).sum()).astype(F32)
            out[t, h * head_dim:(h + 1) * head_dim] = (p.astype(F64) @ vh[:t + 1]).astype(F32)
    return out


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """fround(g / (1 + exp(-g))) * u (src/qwen.ts:199)."""
    g = gate.astype(F64)
    silu = (g / (1.0 + np.exp(-g))).astype(F32)
    return (silu.astype(F64) * up.astype(F64)).astype(F32)


def residual_add(x: np.ndarray, delta: np.ndarray) -> np.ndarray:
    """Element-wise float32 sum (src/qwen.ts:79)."""
    return (x.astype(F64) + delta.astype(F64)).astype(F32)


# ----------------------------------------------------------------------------
# the arrangement of the parts
# ----------------------------------------------------------------------------

def decoder_layer(x, w, prefix, cfg, positions):
    """norm -> q,k,v(+bias) -> rope -> attention -> o + residual -> norm -> SwiGLU MLP + residual
    (src/qwen.ts:164-200)."""
    heads = cfg["num_attention_heads"]
    kv_heads = cfg["num_key_value_heads"]
    head_dim = cfg["hidden_size"] // heads
    eps = cfg["rms_norm_eps"]
    h = rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    q = linear(h, w[prefix + "self_attn.q_proj.weight"], w[prefix + "self_attn.q_proj.bias"])
    k = linear(h, w[prefix + "self_attn.k_proj.weight"], w[prefix + "self_attn.k_proj.bias"])
    v = linear(h, w[prefix + "self_attn.v_proj.weight"], w[prefix + "self_attn.v_proj.bias"])
    q = rope_half_split(q, positions, head_dim, cfg["rope_theta"])
    k = rope_half_split(k, positions, head_dim, cfg["rope_theta"])
    attended = causal_gqa_attention(q, k, v, heads, kv_heads, head_dim)
    x = residual_add(x, linear(attended, w[prefix + "self_attn.o_proj.weight"]))
    f = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    t = swiglu(linear(f, w[prefix + "mlp.gate_proj.weight"]), linear(f, w[prefix + "mlp.up_proj.weight"]))
    return residual_add(x, linear(t, w[prefix + "mlp.down_proj.weight"]))


def hidden_states(cfg: dict, w: dict, tokens, layers=None) -> np.ndarray:
    """Residual stream after the last layer for a whole sequence, [tokens, hidden]."""
    positions = np.arange(len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens)
    count = cfg["num_hidden_layers"] if layers is None else layers
    for l in range(count):
        x = decoder_layer(x, w, f"model.layers.{l}.", cfg, positions)
    return x


def logits(cfg: dict, w: dict, tokens) -> np.ndarray:
    """Logits at every position of a whole sequence, [tokens, vocab] (src/qwen.ts:203).

    The head is the embedding matrix itself when ``tie_word_embeddings``
    (src/qwen.ts:152).
    """
    x = hidden_states(cfg, w, tokens)
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]), head)


def greedy(cfg: dict, w: dict, prompt, count: int) -> list[int]:
    """Greedy continuation; the lowest index wins a tie (src/runner.ts:38-42)."""
    history = list(prompt)
    out = []
    for _ in range(count):
        token = int(np.argmax(logits(cfg, w, history)[-1]))
        out.append(token)
        history.append(token)
    return out
