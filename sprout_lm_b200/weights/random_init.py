"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Which tensors exist, with which shapes, is asked of the model's own parts.  Matrices and
biases are N(0, 0.02), norm gains 1 + N(0, 0.02).  Every tensor has its own generator keyed
by (seed, tensor name), so the values do not depend on the order of generation.  With
``dtype="bfloat16"`` (the default) matrices are rounded to bfloat16 and stored so, while gains
and biases are stored in float32: the true 32-bit path and the bfloat16 path then read exactly
the same weights, and the folder mixes storage types as real checkpoints may.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import torch

from .safetensors_io import write_safetensors

STD = 0.02


def _generator(seed: int, name: str) -> np.random.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return np.random.Generator(np.random.Philox(key=int.from_bytes(digest[:16], "little")))


def random_tensor(seed: int, name: str, shape, init: str) -> torch.Tensor:
    values = _generator(seed, name).standard_normal(size=shape, dtype=np.float32) * np.float32(STD)
    if init == "gain":
        values += np.float32(1.0)
    elif init not in ("matrix", "bias"):
        raise ValueError(f"unknown init kind {init!r} for {name}")
    return torch.from_numpy(values)


def write_random_model(directory, config, seed: int = 0, dtype: str = "bfloat16") -> Path:
    """Create ``directory`` with config.json and model.safetensors for ``config`` (a typed
    configuration of a registered architecture)."""
    from ..models.decoder import DecoderModel
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("dtype must be 'bfloat16' or 'float32'")
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    model = DecoderModel(config.model_spec())
    tensors = {}
    for decl in model.tensor_decls():
        tensor = random_tensor(seed, decl.name, decl.shape, decl.init)
        as_bf16 = dtype == "bfloat16" and decl.init == "matrix"
        tensors[decl.name] = tensor.to(torch.bfloat16) if as_bf16 else tensor
    write_safetensors(directory / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    (directory / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    return directory
