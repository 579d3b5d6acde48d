"""sprout_lm_b200: a small, whole inference engine for one NVIDIA B200.

Public entry points: ``load_model`` (a model folder -> a model on the GPU, chosen by its
config.json), ``generate`` (prompts in, tokens out), ``Engine`` / ``EngineOptions`` (the
scheduler: add, step, cancel, result), ``ModelRunner`` (the step function and the cache),
``write_random_model`` (the random-weights mode).
"""
from .config import ConfigError, Qwen2Config, load_config, parse_config, register_architecture
from .engine.scheduler import Engine, EngineOptions
from .weights import WeightError, write_random_model

__version__ = "0.1.0"


def load_model(directory, dtype="bfloat16", device="cuda:0", weight_budget_bytes=None):
    import torch
    from .models import load_model as _load
    if isinstance(dtype, str):
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    return _load(directory, dtype=dtype, device=device, weight_budget_bytes=weight_budget_bytes)


def generate(model, prompts, max_new_tokens=16, **kwargs):
    from .engine.generate import generate as _generate
    return _generate(model, prompts, max_new_tokens, **kwargs)


def make_engine(model, options=None):
    from .engine.generate import make_engine as _make
    return _make(model, options)


def __getattr__(name):
    if name == "ModelRunner":
        from .engine.step import ModelRunner
        return ModelRunner
    raise AttributeError(name)


__all__ = ["ConfigError", "Engine", "EngineOptions", "Qwen2Config", "WeightError", "generate", "load_config",
           "load_model", "make_engine", "parse_config", "register_architecture", "write_random_model"]
