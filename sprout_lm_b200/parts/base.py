"""Interfaces of the parts that a layer is put together from, and their registries.

A part is built from a ``PartSpec`` (its kind and its constants), says which checkpoint
tensors it reads (``tensor_decls``), loads them (``load``) and runs on the tokens of one step
(``forward``).  No part knows which model it is in: sizes and constants are constructor
parameters, tensor names are a prefix plus names given in the spec.

Categories and what each must provide:

* ``norm``:          ``forward(x, rows=None) -> h``.  ``x`` is the float32 residual stream
                     [tokens, hidden]; ``h`` has the compute dtype.  ``rows`` (int32 indices)
                     selects the rows to produce.
* ``position``:      ``rotary_tables(runtime) -> (cos, sin) | None``: float32 tables
                     [max_positions, rotary_dim / 2] (None: no rotation).  The first
                     ``rotary_dim`` elements of a head turn, pair d by the angle whose cosine and
                     sine stand at [position, d]; pairs are (d, d + rotary_dim / 2), or (2d, 2d + 1)
                     when the part has a true attribute ``interleaved``.
* ``mixer``:         ``cache_spec() -> CacheSpec | None`` (what it keeps per token),
                     ``state_spec() -> StateSpec | None`` (what it keeps per request, of fixed
                     size), ``forward(h, x, ctx, cache, state)``: reads the normed activations
                     ``h``, adds its output to ``x`` in place.
* ``feed_forward``:  ``forward(h, x, ctx)``: adds its output to ``x`` in place.
* ``block``:         arranges a layer's norms, mixer and feed-forward:
                     ``forward(x, ctx, cache, state)``.
* ``embedding``:     ``forward(token_ids) -> x`` (float32 [tokens, hidden]).
* ``head``:          ``forward(h) -> logits`` (float32 [rows, vocab]).

``ctx`` is the step's batch on the device (``engine.batch.StepContext``); ``cache`` a
``CacheView`` of the cache slot the call reads (and writes); ``state`` a ``StateView`` or None.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from ..config.specs import ConfigError, PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str) -> Callable[[type], type]:
    """Class decorator: make ``kind`` constructible for ``category``."""
    if category not in _REGISTRY:
        raise ConfigError(f"unknown part category {category!r}")

    def decorate(cls: type) -> type:
        _REGISTRY[category][kind] = cls
        cls.category = category
        cls.kind = kind
        return cls
    return decorate


def build_part(category: str, spec: PartSpec, prefix: str = ""):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {})))
        raise ConfigError(f"no {category} part of kind {spec.kind!r} is registered (known: {known})") from None
    return cls(prefix=prefix, **spec.params)


def registered_parts(category: str) -> tuple[str, ...]:
    return tuple(sorted(_REGISTRY[category]))


@dataclass(frozen=True)
class TensorDecl:
    """A checkpoint tensor that a part reads.  ``init`` tells the random-weights mode how to
    fill it: ``matrix`` and ``bias`` are N(0, 0.02), ``gain`` is 1 + N(0, 0.02)."""
    name: str
    shape: tuple[int, ...]
    init: str = "matrix"


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token: keys and values of ``kv_heads`` heads of ``head_dim``.
    kind ``full`` keeps every position, ``window`` the last ``window``."""
    kv_heads: int
    head_dim: int
    kind: str = "full"
    window: int | None = None

    @property
    def group_key(self):
        return (self.kind, self.window)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: a tensor of ``shape`` and ``dtype`` per request."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """One cache slot as a mixer call sees it: paged keys and values
    [pages, kv_heads, page_tokens, head_dim], the block tables of the slot's group
    [requests, max_pages] and whether this call appends to the slot."""
    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_tokens: int
    write: bool


@dataclass
class StateView:
    """A layer's state buffer [slots, *shape] and the slot of each request of the step."""
    buffer: torch.Tensor
    slots: torch.Tensor


class Runtime:
    """Where and how a model computes: the device, the compute dtype (float32 for the true
    32-bit path, bfloat16 for serving), the device status word that kernels set instead of
    faulting, and what the model's parts share on the device: zeroed accumulation workspaces
    (``workspace``) and read-only tables such as rotary cosines (``shared``)."""

    def __init__(self, device="cuda:0", dtype=torch.bfloat16):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("sprout_lm_b200 computes on a CUDA device only; there is no CPU path.")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; sprout_lm_b200 has no CPU fallback.")
        self.dtype = dtype
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sm_count = int(torch.cuda.get_device_properties(self.device).multi_processor_count)
        self._workspaces: dict = {}
        self._shared: dict = {}

    def workspace(self, key, shape, dtype=torch.float32) -> torch.Tensor:
        """A zeroed buffer that belongs to this runtime (one model's steps on one stream), made at
        first use.  Whoever accumulates into it leaves it zero again; after a step that failed or
        that flagged its input, ``reset_workspaces`` restores that."""
        buffer = self._workspaces.get(key)
        if buffer is None:
            buffer = self._workspaces[key] = torch.zeros(shape, dtype=dtype, device=self.device)
        return buffer

    def reset_workspaces(self) -> None:
        for buffer in self._workspaces.values():
            buffer.zero_()

    def shared(self, key, build):
        """A read-only device object kept once per runtime (``build()`` makes it at first use): the
        layers of a model share one copy of what depends only on their constants."""
        if key not in self._shared:
            self._shared[key] = build()
        return self._shared[key]


class WeightSource:
    """Hands checkpoint tensors to parts, on the device, each name loaded once.

    ``matrix`` gives a tensor in the compute dtype (a float32 or float16 matrix is rounded to
    bfloat16, to nearest even, on the bfloat16 path: tensor cores take nothing wider);
    ``vector`` gives float32 whatever the stored dtype (widening is exact), so gains and biases
    stored in 32-bit stay 32-bit on both paths.
    """

    def __init__(self, fetch: Callable[[str], torch.Tensor], runtime: Runtime):
        self._fetch = fetch
        self.runtime = runtime
        self._matrices: dict[str, torch.Tensor] = {}

    def raw(self, name: str) -> torch.Tensor:
        return self._fetch(name)

    def matrix(self, name: str) -> torch.Tensor:
        if name not in self._matrices:
            self._matrices[name] = self.to_device_matrix(self._fetch(name))
        return self._matrices[name]

    def to_device_matrix(self, cpu_tensor: torch.Tensor) -> torch.Tensor:
        return cpu_tensor.to(self.runtime.dtype).to(self.runtime.device).contiguous()

    def vector(self, name: str) -> torch.Tensor:
        return self._fetch(name).to(torch.float32).to(self.runtime.device).contiguous()


class Part:
    category = ""
    kind = ""

    def tensor_decls(self) -> list[TensorDecl]:
        return []

    def load(self, source: WeightSource) -> None:
        pass

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        """What this part's launches for a step of one token per request depend on beyond the
        number of requests and the block tables' width (something hashable, or None): a captured
        step is replayed only for steps with the same plan.  ``max_keys`` is the tables' width in
        tokens, ``planned_context`` the longest context the step is laid out for, ``page_tokens``
        the cache's page size."""
        return None
