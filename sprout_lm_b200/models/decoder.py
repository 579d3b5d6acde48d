"""A decoder built from a ``ModelSpec``: embedding, layers, run order, final norm, head.

Nothing here is specific to an architecture.  The run order is data
(``ModelSpec.order``): each entry names a layer and the cache slot its mixer reads and,
unless told otherwise, appends to; a layer may run more than once and may read a slot that
another layer filled.
"""
from __future__ import annotations

from pathlib import Path

import torch

from ..config import ModelSpec, load_config
from ..parts import Runtime, WeightSource, build_block, build_part
from ..weights.checkpoint import Checkpoint


WEIGHT_RESERVE_BYTES = 1 << 30       # left free beside the weights when a model is loaded


class WeightCapacityError(RuntimeError):
    """The model's weights do not fit the budget or the device's free memory."""


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks = [build_block(layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.runtime: Runtime | None = None
        self._decode_plans: dict = {}

    # ------------------------------------------------------------------ weights
    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensor_decls(self):
        decls, seen = [], set()
        for part in self.parts():
            for decl in part.tensor_decls():
                if decl.name in seen:
                    raise ValueError(f"two parts declare the tensor {decl.name}")
                seen.add(decl.name)
                decls.append(decl)
        return decls

    def weight_bytes(self, dtype: torch.dtype) -> int:
        """Device bytes of the resident weights at compute dtype ``dtype``: matrices in that dtype,
        gains and biases in float32."""
        item = torch.empty((), dtype=dtype).element_size()
        total = 0
        for decl in self.tensor_decls():
            count = 1
            for n in decl.shape:
                count *= n
            total += count * (item if decl.init == "matrix" else 4)
        return total

    def load(self, checkpoint: Checkpoint, runtime: Runtime, weight_budget_bytes: int | None = None,
             reserve_bytes: int = WEIGHT_RESERVE_BYTES) -> None:
        """Check the folder's tensors against what the parts declare, check that the weights fit
        the device, then load part by part.  Nothing is copied to the device before both checks
        have passed (the reference's resident upload refuses the same two ways,
        native/cuda-offload.cu:249-252)."""
        expected = {decl.name: decl.shape for decl in self.tensor_decls()}
        checkpoint.check(expected, ignorable=self.spec.ignorable_tensors)
        need = self.weight_bytes(runtime.dtype)
        if weight_budget_bytes is not None and need > weight_budget_bytes:
            raise WeightCapacityError(f"Resident weight budget exceeded: the model's weights take {need / 2**30:.2f} GiB, "
                                      f"the budget is {weight_budget_bytes / 2**30:.2f} GiB.")
        free, _ = torch.cuda.mem_get_info(runtime.device)
        if need + reserve_bytes > free:
            raise WeightCapacityError(f"Insufficient free CUDA memory after reserve: the model's weights take "
                                      f"{need / 2**30:.2f} GiB, {free / 2**30:.2f} GiB are free and "
                                      f"{reserve_bytes / 2**30:.2f} GiB are kept for the cache pool's start and activations.")
        source = WeightSource(lambda name: checkpoint.tensor(name, expected.get(name)), runtime)
        for part in self.parts():
            part.load(source)
        self.runtime = runtime

    # ------------------------------------------------------------------ what the cache manager must provide
    def cache_specs(self):
        """One CacheSpec (or None) per cache slot, taken from the layer that writes the slot."""
        specs = [None] * self.spec.cache_slots
        for call in self.spec.order:
            if call.writes_cache and specs[call.cache] is None:
                specs[call.cache] = self.blocks[call.layer].mixer.cache_spec()
        return specs

    def state_specs(self):
        """One StateSpec (or None) per layer."""
        return [block.mixer.state_spec() for block in self.blocks]

    def decode_plan(self, requests: int, max_keys: int, planned_context: int, page_tokens: int):
        """The parts' plans for a step of one token per request (see ``Part.decode_plan``)."""
        key = (requests, max_keys, planned_context, page_tokens)
        plan = self._decode_plans.get(key)
        if plan is None:
            if len(self._decode_plans) > 4096:
                self._decode_plans.clear()
            plan = self._decode_plans[key] = tuple(block.mixer.decode_plan(*key) for block in self.blocks)
        return plan

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, storage) -> torch.Tensor:
        """Run the step's tokens through the layers in run order; float32 logits
        [len(ctx.logits_rows), vocab], or None when no logits are wanted.  ``storage`` is the device side of the cache
        (``cache.storage.CacheStorage``)."""
        x = self.embedding.forward(ctx.token_ids)
        for call in self.spec.order:
            cache = storage.view(call.cache, ctx, write=call.writes_cache)
            state = storage.state_view(call.layer, ctx)
            self.blocks[call.layer].forward(x, ctx, cache, state)
        if ctx.logits_rows.numel() == 0:
            return None             # nothing wanted: the layers have filled the cache, the head is skipped
        return self.head.forward(self.final_norm.forward(x, rows=ctx.logits_rows))


def load_model(directory, dtype=torch.bfloat16, device="cuda:0", weight_budget_bytes: int | None = None):
    """Model of a folder (config.json + model.safetensors or an index of shards), chosen by
    the folder's config.json through the architecture registry.  ``weight_budget_bytes`` bounds the
    device memory the weights may take; a model beyond it, or beyond the device's free memory, is
    refused before its first tensor is copied."""
    directory = Path(directory)
    config = load_config(directory)
    model = DecoderModel(config.model_spec())
    runtime = Runtime(device, dtype)
    with Checkpoint(directory) as checkpoint:
        model.load(checkpoint, runtime, weight_budget_bytes=weight_budget_bytes)
    model.config = config
    return model
