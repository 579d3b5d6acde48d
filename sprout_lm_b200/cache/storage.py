"""Device side of the cache: paged key/value buffers per cache slot and state buffers per layer.

``plan_groups`` sorts the model's cache slots into groups by what their mixers keep (all
positions, or a window of them); the host-side ``CacheManager`` hands out page ids per
group, and every slot of a group has buffers of its own indexed by those ids:
keys and values [pages, kv_heads, page_tokens, head_dim] in the compute dtype.
"""
from __future__ import annotations

import torch

from ..parts import CacheView, StateView
from .manager import CacheManager, GroupSpec


def plan_groups(model) -> tuple[list[GroupSpec], list[int]]:
    """(groups, group index of every cache slot; -1 for a slot whose mixer keeps nothing per token)."""
    keys: list[tuple] = []
    members: list[list[int]] = []
    slot_group = []
    for slot, spec in enumerate(model.cache_specs()):
        if spec is None:
            slot_group.append(-1)
            continue
        if spec.group_key not in keys:
            keys.append(spec.group_key)
            members.append([])
        index = keys.index(spec.group_key)
        members[index].append(slot)
        slot_group.append(index)
    groups = [GroupSpec(name=f"{kind}{window or ''}", kind=kind, window=window, slots=tuple(members[i]))
              for i, (kind, window) in enumerate(keys)]
    if not groups:
        groups = [GroupSpec(name="empty", kind="full", slots=())]
    return groups, slot_group


def state_slot_count(model, max_requests: int) -> int:
    return max_requests if any(spec is not None for spec in model.state_specs()) else 0


def cache_bytes_per_token(model, dtype: torch.dtype) -> int:
    item = torch.empty((), dtype=dtype).element_size()
    return sum(2 * spec.kv_heads * spec.head_dim * item for spec in model.cache_specs() if spec is not None)


class CapacityError(RuntimeError):
    """The cache pool asked for does not fit the device's free memory."""


RESERVE_BYTES = 1 << 30              # left free for activations, logits and graph pools


def check_capacity(model, slot_group: list[int], num_pages, page_tokens: int) -> None:
    """Refuse a pool that does not fit the device's free memory, before the host tables of its
    pages are built (a mistyped page count must cost neither minutes nor host memory).
    ``num_pages`` is one count for every group or a count per group."""
    runtime = model.runtime
    item = torch.empty((), dtype=runtime.dtype).element_size()
    counts = num_pages if not isinstance(num_pages, int) else [num_pages] * (max(slot_group, default=0) + 1)
    need = sum(2 * counts[slot_group[slot]] * spec.kv_heads * page_tokens * spec.head_dim * item
               for slot, spec in enumerate(model.cache_specs()) if spec is not None)
    free, _ = torch.cuda.mem_get_info(runtime.device)
    if need + RESERVE_BYTES > free:
        raise CapacityError(f"the cache pool needs {need / 2**30:.2f} GiB ({max(counts)} pages of "
                            f"{page_tokens} tokens) but only {free / 2**30:.2f} GiB of device memory is free "
                            f"(1 GiB is kept for activations); use fewer pages")


class CacheStorage:
    def __init__(self, model, manager: CacheManager, slot_group: list[int]):
        runtime = model.runtime
        check_capacity(model, slot_group, [pool.num_pages for pool in manager.pools], manager.page_tokens)
        self.manager = manager
        self.slot_group = slot_group
        self.page_tokens = manager.page_tokens
        self.keys, self.values = [], []
        for slot, spec in enumerate(model.cache_specs()):
            if spec is None:
                self.keys.append(None)
                self.values.append(None)
                continue
            pages = manager.pools[slot_group[slot]].num_pages
            shape = (pages, spec.kv_heads, self.page_tokens, spec.head_dim)
            self.keys.append(torch.zeros(shape, dtype=runtime.dtype, device=runtime.device))
            self.values.append(torch.zeros(shape, dtype=runtime.dtype, device=runtime.device))
        self.states = []
        for spec in model.state_specs():
            if spec is None:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((manager.state_slot_count, *spec.shape), dtype=spec.dtype,
                                               device=runtime.device))

    def view(self, slot: int, ctx, write: bool):
        if self.keys[slot] is None:
            return None
        return CacheView(self.keys[slot], self.values[slot], ctx.block_tables[self.slot_group[slot]],
                         self.page_tokens, write)

    def state_view(self, layer: int, ctx):
        if self.states[layer] is None:
            return None
        return StateView(self.states[layer], ctx.state_slots)

    def clear_state(self, slot: int) -> None:
        """Zero a state slot when a request takes it."""
        for buffer in self.states:
            if buffer is not None:
                buffer[slot].zero_()
