"""The batch of one step: host description and its image on the device.

A step holds, for each request in it, the request's next tokens (a portion of a prompt, or a
single decoded token) and the places among them whose logits are wanted.  ``StepContext`` is
what every part receives: per-token arrays (token id, position, index of its request in the
batch), per-request arrays (start of its tokens, cache length after the step, state slot, block
table per cache group) and the rows whose logits are wanted.  All of it travels to the device
as one int32 buffer in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: ``tokens`` (a list of ints, or a 1-D integer numpy array for
    a long portion) continue the request's cache (``seq``) from position ``seq.length``; ``want``
    are indices into ``tokens`` whose logits are asked for."""
    seq: object
    tokens: list
    want: list = field(default_factory=list)


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    max_q_len: int
    max_context: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    q_start: torch.Tensor
    context_lens: torch.Tensor
    state_slots: torch.Tensor
    logits_rows: torch.Tensor
    block_tables: list
    page_tokens: int
    floats: dict = field(default_factory=dict)      # extra float32 arrays staged with the batch (sampling)
    # the longest context that the step's launches should be laid out for: the step's own, or, in a
    # captured graph, that of the steps it is replayed for (0: max_context)
    planned_context: int = 0

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class BatchStager:
    """Packs a step's arrays into pinned host memory and copies them to one device buffer."""

    def __init__(self, device, num_groups: int, capacity_ints: int = 1 << 16):
        self.device = device
        self.num_groups = num_groups
        self._capacity = 0
        self._host = [None, None]
        self._events = [None, None]
        self._flip = 0
        self._device_buf = None
        self.last_bytes = 0
        self._grow(capacity_ints)

    def _grow(self, ints: int):
        self._capacity = ints
        self._host = [torch.empty(ints, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._events = [None, None]
        self._device_buf = torch.empty(ints, dtype=torch.int32, device=self.device)

    @property
    def device_buffer(self) -> torch.Tensor:
        """The device image of the step's arrays (replaced when a larger one is needed)."""
        return self._device_buf

    def layout(self, T: int, R: int, S: int, max_pages: int, floats=None):
        sizes = [("token_ids", T), ("positions", T), ("seq_of_token", T), ("q_start", R + 1),
                 ("context_lens", R), ("state_slots", R), ("logits_rows", S)]
        sizes += [(f"float:{name}", len(values)) for name, values in (floats or {}).items()]
        sizes += [(f"table{g}", R * max_pages) for g in range(self.num_groups)]
        offsets, at = {}, 0
        for name, n in sizes:
            offsets[name] = (at, n)
            at += _pad4(max(n, 1))
        return offsets, at

    def stage(self, entries, page_tokens: int, fixed_pages: int | None = None, floats=None) -> StepContext:
        """Pack and copy.  ``fixed_pages`` fixes the block tables' width (a replayed CUDA graph
        needs the same layout every time); ``floats`` are extra float32 arrays (name -> values)
        that travel in the same copy."""
        R = len(entries)
        counts = [len(e.tokens) for e in entries]
        T = sum(counts)
        S = sum(len(e.want) for e in entries)
        context = [e.seq.length + n for e, n in zip(entries, counts)]
        max_pages = max(max((len(t) for t in e.seq.tables), default=0) for e in entries)
        max_pages = max(1, max_pages)
        if fixed_pages is not None:
            if max_pages > fixed_pages:
                raise ValueError("block table longer than the fixed table width")
            max_pages = fixed_pages
        offsets, total = self.layout(T, R, S, max_pages, floats)
        if total > self._capacity:
            self._grow(max(total, 2 * self._capacity))
        self._flip ^= 1
        if self._events[self._flip] is not None:
            self._events[self._flip].synchronize()
        host = self._host[self._flip]
        arr = host.numpy()

        def put(name, values):
            at, n = offsets[name]
            arr[at:at + n] = values

        q_start = np.zeros(R + 1, dtype=np.int32)
        np.cumsum(counts, out=q_start[1:])
        put("token_ids", np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries]))
        put("positions", np.concatenate([np.arange(e.seq.length, e.seq.length + n, dtype=np.int32)
                                         for e, n in zip(entries, counts)]))
        put("seq_of_token", np.repeat(np.arange(R, dtype=np.int32), counts))
        put("q_start", q_start)
        put("context_lens", np.asarray(context, dtype=np.int32))
        put("state_slots", np.asarray([e.seq.state_slot for e in entries], dtype=np.int32))
        rows = [q_start[i] + w for i, e in enumerate(entries) for w in e.want]
        if rows:
            put("logits_rows", np.asarray(rows, dtype=np.int32))
        for name, values in (floats or {}).items():
            put(f"float:{name}", np.asarray(values, dtype=np.float32).view(np.int32))
        for g in range(self.num_groups):
            table = np.full((R, max_pages), -1, dtype=np.int32)
            for i, e in enumerate(entries):
                pages = e.seq.tables[g]
                table[i, :len(pages)] = pages
            put(f"table{g}", table.reshape(-1))
        self._device_buf[:total].copy_(host[:total], non_blocking=True)
        self.last_bytes = total * 4
        event = torch.cuda.Event()
        event.record()
        self._events[self._flip] = event

        def view(name, shape=None):
            at, n = offsets[name]
            v = self._device_buf[at:at + n]
            return v.view(shape) if shape else v

        return StepContext(
            num_tokens=T, num_seqs=R, max_q_len=max(counts), max_context=max(context),
            token_ids=view("token_ids"), positions=view("positions"), seq_of_token=view("seq_of_token"),
            q_start=view("q_start"), context_lens=view("context_lens"), state_slots=view("state_slots"),
            logits_rows=view("logits_rows"),
            block_tables=[view(f"table{g}", (R, max_pages)) for g in range(self.num_groups)],
            page_tokens=page_tokens,
            floats={name: view(f"float:{name}").view(torch.float32) for name in (floats or {})})
