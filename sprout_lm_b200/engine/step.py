"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``ModelRunner`` owns the model, the cache manager (host) and the cache storage (device).
``step`` runs exactly the tokens it is given, as one batch: portions of prompts beside single
decoded tokens, cut anywhere.  It appends their keys and values to the requests' pages and
returns float32 logits at the wanted places.  It samples nothing and it does not advance the
requests' lengths until the launches have been issued without error.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels, sampling
from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, check_capacity, plan_groups, state_slot_count
from .batch import BatchStager, StepContext, StepEntry


class StepError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, model, num_pages: int, page_tokens: int = 16, max_requests: int = 64,
                 prefix_caching: bool = True):
        if model.runtime is None:
            raise StepError("the model has no weights loaded")
        self.model = model
        self.runtime = model.runtime
        groups, slot_group = plan_groups(model)
        check_capacity(model, slot_group, num_pages, page_tokens)
        self.manager = CacheManager(groups, num_pages, page_tokens,
                                    state_slots=state_slot_count(model, max_requests),
                                    prefix_caching=prefix_caching)
        self.storage = CacheStorage(model, self.manager, slot_group)
        self.stager = BatchStager(self.runtime.device, len(groups))
        self._groups_in_use = [g for g in range(len(groups)) if self.storage.slot_group.count(g)]   # groups that hold some layer's cache
        self.page_tokens = page_tokens
        self.max_requests = max_requests
        self.vocab_size = model.spec.vocab_size
        self.max_positions = model.spec.max_positions
        self.eos_token_ids = tuple(model.spec.eos_token_ids)
        self.steps_run = 0
        self.last_decode_graph = None      # the captured decode step that ran last
        self._ahead = None                 # (signature, graph, ticket, feed rows) of a decode step launched before it was asked for
        self._last_sampled: list = []      # the tokens of the decode step collected last (what a step launched behind it was fed)
        self.takes_next_step = True        # step_and_sample(..., then=...) launches the step after before it reads this one
        # what decode steps sample into and what a step launched behind another reads its tokens from
        self.fed_tokens = torch.zeros(max(1024, max_requests), dtype=torch.int32, device=self.runtime.device)
        self.ahead_used = 0                # such steps that the scheduler then asked for as launched
        self.ahead_dropped = 0             # and those it did not (their work is done again by the step that came instead)
        # bytes copied to and from the device by steps (the batch's arrays up, token ids or logits down)
        self.stats = {"h2d_bytes": 0, "d2h_bytes": 0}
        from .graphs import GraphCache, StepGraphs
        self.graphs = GraphCache(self)
        self.step_graphs = StepGraphs(self)

    # ------------------------------------------------------------------ requests' caches
    def new_sequence(self, tokens=None):
        """A request's cache; with ``tokens`` and prefix caching, starting from the longest
        published prefix of them."""
        seq = self.manager.reuse_prefix(tokens) if tokens is not None else self.manager.create()
        if seq.state_slot >= 0:
            self.storage.clear_state(seq.state_slot)
        return seq

    def reserve(self, seq, upto: int) -> bool:
        """Pages for all positions below ``upto`` in every group; False when the pool runs out
        (pages taken so far stay with the request)."""
        groups = range(len(self.manager.groups))
        while True:
            capacity = min(seq.capacity(g) for g in groups)
            if capacity >= upto:
                return True
            if not self.manager.reserve(seq, min(upto, capacity + self.page_tokens)):
                return False

    def release(self, seq) -> None:
        self.manager.release(seq)

    # ------------------------------------------------------------------ the step
    def validate(self, entries) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.vocab_size
        groups = self._groups_in_use
        for e in entries:
            if id(e.seq) in seen:
                raise StepError("a request appears twice in one step")
            seen.add(id(e.seq))
            if e.seq.released:
                raise StepError("a request's cache was released")
            tokens = e.tokens
            if len(tokens) == 0:
                raise StepError("an entry needs at least one token")
            if isinstance(tokens, np.ndarray):                   # a long portion, checked at once
                if tokens.ndim != 1 or tokens.dtype.kind != "i" or int(tokens.min()) < 0 or int(tokens.max()) >= vocab:
                    raise StepError("Invalid token ID.")
            else:
                for t in tokens:
                    if type(t) is not int or t < 0 or t >= vocab:
                        raise StepError("Invalid token ID.")
            end = e.seq.length + len(tokens)
            if end > self.max_positions:
                raise StepError("Invalid position: the request exceeds the model's context limit.")
            for g in groups:
                if e.seq.capacity(g) < end:
                    raise StepError("Reserve physical pages before running a token.")
            for w in e.want:
                if type(w) is not int or w < 0 or w >= len(tokens):
                    raise StepError("a wanted place lies outside the entry's tokens")

    # ------------------------------------------------------------------ a decode step launched ahead
    @staticmethod
    def _signature(entries, temperatures, uniforms, shift: int = 0):
        return (tuple((id(e.seq), e.seq.length + shift) for e in entries), tuple(temperatures), tuple(uniforms))

    def _launch_next(self, then) -> bool:
        """Start the decode step that follows the one just launched, before that one has been read
        back: ``then`` = (entries, temperatures, uniforms, feed_rows), the entries with placeholder
        tokens; request i's real token is row ``feed_rows[i]`` of the tokens the step in flight
        samples, and the launch takes it from there on the device.  The scheduler gives ``then``
        when it knows what the next step will be unless a request ends with this step's token; the
        next ``step_and_sample`` takes the result if it asks for just that batch, any other call
        waits for the launch and lets it go.  (What it wrote to the cache, the step that comes
        instead writes again; models with per-request state never launch ahead.)"""
        entries, temperatures, uniforms, feed_rows = then
        if self._ahead is not None or not self.graphs.enabled or self.manager.state_slot_count or not entries:
            return False
        if len(entries) > self.fed_tokens.numel() or any(len(e.tokens) != 1 or e.want != [0] for e in entries):
            return False
        for e in entries:
            if e.seq.released or e.seq.length + 2 > self.max_positions or not self.reserve(e.seq, e.seq.length + 2):
                return False                       # the planner decides what happens when pages run out
        graph = self.graphs.get(entries, shift=1)
        if graph.graph is None:
            return False                           # a first use runs eagerly and captures: through the ordinary path
        ticket = graph.launch(entries, temperatures, uniforms, shift=1, feed_rows=list(feed_rows))
        self._ahead = (self._signature(entries, temperatures, uniforms, shift=1), graph, ticket, list(feed_rows))
        return True

    def _take_ahead(self, entries, temperatures, uniforms):
        """(graph, ticket) of the step launched ahead if it is the step now asked for, else None
        (after waiting for it)."""
        if self._ahead is None:
            return None
        signature, graph, ticket, feed_rows = self._ahead
        self._ahead = None
        if entries is not None and all(len(e.tokens) == 1 and e.want == [0] for e in entries) \
                and signature == self._signature(entries, temperatures, uniforms) \
                and all(row < len(self._last_sampled) and e.tokens[0] == self._last_sampled[row]
                        for e, row in zip(entries, feed_rows)):
            self.ahead_used += 1
            return graph, ticket
        graph.collect(ticket)
        self.ahead_dropped += 1
        return None

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits [wanted places, vocab] in the order of the
        entries and of their ``want`` lists, or None when nothing is wanted.  The requests'
        lengths are advanced."""
        self._take_ahead(None, None, None)
        self.validate(entries)
        key, width = self.step_graphs.plan(entries, sample=False)
        ctx = self.stager.stage(entries, self.page_tokens, fixed_pages=width)
        if key is None:
            logits = self.forward(ctx)
        else:
            logits, _ = self.step_graphs.run(key, ctx, sample=False)
            if logits is not None:
                logits = logits.clone()       # a replay of the same sizes writes the same memory again
        for e in entries:
            e.seq.length += len(e.tokens)
            self.manager.trim(e.seq)
        self.steps_run += 1
        return logits

    def step_and_sample(self, entries: list[StepEntry], temperatures, uniforms, then=None) -> list[int]:
        """Run one batch and sample at every wanted place; the new token ids, in the order of the
        entries.  Only token ids come back from the device.  A batch of single decode tokens
        runs as a replayed CUDA graph; with ``then`` (see ``_launch_next``) the decode step after
        it is launched before this one's tokens are waited for."""
        self.validate(entries)
        decode_only = self.graphs.enabled and all(len(e.tokens) == 1 and e.want == [0] for e in entries)
        taken = self._take_ahead(entries, temperatures, uniforms)
        if decode_only:
            if taken is None:
                graph = self.graphs.get(entries)
                if graph.graph is None:
                    sampled = graph.run(entries, temperatures, uniforms)      # first use: runs eagerly, then captures
                    ticket = None
                else:
                    ticket = graph.launch(entries, temperatures, uniforms)
            else:
                graph, ticket = taken
            if ticket is not None:
                if then is not None:
                    self._launch_next(then)
                sampled = graph.collect(ticket)
            self.last_decode_graph = graph
            self._last_sampled = sampled
            self.stats["h2d_bytes"] += graph.stager.last_bytes
            self.stats["d2h_bytes"] += len(sampled) * 4
            for e in entries:
                e.seq.length += 1
                self.manager.trim(e.seq)
            self.steps_run += 1
            return sampled
        floats = {"temperature": temperatures, "uniform": uniforms} if temperatures else None
        key, width = self.step_graphs.plan(entries, sample=bool(temperatures))
        ctx = self.stager.stage(entries, self.page_tokens, fixed_pages=width, floats=floats)
        self.stats["h2d_bytes"] += self.stager.last_bytes
        if key is not None:
            _, tokens = self.step_graphs.run(key, ctx, sample=bool(temperatures))
        else:
            logits = self.forward(ctx)
            tokens = None
            if logits is not None:
                tokens = sampling.sample(logits, self.runtime.status, ctx.floats["temperature"], ctx.floats["uniform"])
        for e in entries:
            e.seq.length += len(e.tokens)
            self.manager.trim(e.seq)
        self.steps_run += 1
        if tokens is None:
            return []
        self.stats["d2h_bytes"] += tokens.numel() * 4
        return tokens.tolist()

    def decode_loop(self, entries, temperatures, uniforms, max_steps: int):
        """A device-side run of decode steps (see ``graphs.DecodeLoop``): pages for ``max_steps``
        more tokens per request are reserved here."""
        from .graphs import DecodeLoop
        self._take_ahead(None, None, None)
        for e in entries:
            if not self.reserve(e.seq, e.seq.length + 1 + max_steps):
                raise StepError("not enough pages for a device-side decode loop")
        self.validate(entries)
        return DecodeLoop(self, entries, temperatures, uniforms, max_steps)

    def forward(self, ctx: StepContext):
        try:
            return self.model.forward(ctx, self.storage)
        except BaseException:
            # a launch was refused between a product into a workspace and the kernel that empties it
            self.runtime.reset_workspaces()
            raise

    def check_status(self) -> None:
        """Read the device status word (synchronises); raise if a kernel flagged bad input.  A
        flagged step may have left sums in the accumulation workspaces: they are zeroed, so that the
        next step starts clean."""
        self._take_ahead(None, None, None)
        word = int(self.runtime.status.item())
        if word:
            self.runtime.status.zero_()
            self.runtime.reset_workspaces()
            raise StepError("device status: " + kernels.describe_status(word))

    # ------------------------------------------------------------------ sampling
    def sample(self, logits: torch.Tensor, temperatures=None, uniforms=None) -> torch.Tensor:
        """Token ids (int32, device) from float32 logits [rows, vocab]; a row is greedy where its
        temperature is 0, else drawn from softmax(logits / temperature) at its uniform number.
        ``temperatures`` and ``uniforms`` are tensors or sequences of floats, one per row."""
        def on_device(values):
            if values is None or isinstance(values, torch.Tensor):
                return values
            return torch.tensor(list(values), dtype=torch.float32).to(logits.device, non_blocking=True)
        if temperatures is not None and not isinstance(temperatures, torch.Tensor) and not any(temperatures):
            temperatures = uniforms = None
        return sampling.sample(logits, self.runtime.status, on_device(temperatures), on_device(uniforms))
