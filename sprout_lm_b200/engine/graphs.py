"""Decode steps as replayed CUDA graphs.

A decode step of a small model is a hundred-odd short kernels; launched one by one from the
host they cost more than they run.  For steps in which every request brings exactly one token
the runner captures the whole step (all layers, the head, sampling) once per batch size into
a CUDA graph over fixed device buffers; afterwards a step is one copy of the batch's arrays
into those buffers and one graph launch.  ``DecodeLoop`` goes further for runs of decode steps
that need no host decision in between: a small kernel feeds the sampled tokens back as the
next inputs on the device, so the steps replay back to back.
"""
from __future__ import annotations

import contextlib
import gc

import numpy as np
import torch

from .. import kernels, sampling
from .batch import StepContext


@contextlib.contextmanager
def guarded_capture(graph: "torch.cuda.CUDAGraph"):
    """Stream capture into ``graph`` on a side stream.

    Freeing an older graph while a new one is being captured is a CUDA call that invalidates the
    capture, so the garbage collector rests meanwhile (objects freed by reference count are the
    caller's business).  The capture is begun and ended directly: ``torch.cuda.graph`` would
    synchronise the device, collect garbage and empty the allocator's cache first, some 30 ms that
    a serving loop which captures new step shapes as they come cannot afford."""
    was_enabled = gc.isenabled()
    gc.disable()
    current = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    side.wait_stream(current)
    try:
        with torch.cuda.stream(side):
            graph.capture_begin(capture_error_mode="relaxed")
            try:
                yield
            finally:
                graph.capture_end()
        current.wait_stream(side)
    finally:
        if was_enabled:
            gc.enable()


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class DecodeGraph:
    """One captured decode step for ``requests`` requests and block tables ``table_pages`` wide.

    The step's arrays live in one device buffer with a fixed layout, mirrored by a host array that
    is updated in place: token ids, positions and lengths every step, block-table cells only where
    a request's table grew (or wholly, when the requests of the step changed).  A launch copies
    the mirror into one of a few pinned buffers and from there to the device, replays the captured
    kernels and copies the sampled tokens into pinned memory; an event marks its end, so that a
    second step can be launched before the first one's tokens are read (``launch`` / ``collect``).
    Such a step takes its input tokens on the device, from the tokens the step before sampled
    (``feed_rows``): the captured kernels begin with that gather and sample into the runner's
    ``fed_tokens``."""

    RING = 3            # pinned buffers per graph: more launches than two are never in flight

    def __init__(self, runner, requests: int, table_pages: int, planned_context: int = 0):
        self.runner = runner
        self.requests = R = requests
        self.table_pages = table_pages
        self.groups = len(runner.manager.groups)
        device = runner.runtime.device
        sizes = [("token_ids", R), ("positions", R), ("seq_of_token", R), ("q_start", R + 1), ("context_lens", R),
                 ("state_slots", R), ("logits_rows", R), ("temperature", R), ("uniform", R), ("feed_rows", R)]
        sizes += [(f"table{g}", R * table_pages) for g in range(self.groups)]
        self.offsets, at = {}, 0
        for name, n in sizes:
            self.offsets[name] = (at, n)
            at += (n + 3) & ~3
        self.total = at
        self.array = np.zeros(at, dtype=np.int32)
        self.floats = self.array.view("float32")
        self.pinned = [torch.zeros(at, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.pinned_tokens = [torch.zeros(R, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING          # the end of the launch that used the slot last, until it is collected
        self.slot = 0
        self.device_buf = torch.zeros(at, dtype=torch.int32, device=device)
        self.last_bytes = at * 4
        # what a capture keeps on the device, roughly: the logits, and the activations of a layer or two
        self.nbytes = R * runner.vocab_size * 4 + at * 4 + R * (1 << 18) + (1 << 20)
        put = self._put
        put("seq_of_token", range(R))
        put("q_start", range(R + 1))
        put("logits_rows", range(R))
        put("feed_rows", [-1] * R)
        for g in range(self.groups):
            put(f"table{g}", [-1] * (R * table_pages))
        view = self._view
        self.ctx = StepContext(
            num_tokens=R, num_seqs=R, max_q_len=1, max_context=table_pages * runner.page_tokens,
            token_ids=view("token_ids"), positions=view("positions"), seq_of_token=view("seq_of_token"),
            q_start=view("q_start"), context_lens=view("context_lens"), state_slots=view("state_slots"),
            logits_rows=view("logits_rows"),
            block_tables=[view(f"table{g}").view(R, table_pages) for g in range(self.groups)],
            page_tokens=runner.page_tokens,
            floats={"temperature": view("temperature").view(torch.float32), "uniform": view("uniform").view(torch.float32)},
            planned_context=planned_context)
        self._seqs = None
        self._known = None                # pages of each request's tables already in the host mirror
        self.graph = None
        self.tokens = None
        self.logits = None
        self.last_logits = None           # float32 [requests, vocab] of the step that ran last (tests read them)
        self.launches = 0

    def _put(self, name, values):
        at, n = self.offsets[name]
        self.array[at:at + n] = values

    def _view(self, name):
        at, n = self.offsets[name]
        return self.device_buf[at:at + n]

    @property
    def stager(self):                     # the bytes of the last copy, for the runner's statistics
        return self

    def stage(self, entries, temperatures, uniforms, copy: bool = True, shift: int = 0, feed_rows=None) -> StepContext:
        """Fill the host mirror; with ``copy`` also send it to the device.  ``shift``: the requests
        will be this many tokens longer when the step runs than they are now (a step launched
        behind one that is still in flight); ``feed_rows``: per request the row of the step before
        whose sampled token is this step's input, taken on the device (the staged token ids are
        placeholders then)."""
        R, P = self.requests, self.table_pages
        lengths = [e.seq.length + shift for e in entries]
        self._put("token_ids", [e.tokens[0] for e in entries])
        self._put("positions", lengths)
        self._put("context_lens", [n + 1 for n in lengths])
        self._put("feed_rows", feed_rows if feed_rows is not None else [-1] * R)
        at, n = self.offsets["temperature"]
        self.floats[at:at + n] = temperatures
        at, n = self.offsets["uniform"]
        self.floats[at:at + n] = uniforms
        same = self._seqs is not None and all(e.seq is s for e, s in zip(entries, self._seqs))
        if not same:
            self._seqs = [e.seq for e in entries]
            self._known = [[0] * R for _ in range(self.groups)]
            self._put("state_slots", [e.seq.state_slot for e in entries])
            for g in range(self.groups):
                self._put(f"table{g}", [-1] * (R * P))
        for g in range(self.groups):
            base = self.offsets[f"table{g}"][0]
            known = self._known[g]
            for i, e in enumerate(entries):
                pages = e.seq.tables[g]
                count = len(pages)
                if count > P:
                    raise ValueError("block table longer than the graph's table width")
                if count != known[i] or not same:
                    # window groups rewrite cells that were given back (-1): take the whole row then
                    lo = 0 if self.runner.manager.groups[g].kind == "window" else known[i]
                    self.array[base + i * P + lo:base + i * P + count] = pages[lo:]
                    known[i] = count
                elif self.runner.manager.groups[g].kind == "window":
                    self.array[base + i * P:base + i * P + count] = pages
        if copy:
            self._send()
        return self.ctx

    def _send(self) -> int:
        """The mirror -> the next pinned buffer -> the device; the slot used."""
        slot = self.slot
        self.slot = (slot + 1) % self.RING
        if self.events[slot] is not None:
            self.events[slot].synchronize()       # an uncollected launch still owns the buffer
            self.events[slot] = None
        self.pinned[slot].numpy()[:] = self.array
        self.device_buf.copy_(self.pinned[slot], non_blocking=True)
        return slot

    def _forward(self, ctx):
        logits = self.runner.model.forward(ctx, self.runner.storage)
        tokens = sampling.sample(logits, self.runner.runtime.status, ctx.floats["temperature"], ctx.floats["uniform"],
                                 out=self.runner.fed_tokens[:self.requests])
        return logits, tokens

    def _finish(self, slot: int) -> int:
        self.pinned_tokens[slot].copy_(self.tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[slot] = event
        return slot

    def run(self, entries, temperatures, uniforms) -> list:
        """Stage the batch and run the step; the sampled token ids, on the host."""
        if self.graph is None:
            # First use: this call's step runs eagerly (that also does the kernels' first-use
            # set-up), then the same launches are captured for later calls.  Capturing records
            # without running, so the step has run exactly once: a mixer that updates
            # per-request state must not see a step twice.
            ctx = self.stage(entries, temperatures, uniforms)
            self.last_logits, tokens = self._forward(ctx)
            result = tokens.tolist()
            before = kernels.LAUNCHES
            graph = torch.cuda.CUDAGraph()
            with guarded_capture(graph):
                kernels.feed_tokens(ctx.token_ids, self._view("feed_rows"), self.runner.fed_tokens, self.runner.vocab_size)
                self.logits, self.tokens = self._forward(ctx)
            self.launches = kernels.LAUNCHES - before
            self.graph = graph
            return result
        return self.collect(self.launch(entries, temperatures, uniforms))

    def launch(self, entries, temperatures, uniforms, shift: int = 0, feed_rows=None) -> int:
        """Stage the batch and start the captured step; ``collect`` with the returned ticket waits
        for it.  The host is free in between, and may launch the step after it."""
        self.stage(entries, temperatures, uniforms, copy=False, shift=shift, feed_rows=feed_rows)
        slot = self._send()
        self.graph.replay()
        return self._finish(slot)

    def collect(self, slot: int) -> list:
        self.events[slot].synchronize()                # the tokens are in pinned memory
        self.events[slot] = None
        self.last_logits = self.logits
        return self.pinned_tokens[slot].tolist()


class GraphCache:
    """Captured decode steps, by (number of requests, table width, the parts' launch plans).

    A serving loop meets many keys: every batch size on the way up and down, a wider table every
    ``page_multiple`` pages, another attention plan every few 128 keys of context; a run of 64
    requests uses some thirty.  Each capture owns device memory (its activations and its [requests,
    vocabulary] float32 logits), pinned mirrors and a CUDA graph, so the cache is bounded: at most
    ``limit`` captures and ``budget_bytes`` of what they hold (``DecodeGraph.nbytes``, an estimate led
    by the logits; by default 1/24 of the device's memory).  Beyond either the least recently used
    capture is dropped (outside any capture: ``get`` runs before the step is staged).  The bounds
    are generous on purpose: a capture costs some ten milliseconds, a dropped one that is needed
    again costs them again."""

    def __init__(self, runner, page_multiple: int = 64, limit: int = 256, budget_bytes: int | None = None):
        self.runner = runner
        self.page_multiple = page_multiple
        self.limit = max(1, limit)
        if budget_bytes is None:
            device = getattr(getattr(runner, "runtime", None), "device", None)
            total = torch.cuda.get_device_properties(device).total_memory if device is not None and torch.cuda.is_available() else 0
            budget_bytes = total // 24 if total else 1 << 62
        self.budget_bytes = budget_bytes
        self.graphs: dict = {}             # insertion order is the order of last use
        self.enabled = True
        self.evictions = 0
        self.keys_used = 0                 # keys asked for that were not held (captures made or to be made)

    def held_bytes(self) -> int:
        return sum(getattr(g, "nbytes", 0) for g in self.graphs.values())

    def key_for(self, entries, shift: int = 0):
        pages = 1
        for e in entries:
            for table in e.seq.tables:
                if len(table) > pages:
                    pages = len(table)
        # A graph serves the steps of its number of requests and table width whose parts lay their
        # launches out alike: the parts say what theirs depend on (decode attention: how it
        # divides the keys, which follows the contexts' length in steps of 128).
        width = _round_up(pages, self.page_multiple)
        longest = 1 + shift + max(e.seq.length for e in entries)
        planned = min(width * self.runner.page_tokens, _round_up(longest, 128))
        plan = self.runner.model.decode_plan(len(entries), width * self.runner.page_tokens, planned, self.runner.page_tokens)
        return (len(entries), width, plan), width, planned

    def get(self, entries, shift: int = 0) -> DecodeGraph:
        key, width, planned = self.key_for(entries, shift)
        graph = self.graphs.pop(key, None)
        if graph is None:
            self.keys_used += 1
            graph = self.make(len(entries), width, planned)
            room = self.budget_bytes - getattr(graph, "nbytes", 0)
            while self.graphs and (len(self.graphs) >= self.limit or self.held_bytes() > room):
                oldest = next(iter(self.graphs))
                del self.graphs[oldest]    # its CUDA graph, buffers and pinned mirrors go with it
                self.evictions += 1
        self.graphs[key] = graph           # most recently used: last
        return graph

    def make(self, requests: int, width: int, planned: int) -> DecodeGraph:
        return DecodeGraph(self.runner, requests, width, planned)


class StepGraphs:
    """Steps with prompt portions, replayed when their shape comes again.

    A prefill step of a small model is two hundred launches that the host enqueues more slowly
    than the device runs them.  A step whose sizes (tokens, requests, wanted rows, block-table
    width rounded up to ``page_multiple``) have come ``after`` times is captured after it has
    run, and later steps of the same sizes replay the capture: the batch's arrays live at fixed
    offsets of the stager's device buffer, so only their contents change.  Chunked prefill of
    long prompts at a fixed chunk size makes such steps; the mixed steps of a busy server rarely
    repeat their sizes, and a capture costs milliseconds and holds its own activations, so sizes
    must have come three times first, a few captures are kept, and steps that ask for many
    logits rows are not captured.  When the captures are full, a new shape takes the place of the
    least used one only once it has been used twice as often (uses are halved now and then, so
    the count follows the recent past): shapes that take turns do not capture over one another."""

    def __init__(self, runner, limit: int = 4, min_tokens: int = 128, max_rows: int = 64, page_multiple: int = 64,
                 after: int = 3):
        self.runner = runner
        self.limit, self.min_tokens, self.max_rows, self.page_multiple = limit, min_tokens, max_rows, page_multiple
        self.after = after
        self.seen: dict = {}              # key -> times used of late (run eagerly or replayed)
        self.captured: dict = {}          # key -> (graph, logits, tokens, device buffer)
        self.enabled = True
        self.replays = 0
        self._steps = 0

    def plan(self, entries, sample: bool):
        """(key, table width) for a step that may be captured, else (None, None)."""
        if not self.enabled:
            return None, None
        tokens = sum(len(e.tokens) for e in entries)
        rows = sum(len(e.want) for e in entries)
        if tokens < self.min_tokens or rows > self.max_rows or all(len(e.tokens) == 1 for e in entries):
            return None, None
        pages = 1
        for e in entries:
            for table in e.seq.tables:
                pages = max(pages, len(table))
        width = _round_up(pages, self.page_multiple)
        return (tokens, len(entries), rows, width, sample), width

    def run(self, key, ctx, sample: bool):
        """Run the staged step ``ctx``; (logits or None, sampled tokens or None), both on the
        device and valid until the next step of the same sizes."""
        runner = self.runner
        buffer = runner.stager.device_buffer
        self._steps += 1
        if self._steps % 1024 == 0:       # the counts follow the recent past
            self.seen = {k: n // 2 for k, n in self.seen.items() if n >= 2 or k in self.captured}
        uses = self.seen[key] = self.seen.get(key, 0) + 1
        held = self.captured.get(key)
        if held is not None and held[3] is buffer:
            held[0].replay()
            self.replays += 1
            return held[1], held[2]
        logits, tokens = self._forward(ctx, sample)
        if held is not None:
            del self.captured[key]        # recorded for another device buffer (the stager grew)
        if uses >= self.after:
            if len(self.captured) >= self.limit:
                least = min(self.captured, key=lambda k: self.seen.get(k, 0))
                if uses < 2 * max(1, self.seen.get(least, 0)):
                    return logits, tokens
                del self.captured[least]
            # the step has run; record the same launches for the next time these sizes come
            graph = torch.cuda.CUDAGraph()
            with guarded_capture(graph):
                recorded = self._forward(ctx, sample)
            self.captured[key] = (graph, recorded[0], recorded[1], buffer)
        return logits, tokens

    def _forward(self, ctx, sample: bool):
        runner = self.runner
        logits = runner.forward(ctx)
        tokens = None
        if sample and logits is not None:
            tokens = sampling.sample(logits, runner.runtime.status, ctx.floats["temperature"], ctx.floats["uniform"])
        return logits, tokens


class DecodeLoop:
    """``steps`` decode steps on the device without the host in between: after each step a
    kernel makes the sampled tokens the next inputs.  Pages for all the steps must have been
    reserved.  The scheduler does not use it (it looks at every token for end-of-sequence); the
    benchmark times the device's share of a decode step with it, and the tests hold its tokens
    against the scheduler's.

    A captured step is laid out for contexts up to a bound (the attention's launches follow the
    contexts' length); the loop holds one capture per stretch of ``SEGMENT`` tokens of context that
    its steps will cross, all recorded before the first replay, and replays the one whose stretch
    the next step's longest context lies in."""

    SEGMENT = 256

    def __init__(self, runner, entries, temperatures, uniforms, max_steps: int):
        self.runner = runner
        self.requests = len(entries)
        pages = max(max((len(t) for t in e.seq.tables), default=1) for e in entries)
        # at least as wide as the engine's captured steps have their tables (the attention's plan follows the
        # width: eight splits of a short context merge faster than five), beyond that in steps of 8 pages
        width = max(runner.graphs.page_multiple, _round_up(pages, 8))
        self.longest = 1 + max(e.seq.length for e in entries)          # the longest context of the next step
        self.limit = width * runner.page_tokens
        self.max_steps = max_steps
        self.inner = DecodeGraph(runner, self.requests, width, self._bound(self.longest))
        self.entries = entries
        device = runner.runtime.device
        self.history = torch.zeros((max_steps, self.requests), dtype=torch.int32, device=device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.ctx = self.inner.stage(entries, temperatures, uniforms)
        self.graphs: dict = {}            # bound -> captured step
        self.graph = None
        self.launches_per_step = 0
        self.steps_done = 0

    def _bound(self, longest: int) -> int:
        return min(self.limit, _round_up(longest, self.SEGMENT))

    def _one_step(self):
        logits, tokens = self.inner._forward(self.ctx)
        kernels.advance_decode(self.ctx.token_ids, self.ctx.positions, self.ctx.context_lens, tokens,
                               self.history, self.counter)

    def capture(self):
        self.ctx.planned_context = self._bound(self.longest)
        self._one_step()                       # warm-up: also a real step
        self.steps_done += 1
        self.longest += 1
        torch.cuda.synchronize()
        last = self.longest + self.max_steps
        bound = self._bound(self.longest)
        while True:
            self.ctx.planned_context = bound
            before = kernels.LAUNCHES
            graph = torch.cuda.CUDAGraph()
            with guarded_capture(graph):
                self._one_step()               # capturing does not execute: nothing advances
            self.launches_per_step = self.launches_per_step or kernels.LAUNCHES - before
            self.graphs[bound] = graph
            if bound >= min(last, self.limit):
                break
            bound = self._bound(bound + 1)
        self.graph = self.graphs[self._bound(self.longest)]

    def run(self, steps: int) -> None:
        if self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graphs[self._bound(self.longest)].replay()
            self.longest += 1
        self.steps_done += steps

    def finish(self) -> torch.Tensor:
        """Synchronise, advance the requests' lengths by the steps done; tokens [steps, requests]."""
        torch.cuda.synchronize()
        for e in self.entries:
            e.seq.length += self.steps_done
        return self.history[:self.steps_done].cpu()
