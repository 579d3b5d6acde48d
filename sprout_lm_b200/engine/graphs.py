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

import torch

from .. import kernels
from .batch import BatchStager


@contextlib.contextmanager
def guarded_capture(graph: "torch.cuda.CUDAGraph"):
    """Stream capture that the garbage collector cannot disturb: freeing an older graph while a
    new one is being captured is a CUDA call that invalidates the capture, so garbage is
    collected before and the collector rests meanwhile."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, capture_error_mode="relaxed"):
            yield
    finally:
        if was_enabled:
            gc.enable()


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class DecodeGraph:
    """One captured decode step for ``requests`` requests and block tables ``table_pages`` wide."""

    def __init__(self, runner, requests: int, table_pages: int):
        self.runner = runner
        self.requests = requests
        self.table_pages = table_pages
        self.stager = BatchStager(runner.runtime.device, len(runner.manager.groups))
        self.graph = None
        self.tokens = None
        self.logits = None
        self.launches = 0

    def _forward(self, ctx):
        logits = self.runner.model.forward(ctx, self.runner.storage)
        tokens = torch.empty(self.requests, dtype=torch.int32, device=logits.device)
        kernels.sample(logits, tokens, self.runner.runtime.status, ctx.floats["temperature"], ctx.floats["uniform"])
        return logits, tokens

    def stage(self, entries, temperatures, uniforms):
        return self.stager.stage(entries, self.runner.page_tokens, fixed_pages=self.table_pages,
                                 floats={"temperature": temperatures, "uniform": uniforms})

    def run(self, entries, temperatures, uniforms) -> torch.Tensor:
        """Stage the batch and run the step; the sampled tokens (int32, device)."""
        ctx = self.stage(entries, temperatures, uniforms)
        if self.graph is None:
            # First use: this call's step runs eagerly (that also does the kernels' first-use
            # set-up), then the same launches are captured for later calls.  Capturing records
            # without running, so the step has run exactly once: a mixer that updates
            # per-request state must not see a step twice.
            _, tokens = self._forward(ctx)
            before = kernels.LAUNCHES
            graph = torch.cuda.CUDAGraph()
            with guarded_capture(graph):
                self.logits, self.tokens = self._forward(ctx)
            self.launches = kernels.LAUNCHES - before
            self.graph = graph
            return tokens
        self.graph.replay()
        return self.tokens


class GraphCache:
    def __init__(self, runner, page_multiple: int = 8):
        self.runner = runner
        self.page_multiple = page_multiple
        self.graphs: dict = {}
        self.enabled = True

    def get(self, entries) -> DecodeGraph:
        pages = max(max((len(t) for t in e.seq.tables), default=1) for e in entries)
        key = (len(entries), _round_up(max(pages, 1), self.page_multiple))
        graph = self.graphs.get(key)
        if graph is None:
            graph = self.graphs[key] = DecodeGraph(self.runner, *key)
        return graph


class DecodeLoop:
    """``steps`` decode steps on the device without the host in between: after each step a
    kernel makes the sampled tokens the next inputs.  Pages for all the steps must have been
    reserved.  Used when no request can finish or arrive in between, and by the benchmark to
    time the device's share of a decode step."""

    def __init__(self, runner, entries, temperatures, uniforms, max_steps: int):
        self.runner = runner
        self.requests = len(entries)
        pages = max(max((len(t) for t in e.seq.tables), default=1) for e in entries)
        self.inner = DecodeGraph(runner, self.requests, _round_up(pages, 8))
        self.entries = entries
        device = runner.runtime.device
        self.history = torch.zeros((max_steps, self.requests), dtype=torch.int32, device=device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.ctx = self.inner.stage(entries, temperatures, uniforms)
        self.graph = None
        self.launches_per_step = 0
        self.steps_done = 0

    def _one_step(self):
        logits, tokens = self.inner._forward(self.ctx)
        kernels.advance_decode(self.ctx.token_ids, self.ctx.positions, self.ctx.context_lens, tokens,
                               self.history, self.counter)

    def capture(self):
        self._one_step()                       # warm-up: also a real step
        self.steps_done += 1
        torch.cuda.synchronize()
        before = kernels.LAUNCHES
        graph = torch.cuda.CUDAGraph()
        with guarded_capture(graph):
            self._one_step()
        self.launches_per_step = kernels.LAUNCHES - before
        self.graph = graph
        # capturing does not execute: nothing advanced

    def run(self, steps: int) -> None:
        if self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graph.replay()
        self.steps_done += steps

    def finish(self) -> torch.Tensor:
        """Synchronise, advance the requests' lengths by the steps done; tokens [steps, requests]."""
        torch.cuda.synchronize()
        for e in self.entries:
            e.seq.length += self.steps_done
        return self.history[:self.steps_done].cpu()
