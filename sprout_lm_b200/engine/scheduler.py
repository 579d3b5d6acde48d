"""The scheduler: continuous batching with chunked prefill, prefix reuse and preemption.

Policy and vocabulary are the reference engine's (src/engine.ts:42-241): requests are admitted
first-come first-served while fewer than ``max_sequences`` run; each step has a token budget;
decoding requests go first, then the others by arrival; a prompt advances by at most
``prefill_chunk_size`` tokens a step; a request yields at most one new token a step; when
pages run out an unused prefix page is evicted, else the youngest running request that is
younger than the one asking is preempted (its pages freed, its output kept, itself put at
the back of the queue), else the asking request preempts itself.  Older requests are never
preempted for younger ones, so a crowded pool still makes progress.  A preempted request,
once readmitted, recomputes prompt and output (phase ``recompute``) and then decodes on.

Where the reference runs token by token, this engine plans first and launches once: every
page reservation, eviction and preemption of a step is decided on the host, the requests
that remain form one batch for the step function, and one sampling launch draws all new
tokens; only token ids come back from the device.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field

import numpy as np

from ..sampling import uniform_for
from .batch import StepEntry


@dataclass
class EngineOptions:
    """Names and meanings of the reference's EngineOptions (src/engine.ts:18-26), in snake case."""
    block_size: int = 16
    num_blocks: int = 256
    max_sequences: int = 64
    max_batch_tokens: int = 2048
    prefill_chunk_size: int = 512
    prefix_caching: bool = True
    record_trace: bool = True
    # Not in the reference, which admits a waiting request whenever a sequence slot is free: with a
    # pool that cannot hold all requests a preempted request then comes straight back, takes pages
    # and is preempted again, tick after tick.  With this option a request waits in the queue
    # until the pool can hold its history beside what the running requests still have to take.
    admit_within_pool: bool = False
    # Not in the reference either: start the next decode step before this step's tokens are read,
    # when it is already known what that step will be (see Engine._next_step).
    launch_ahead: bool = True

    def validate(self):
        for name, value in asdict(self).items():
            if name in ("prefix_caching", "record_trace", "admit_within_pool", "launch_ahead"):
                if not isinstance(value, bool):
                    raise ValueError(f"{name} must be a boolean.")
            elif not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer.")


@dataclass
class Request:
    id: str
    order: int
    prompt: list
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False
    output: list = field(default_factory=list)
    status: str = "waiting"            # waiting | running | finished | cancelled
    seq: object = None
    prefix_hits: int = 0
    finish_reason: str | None = None
    prompt_array: object = None        # the prompt as an int32 numpy array


class StepReport(dict):
    """What a step did: ``tick``, ``work``, ``events`` and ``memory`` (the page accounting after
    the step, src/engine.ts:189).  ``memory`` lists every page, so it is taken when the step ends
    only if someone reads it."""

    def __init__(self, tick, work, events, cache):
        super().__init__(tick=tick, work=work, events=events)
        self._cache = cache

    def __missing__(self, key):
        if key == "memory":
            self["memory"] = self._cache.snapshot()
            return self["memory"]
        raise KeyError(key)

    def resolve(self) -> "StepReport":
        """Take the memory snapshot now (before the next step changes the pages)."""
        self["memory"]
        return self

    def keys(self):
        self.resolve()
        return super().keys()

    def __iter__(self):
        self.resolve()
        return super().__iter__()

    def items(self):
        self.resolve()
        return super().items()


class Engine:
    """``runner`` provides the model side: ``vocab_size``, ``max_positions``, ``eos_token_ids``,
    ``manager`` (the cache manager), ``new_sequence(tokens | None)``, ``reserve(seq, upto)``,
    ``release(seq)`` and ``step_and_sample(entries, temperatures, uniforms) -> token ids``: run
    the batch, sample at every wanted place (greedy where the temperature is 0, else at the
    given uniform number) and return the new tokens in the order of the entries."""

    def __init__(self, runner, options: EngineOptions | None = None):
        self.options = options or EngineOptions()
        self.options.validate()
        self.runner = runner
        self.cache = runner.manager
        self.trace: list = []
        self._requests: dict = {}
        self._active: dict = {}
        self._waiting: list = []
        self._tick = 0
        self._next_order = 0
        self._step_events = None

    # ------------------------------------------------------------------ requests
    def add(self, id: str, prompt, max_new_tokens: int, temperature: float = 0.0, seed: int = 0,
            ignore_eos: bool = False) -> None:
        if not id or not isinstance(id, str) or id in self._requests:
            raise ValueError("Request ID must be nonempty and unique.")
        prompt = list(prompt)
        if not prompt or any(not isinstance(t, int) or isinstance(t, bool) or t < 0 or t >= self.runner.vocab_size
                             for t in prompt):
            raise ValueError("Prompt must contain valid token IDs.")
        if not isinstance(max_new_tokens, int) or isinstance(max_new_tokens, bool) or max_new_tokens <= 0:
            raise ValueError("maxNewTokens must be a positive integer.")
        if not isinstance(temperature, (int, float)) or temperature < 0:
            raise ValueError("temperature must be a number >= 0.")
        # the last sampled token needs no cache slot: it is never fed back (src/engine.ts:80-81)
        slots = len(prompt) + max_new_tokens - 1
        if slots > self.runner.max_positions:
            raise ValueError("Request exceeds the model context limit.")
        if slots > self.options.num_blocks * self.options.block_size:
            raise ValueError("Request cannot fit alone in the KV pool. Increase numBlocks or shorten it.")
        request = Request(id=id, order=self._next_order, prompt=prompt, max_new_tokens=max_new_tokens,
                          temperature=float(temperature), seed=int(seed), ignore_eos=bool(ignore_eos),
                          prompt_array=np.asarray(prompt, dtype=np.int32))
        self._next_order += 1
        self._requests[id] = request
        self._waiting.append(id)
        self._emit("queued", request, f"{len(prompt)} prompt tokens")

    @property
    def pending(self) -> bool:
        return bool(self._active) or bool(self._waiting)

    def forget(self, id: str) -> bool:
        request = self._requests.get(id)
        if request is None or request.status in ("waiting", "running"):
            return False
        del self._requests[id]
        return True

    def cancel(self, id: str) -> bool:
        request = self._requests.get(id)
        if request is None or request.status in ("finished", "cancelled"):
            return False
        if request.seq is not None:
            self.runner.release(request.seq)
            request.seq = None
        request.status = "cancelled"
        self._active.pop(id, None)
        self._waiting = [other for other in self._waiting if other != id]
        self._emit("cancelled", request, "Released live KV references")
        return True

    def result(self, id: str) -> dict:
        request = self._requests.get(id)
        if request is None:
            raise KeyError(f"Unknown request: {id}")
        seq = request.seq
        return {"id": id, "status": request.status, "output": list(request.output),
                "finishReason": request.finish_reason, "computedTokens": seq.length if seq else 0,
                "blockTable": list(seq.blocks) if seq else [], "prefixHits": request.prefix_hits}

    # ------------------------------------------------------------------ one scheduling iteration
    def step(self) -> dict:
        events: list = []
        self._step_events = events
        try:
            return self._run_step(events)
        finally:
            self._step_events = None

    def _phase(self, request: Request) -> str:
        if not request.output:
            return "prefill"
        return "recompute" if request.seq.length < len(request.prompt) + len(request.output) - 1 else "decode"

    def _run_step(self, events: list) -> dict:
        self._tick += 1
        self._admit()
        budget = self.options.max_batch_tokens
        # decoding first (latency), then by arrival (src/engine.ts:143-144)
        batch = sorted(self._active.values(), key=lambda r: (self._phase(r) != "decode", r.order))
        planned: list = []                # (request, phase, start, tokens, wants_token)
        for request in batch:
            if not budget:
                break
            if request.status != "running":
                continue                   # preempted by an older request while planning
            # the request's history is prompt + output; it is sliced below without being built
            prompt, output = request.prompt, request.output
            total = len(prompt) + len(output)
            phase = self._phase(request)
            start = request.seq.length
            remaining = total - start - (1 if phase == "recompute" else 0)
            count = min(budget, 1 if phase == "decode" else self.options.prefill_chunk_size, remaining)
            computed = 0
            if count > 1 and self.runner.reserve(request.seq, start + count):
                computed = count           # the whole portion has its pages: nothing to decide
            else:
                # token by token (src/engine.ts:153-156): where the pool runs out, younger
                # requests are preempted, or this one stops at the tokens it has pages for
                for i in range(count):
                    if not self._reserve(request, start + i + 1, planned):
                        break
                    computed += 1
            budget -= computed
            if computed and request.status == "running":
                end = start + computed
                if start >= len(prompt):
                    tokens = output[start - len(prompt):end - len(prompt)]
                elif end <= len(prompt):
                    # a long portion travels as a view of the prompt's array (no per-token work on the host)
                    tokens = request.prompt_array[start:end] if computed >= 64 else prompt[start:end]
                else:
                    tokens = prompt[start:] + output[:end - len(prompt)]
                planned.append((request, phase, start, tokens, end == total))
        work = []
        if planned:
            entries = [StepEntry(r.seq, tokens, [len(tokens) - 1] if wants else [])
                       for r, _, _, tokens, wants in planned]
            rows = [(r, len(r.output)) for r, _, _, _, wants in planned if wants]
            temperatures = [r.temperature for r, _ in rows]
            uniforms = [uniform_for(r.seed, r.id, index) if r.temperature > 0 else 0.0 for r, index in rows]
            then = self._next_step(planned)
            if then is not None:
                sampled = self.runner.step_and_sample(entries, temperatures, uniforms, then=then)
            else:
                sampled = self.runner.step_and_sample(entries, temperatures, uniforms)
            sampled = [int(t) for t in sampled]
            if len(sampled) != len(rows) or any(t < 0 or t >= self.runner.vocab_size for t in sampled):
                raise RuntimeError("Runner returned invalid sampled token.")
            row = 0
            for request, phase, start, tokens, wants in planned:
                seq = request.seq
                table = list(seq.blocks)
                if self.options.prefix_caching:
                    self.cache.publish(request.prompt, seq)
                if wants:
                    self._accept(request, sampled[row])
                    row += 1
                work.append({"id": request.id, "phase": phase, "from": start, "tokens": len(tokens),
                             "blockTable": table})
        return StepReport(tick=self._tick, work=work, events=events, cache=self.cache)

    def _next_step(self, planned: list):
        """The decode step after the planned one, when it is known already: every running request
        decodes one token in this step, nobody waits to be admitted, and the requests that do not
        reach their length with this step's token go on (unless that token ends them).  A runner
        that can (``takes_next_step``) launches it behind this step, with each request's token
        taken on the device from the row of this step that samples it, so that the device does not
        wait while the host reads this step's tokens and accounts for them.  The next call plans as
        always; if it arrives at the same batch it takes the result, if not (a request ended, was
        added or cancelled) the launch is dropped and nothing is lost but its work."""
        if not self.options.launch_ahead or not getattr(self.runner, "takes_next_step", False) or self._waiting \
                or len(planned) != len(self._active) or any(phase != "decode" or not wants for _, phase, _, _, wants in planned):
            return None
        rows = [(i, r) for i, (r, _, _, _, _) in enumerate(planned) if len(r.output) + 1 < r.max_new_tokens]
        if not rows:
            return None
        entries = [StepEntry(r.seq, [0], [0]) for _, r in rows]
        temperatures = [r.temperature for _, r in rows]
        uniforms = [uniform_for(r.seed, r.id, len(r.output) + 1) if r.temperature > 0 else 0.0 for _, r in rows]
        return entries, temperatures, uniforms, [i for i, _ in rows]

    def _accept(self, request: Request, token: int) -> None:
        request.output.append(token)
        self._emit("token", request, str(token))
        eos = (not request.ignore_eos) and token in self.runner.eos_token_ids
        if eos or len(request.output) == request.max_new_tokens:
            request.finish_reason = "eos" if eos else "length"
            request.status = "finished"
            self.runner.release(request.seq)
            request.seq = None
            del self._active[request.id]
            self._emit("finished", request, f"{len(request.output)} output tokens")

    def _admit(self) -> None:
        while len(self._active) < self.options.max_sequences and self._waiting:
            if not self.cache.can_create():
                break
            if self.options.admit_within_pool and self._active and not self._fits(self._requests[self._waiting[0]]):
                break                      # first come, first served: nobody overtakes the head of the queue
            request = self._requests[self._waiting.pop(0)]
            history = request.prompt + request.output
            request.seq = self.runner.new_sequence(history if self.options.prefix_caching else None)
            request.prefix_hits += request.seq.length
            request.status = "running"
            self._active[request.id] = request
            self._emit("admitted", request,
                       f"Reused {request.seq.length} prefix tokens; pages [{','.join(map(str, request.seq.blocks))}]")

    def _fits(self, request: Request) -> bool:
        """Whether the pool can hold the request's history (and a page to grow into) beside the
        pages that the running requests have yet to take for theirs."""
        page = self.options.block_size
        pages_for = lambda r: -(-(len(r.prompt) + len(r.output)) // page) + 1
        owed = sum(max(0, pages_for(r) - len(r.seq.blocks)) for r in self._active.values())
        return self.cache.available_pages() - owed >= pages_for(request)

    def _reserve(self, request: Request, upto: int, planned: list) -> bool:
        while not self.runner.reserve(request.seq, upto):
            younger = [other for other in self._active.values() if other.order > request.order]
            if not younger:
                self._preempt(request, planned)
                return False
            self._preempt(max(younger, key=lambda r: r.order), planned)
        return True

    def _preempt(self, request: Request, planned: list) -> None:
        self.runner.release(request.seq)
        request.seq = None
        request.status = "waiting"
        del self._active[request.id]
        self._waiting.append(request.id)
        planned[:] = [item for item in planned if item[0] is not request]
        self._emit("preempted", request, "Keep output tokens; rebuild missing KV after readmission")

    def _emit(self, kind: str, request: Request, detail: str) -> None:
        event = {"tick": self._tick, "id": request.id, "type": kind, "detail": detail}
        if kind == "token":
            event["token"] = request.output[-1]
            event["index"] = len(request.output) - 1
        elif kind == "finished":
            event["finishReason"] = request.finish_reason
        if self.options.record_trace:
            self.trace.append(event)
        if self._step_events is not None:
            self._step_events.append(event)
