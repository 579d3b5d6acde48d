"""The Python entry point: prompts (token ids) in, generated token ids out.

``generate`` builds a runner and a scheduler sized for the prompts, adds every prompt as a
request and steps the scheduler until all have finished: continuous batching, chunked
prefill, prefix reuse, greedy or seeded temperature sampling.
"""
from __future__ import annotations

from .scheduler import Engine, EngineOptions
from .step import ModelRunner


def make_engine(model, options: EngineOptions | None = None) -> Engine:
    options = options or EngineOptions()
    runner = ModelRunner(model, num_pages=options.num_blocks, page_tokens=options.block_size,
                         max_requests=options.max_sequences, prefix_caching=options.prefix_caching)
    return Engine(runner, options)


def default_options(prompts, max_new_tokens: int, block_size: int = 16, max_sequences: int = 64) -> EngineOptions:
    """A pool that holds ``max_sequences`` of the longest request at once."""
    longest = max(len(p) for p in prompts) + max_new_tokens
    pages_each = -(-longest // block_size)
    live = min(len(prompts), max_sequences)
    return EngineOptions(block_size=block_size, num_blocks=max(1, pages_each * live), max_sequences=max_sequences)


def generate(model, prompts, max_new_tokens: int = 16, temperature: float = 0.0, seed: int = 0,
             ignore_eos: bool = False, options: EngineOptions | None = None, engine: Engine | None = None):
    """Generate for every prompt (a list of token ids).  Returns one dict per prompt:
    ``output`` (token ids), ``finish_reason`` (``eos`` or ``length``), ``prefix_hits``."""
    prompts = [list(p) for p in prompts]
    if not prompts:
        return []
    if engine is None:
        engine = make_engine(model, options or default_options(prompts, max_new_tokens))
    ids = [f"request-{i}" for i in range(len(prompts))]
    for ident, prompt in zip(ids, prompts):
        engine.add(ident, prompt, max_new_tokens, temperature=temperature, seed=seed, ignore_eos=ignore_eos)
    guard = 0
    while engine.pending:
        engine.step()
        guard += 1
        if guard > 1_000_000:
            raise RuntimeError("the scheduler made no progress")
    engine.runner.check_status()
    results = []
    for ident in ids:
        r = engine.result(ident)
        results.append({"output": r["output"], "finish_reason": r["finishReason"], "prefix_hits": r["prefixHits"]})
        engine.forget(ident)
    return results
