"""The scheduler's decisions, on the host with a stand-in model: admission, budget, portions,
decode-first order, prefix reuse, what happens when pages run out, cancel, validation, EOS,
sampling that no batching can change.  After the reference's scenarios
(test/engine.test.ts:45-155, test/qwen.test.ts:48-92)."""
import pytest

from sprout_lm_b200.engine import Engine, EngineOptions, uniform_for
from stub_runner import StubRunner, reference_output


def make(options=None, **runner_args):
    options = options or EngineOptions(block_size=4, num_blocks=64, max_sequences=4, max_batch_tokens=8,
                                       prefill_chunk_size=4)
    options.validate()
    runner = StubRunner(options.num_blocks, options.block_size, prefix_caching=options.prefix_caching, **runner_args)
    return Engine(runner, options)


def drain(engine, limit=2000):
    reports = []
    while engine.pending:
        assert len(reports) < limit, "scheduler must make progress"
        report = engine.step()
        assert sum(w["tokens"] for w in report["work"]) <= engine.options.max_batch_tokens
        assert all(p["refs"] >= 0 and p["activeRefs"] >= 0 for p in report["memory"]["pages"])
        engine.cache.check_invariants()
        reports.append(report)
    return reports


def test_continuous_batching_admits_a_late_request_and_mixes_phases():
    engine = make(EngineOptions(block_size=4, num_blocks=64, max_sequences=3, max_batch_tokens=6, prefill_chunk_size=3))
    prompts = [[1], list(range(2, 15)), [7, 8, 9, 10]]
    engine.add("A", prompts[0], 6)
    engine.add("B", prompts[1], 3)
    engine.step()
    engine.add("C", prompts[2], 2)
    reports = drain(engine)
    assert any(any(w["phase"] == "decode" for w in r["work"]) and any(w["phase"] == "prefill" for w in r["work"])
               for r in reports)
    for name, prompt, count in zip("ABC", prompts, (6, 3, 2)):
        assert engine.result(name)["status"] == "finished"
        assert engine.result(name)["output"] == reference_output(prompt, count, 50)
    kinds = [(e["id"], e["type"]) for e in engine.trace]
    assert kinds.index(("C", "admitted")) < kinds.index(("B", "finished"))
    # one batch a step: the stand-in saw every step's work as one call
    assert len(engine.runner.steps) == 1 + len([r for r in reports if r["work"]])


def test_decode_goes_first_and_portions_respect_chunk_and_budget():
    engine = make(EngineOptions(block_size=4, num_blocks=64, max_sequences=4, max_batch_tokens=6, prefill_chunk_size=4))
    engine.add("A", [1, 2], 5)
    engine.step()                                       # A prefilled, first token out
    engine.add("B", list(range(1, 12)), 2)
    report = engine.step()
    assert [(w["id"], w["phase"], w["tokens"]) for w in report["work"]] == [("A", "decode", 1), ("B", "prefill", 4)]
    report = engine.step()
    assert [(w["id"], w["from"], w["tokens"]) for w in report["work"]] == [("A", 3, 1), ("B", 4, 4)]
    engine.add("C", list(range(20, 30)), 1)
    report = engine.step()                              # budget 6: A 1, B 3 (its rest), C 2
    assert [(w["id"], w["tokens"]) for w in report["work"]] == [("A", 1), ("B", 3), ("C", 2)]
    drain(engine)


def test_prefix_sharing_reuses_pages_and_recomputes_the_last_prompt_token():
    engine = make(EngineOptions(block_size=2, num_blocks=64, max_sequences=4, max_batch_tokens=8, prefill_chunk_size=8))
    prompt = [3, 4, 5, 6]                               # exactly two pages
    engine.add("A", prompt, 4)
    engine.step()
    a_pages = engine.result("A")["blockTable"]
    engine.add("B", prompt, 4)
    report = engine.step()
    assert engine.result("B")["prefixHits"] == 2
    assert engine.result("B")["blockTable"][0] == a_pages[0]
    assert report["memory"]["pages"][a_pages[0]]["activeRefs"] == 2
    drain(engine)
    assert engine.result("A")["output"] == engine.result("B")["output"] == reference_output(prompt, 4, 50)
    assert all(p["activeRefs"] == 0 for p in engine.cache.snapshot()["pages"])
    engine.cache.clear_prefixes()
    assert engine.cache.snapshot()["freePages"] == 64


def test_same_suffix_after_other_context_does_not_hit():
    engine = make(EngineOptions(block_size=2, num_blocks=64, max_sequences=4, max_batch_tokens=8, prefill_chunk_size=8))
    engine.add("A", [1, 2, 3, 4, 5], 1)
    drain(engine)
    engine.add("B", [9, 8, 3, 4, 5], 1)
    drain(engine)
    assert engine.result("B")["prefixHits"] == 0
    assert engine.result("B")["output"] == reference_output([9, 8, 3, 4, 5], 1, 50)


@pytest.mark.parametrize("prefix_caching", [False, True])
def test_pages_run_out_preempt_and_recompute_without_changing_outputs(prefix_caching):
    options = EngineOptions(block_size=2, num_blocks=5, max_sequences=4, max_batch_tokens=6, prefill_chunk_size=2,
                            prefix_caching=prefix_caching)
    engine = make(options)
    prompts = [[1, 1], [2, 2], [3, 3]]
    for i, prompt in enumerate(prompts):
        engine.add(str(i), prompt, 7)
    reports = drain(engine)
    assert any(e["type"] == "preempted" for e in engine.trace)
    assert any(w["phase"] == "recompute" for r in reports for w in r["work"])
    for i, prompt in enumerate(prompts):
        assert engine.result(str(i))["output"] == reference_output(prompt, 7, 50)
    # the oldest request is never preempted
    assert not any(e["type"] == "preempted" and e["id"] == "0" for e in engine.trace)
    engine.cache.clear_prefixes()
    assert engine.cache.snapshot()["freePages"] == 5


def test_a_preempted_request_goes_to_the_back_and_keeps_its_output():
    options = EngineOptions(block_size=2, num_blocks=4, max_sequences=2, max_batch_tokens=4, prefill_chunk_size=2,
                            prefix_caching=False)
    engine = make(options)
    engine.add("old", [1, 2, 3], 5)
    engine.add("young", [4, 5, 6], 5)
    engine.add("later", [7], 1)
    seen = []
    while engine.pending:
        report = engine.step()
        for e in report["events"]:
            if e["type"] == "preempted":
                seen.append((e["id"], list(engine.result(e["id"])["output"]), list(engine._waiting)))
    assert seen and all(name != "old" for name, _, _ in seen)
    name, kept, queue = seen[0]
    assert queue[-1] == name                            # behind "later"
    for ident, prompt, count in (("old", [1, 2, 3], 5), ("young", [4, 5, 6], 5), ("later", [7], 1)):
        assert engine.result(ident)["output"] == reference_output(prompt, count, 50)
    assert engine.result(name)["output"][:len(kept)] == kept


def test_a_request_alone_that_cannot_continue_preempts_itself_only_when_others_hold_pages():
    # two requests, pool of 3 pages of 2: the younger is preempted, the older always finishes
    options = EngineOptions(block_size=2, num_blocks=3, max_sequences=2, max_batch_tokens=4, prefill_chunk_size=4,
                            prefix_caching=False)
    engine = make(options)
    engine.add("a", [1, 2, 3], 4)                       # needs 6 slots = 3 pages: fits alone
    engine.add("b", [4, 5, 6], 4)
    drain(engine)
    assert engine.result("a")["output"] == reference_output([1, 2, 3], 4, 50)
    assert engine.result("b")["output"] == reference_output([4, 5, 6], 4, 50)


def test_cancel_running_and_queued_without_harming_a_sibling():
    engine = make(EngineOptions(block_size=2, num_blocks=16, max_sequences=2, max_batch_tokens=8, prefill_chunk_size=8))
    prompt = [1, 2, 3, 4, 5]
    engine.add("A", prompt, 6)
    engine.add("B", prompt, 6)
    engine.add("Q", [9], 3)
    engine.step()
    engine.step()
    assert engine.cancel("B") and engine.cancel("Q")
    assert not engine.cancel("B") and not engine.cancel("nope")
    assert engine.result("B")["status"] == "cancelled" and engine.result("Q")["status"] == "cancelled"
    drain(engine)
    assert engine.result("A")["output"] == reference_output(prompt, 6, 50)
    assert all(p["activeRefs"] == 0 for p in engine.cache.snapshot()["pages"])
    assert engine.forget("B") and not engine.forget("B")
    with pytest.raises(KeyError):
        engine.result("B")


def test_input_validation():
    with pytest.raises(ValueError):
        make(EngineOptions(block_size=0))
    with pytest.raises(ValueError):
        make(EngineOptions(prefix_caching=1))
    engine = make(EngineOptions(block_size=2, num_blocks=4, max_sequences=2, max_batch_tokens=8, prefill_chunk_size=8),
                  max_positions=64)
    for bad in ([], [-1], [50], [1.5]):
        with pytest.raises(ValueError, match="valid token IDs"):
            engine.add("x", bad, 1)
    with pytest.raises(ValueError, match="positive integer"):
        engine.add("x", [1], 0)
    with pytest.raises(ValueError, match="cannot fit alone"):
        engine.add("x", [1] * 8, 2)                     # 9 slots > 8
    with pytest.raises(ValueError, match="context limit"):
        make(EngineOptions(block_size=16, num_blocks=64), max_positions=8).add("x", [1] * 8, 2)
    engine.add("x", [1] * 8, 1)                         # 8 slots fit exactly
    with pytest.raises(ValueError, match="unique"):
        engine.add("x", [1], 1)
    with pytest.raises(ValueError, match="unique"):
        engine.add("", [1], 1)


def test_eos_is_sampled_once_counted_and_frees_pages_early():
    first = reference_output([5, 6], 3, 50)
    engine = make(EngineOptions(block_size=2, num_blocks=8, max_sequences=2, max_batch_tokens=8, prefill_chunk_size=8),
                  eos_token_ids=(first[1],))
    engine.add("A", [5, 6], 10)
    engine.add("B", [5, 6], 10, ignore_eos=True)
    drain(engine)
    a, b = engine.result("A"), engine.result("B")
    assert a["output"] == first[:2] and a["finishReason"] == "eos"
    assert b["output"][:3] == first and len(b["output"]) == 10 and b["finishReason"] == "length"
    finished = [e for e in engine.trace if e["type"] == "finished" and e["id"] == "A"]
    assert finished[0]["finishReason"] == "eos"


def test_temperature_sampling_depends_on_seed_request_and_index_only():
    assert uniform_for(1, "a", 0) == uniform_for(1, "a", 0)
    assert len({uniform_for(1, "a", 0), uniform_for(2, "a", 0), uniform_for(1, "b", 0), uniform_for(1, "a", 1)}) == 4
    assert all(0.0 <= uniform_for(s, "r", i) < 1.0 for s in range(20) for i in range(20))
    outputs = []
    for options in (EngineOptions(block_size=8, num_blocks=64, max_sequences=4, max_batch_tokens=64, prefill_chunk_size=64),
                    EngineOptions(block_size=8, num_blocks=6, max_sequences=4, max_batch_tokens=5, prefill_chunk_size=3),
                    EngineOptions(block_size=2, num_blocks=18, max_sequences=2, max_batch_tokens=3, prefill_chunk_size=7,
                                  prefix_caching=False)):
        engine = make(options)
        prompts = {"p": [1, 2, 3], "q": list(range(1, 25)), "r": list(range(1, 17)) + [40]}
        for name, prompt in prompts.items():
            engine.add(name, prompt, 12, temperature=0.8, seed=5)
        drain(engine)
        outputs.append({name: engine.result(name)["output"] for name in prompts})
    assert outputs[0] == outputs[1] == outputs[2]
    greedy = make()
    greedy.add("p", [1, 2, 3], 12)
    drain(greedy)
    assert greedy.result("p")["output"] != outputs[0]["p"]       # temperature does draw other tokens


def test_a_model_failure_leaves_the_error_with_the_caller():
    engine = make()
    engine.runner.fail_after = 1
    engine.add("A", [1, 2, 3], 4)
    engine.step()
    with pytest.raises(RuntimeError, match="model failure"):
        engine.step()


def test_step_report_has_the_reference_fields():
    engine = make(EngineOptions(block_size=4, num_blocks=8, max_sequences=2, max_batch_tokens=8, prefill_chunk_size=4))
    engine.add("A", [1, 2, 3, 4, 5], 2)
    report = engine.step()
    assert set(report) == {"tick", "work", "events", "memory"} and report["tick"] == 1
    assert report["work"] == [{"id": "A", "phase": "prefill", "from": 0, "tokens": 4, "blockTable": [0]}]
    assert [e["type"] for e in report["events"]] == ["admitted"]
    assert set(report["memory"]) >= {"totalPages", "freePages", "cachedPages", "evictions", "pages"}
    report = engine.step()
    assert report["work"][0]["from"] == 4 and [e["type"] for e in report["events"]] == ["token"]
    assert report["events"][0]["index"] == 0 and report["events"][0]["token"] == engine.result("A")["output"][0]


@pytest.mark.parametrize("prefix_caching", [False, True])
def test_admission_within_the_pool_stops_the_preemption_loop(prefix_caching):
    """A pool that holds about half of what eight long requests need.  With the reference's
    admission a preempted request comes straight back and is preempted again; held back until the
    pool can take it, requests wait instead.  The outputs are the same either way."""
    prompts = [[(7 * i + j) % 40 + 1 for j in range(30)] for i in range(8)]

    def run(admit_within_pool):
        options = EngineOptions(block_size=4, num_blocks=40, max_sequences=8, max_batch_tokens=64, prefill_chunk_size=16,
                                prefix_caching=prefix_caching, admit_within_pool=admit_within_pool)
        engine = make(options)
        for i, prompt in enumerate(prompts):
            engine.add(f"r{i}", prompt, 20)
        reports = drain(engine, limit=5000)
        preempted = sum(1 for r in reports for e in r["events"] if e["type"] == "preempted")
        assert engine.cache.snapshot()["freePages"] + engine.cache.snapshot()["cachedPages"] == 40
        return [engine.result(f"r{i}")["output"] for i in range(8)], preempted, len(reports)

    plain, plain_preempted, plain_ticks = run(False)
    held, held_preempted, held_ticks = run(True)
    assert held == plain == [reference_output(p, 20, 50) for p in prompts]
    assert plain_preempted > 3 * max(held_preempted, 1)          # the loop is gone
    assert held_ticks <= plain_ticks


class AheadRunner:
    """A stub runner that takes the decode step after the one it is asked for (``then``), as the
    device-side runner does with a graph launched behind the step in flight: it notes which batch
    that step is (the requests one token longer, each fed the token its row of this step sampled)
    and counts whether the next call asks for just that batch."""

    takes_next_step = True

    def __init__(self, inner):
        self.inner = inner
        self.pending = None
        self.launched, self.used, self.dropped = 0, 0, 0

    def __getattr__(self, name):
        return getattr(self.inner, name)

    @staticmethod
    def signature(entries, tokens, temperatures, uniforms):
        return (tuple((id(e.seq), e.seq.length, t) for e, t in zip(entries, tokens)), tuple(temperatures), tuple(uniforms))

    def step_and_sample(self, entries, temperatures, uniforms, then=None):
        pending, self.pending = self.pending, None
        if pending is not None:
            if all(len(e.tokens) == 1 for e in entries) and \
                    pending == self.signature(entries, [e.tokens[0] for e in entries], temperatures, uniforms):
                self.used += 1
            else:
                self.dropped += 1
        sampled = self.inner.step_and_sample(entries, temperatures, uniforms)
        if then is not None:
            assert all(len(e.tokens) == 1 and e.want == [0] for e in entries), "only a decode step has a known successor"
            next_entries, next_temperatures, next_uniforms, rows = then
            assert all(len(e.tokens) == 1 and e.want == [0] for e in next_entries)
            assert [e.seq for e in next_entries] == [entries[row].seq for row in rows], "a request is fed its own row"
            if all(self.inner.reserve(e.seq, e.seq.length + 1) for e in next_entries):
                self.pending = self.signature(next_entries, [sampled[row] for row in rows], next_temperatures, next_uniforms)
                self.launched += 1
        return sampled


def test_a_token_that_ends_a_request_lets_the_step_launched_behind_it_go():
    """The step after is handed over before this step's tokens are known; when one of them is an
    end-of-sequence token the request is gone from the next plan and the launched step is not
    the step asked for.  The survivors' tokens are what they would have been."""
    prompts = [[3, 9, 27], [4, 16, 2, 8], [5, 25]]
    free = [reference_output(p, 14, 50) for p in prompts]
    # an end-of-sequence token that the second request produces in the middle and the others never do
    others = set(free[0]) | set(free[2])
    at = next((i for i in range(3, 12) if free[1][i] not in others and free[1][i] not in free[1][:i]), None)
    assert at is not None, "the stub's token rule changed: pick other prompts"
    stub = StubRunner(40, 4)
    stub.eos_token_ids = (free[1][at],)
    runner = AheadRunner(stub)
    engine = Engine(runner, EngineOptions(block_size=4, num_blocks=40, max_sequences=4, max_batch_tokens=16, prefill_chunk_size=8))
    for i, prompt in enumerate(prompts):
        engine.add(f"r{i}", prompt, 14)
    while engine.pending:
        engine.step()
    assert engine.result("r1")["output"] == free[1][:at + 1] and engine.result("r1")["finishReason"] == "eos"
    assert engine.result("r0")["output"] == free[0] and engine.result("r2")["output"] == free[2]
    assert runner.dropped >= 1 and runner.used >= 8
    engine.cache.check_invariants()


def test_the_next_decode_step_is_launched_ahead_only_when_it_is_known():
    """With every running request decoding on and nobody waiting, the scheduler hands the step
    after to the runner together with the step; a late arrival, a cancellation or a request that
    ends makes the next plan differ and the launch is dropped.  Tokens are the same either way."""
    import numpy as np
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, 50, n)] for n in (5, 11, 7)]

    def run(launch_ahead):
        options = EngineOptions(block_size=4, num_blocks=40, max_sequences=4, max_batch_tokens=8, prefill_chunk_size=4,
                                launch_ahead=launch_ahead)
        runner = AheadRunner(StubRunner(40, 4))
        engine = Engine(runner, options)
        engine.add("a", prompts[0], 12)
        engine.add("b", prompts[1], 9)
        steps = 0
        while engine.pending:
            engine.step()
            steps += 1
            if steps == 8:
                engine.add("c", prompts[2], 6)            # a late arrival: the step launched ahead is not the next step
            if steps == 14:
                engine.cancel("c")
        return engine, runner

    plain_engine, plain_runner = run(False)
    engine, runner = run(True)
    assert plain_runner.launched == 0
    assert runner.launched > 5 and runner.used >= runner.launched - 3 and runner.dropped >= 1
    # a launch that nothing asked for any more (its requests were cancelled) stays with the runner, which lets it go
    assert runner.launched - 1 <= runner.used + runner.dropped <= runner.launched
    for rid, prompt, count in (("a", prompts[0], 12), ("b", prompts[1], 9)):
        assert engine.result(rid)["output"] == plain_engine.result(rid)["output"] == reference_output(prompt, count, 50)
    engine.cache.check_invariants()
