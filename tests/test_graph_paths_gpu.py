"""The paths that generation and the benchmark really take, against the plain implementation.

Decoding through the scheduler replays captured CUDA graphs (``DecodeGraph``), keyed by the number
of requests, the block tables' width and the attention's split plan, with a host mirror that is
updated in place; the benchmark's device-side loop (``DecodeLoop``) feeds tokens back without the
host; mixed steps whose sizes repeat are captured too (``StepGraphs``), with sampling inside.
Here each of them runs for hundreds of tokens, across changes of plan and of table width, on both
sides of the small-batch kernels' token tiles (8 and 16 tokens), and what it computes is compared with the
plain implementation: logits where they can be read, tokens otherwise.
"""
import numpy as np
import pytest
import torch

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(base, name) for name in helpers.TINY}


def check_tokens(model_dir, prompt, output, dtype, label, tol=None):
    """Every generated token against the plain implementation's logits for the same history (the
    engine's own earlier tokens): in 32-bit the plain argmax unless the two best logits are a
    rounding apart, in bfloat16 a token within bfloat16's reach of the best."""
    rows = helpers.plain_logits(model_dir, list(prompt) + list(output))
    tol = tol if tol is not None else TOL[dtype]
    for i, token in enumerate(output):
        row = rows[len(prompt) - 1 + i]
        best = float(row.max())
        if dtype == "float32":
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 4 * tol:
                assert token == int(np.argmax(row)), f"{label}: output {i} is {token}, plain says {int(np.argmax(row))}"
        assert row[token] >= best - 4 * tol, f"{label}: output {i} ({token}) lies {best - row[token]:.3e} below the best logit"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,batch", [("A", 3), ("A", 9), ("B", 3), ("B", 9), ("A", 18)])
def test_long_generation_through_the_scheduler(model_dirs, name, batch, dtype):
    """300 and more decoded tokens per request through the scheduler: the captured decode steps
    are re-keyed on the way (requests finish one after the other, so the batch shrinks; B's block
    tables widen past 64 pages; the attention's plan may follow the context) and every token stays
    the plain implementation's."""
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    sizes, _, page = helpers.TINY[name]
    model = load_model(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(17 + batch)
    new_tokens = 310
    longest = sizes["max_position_embeddings"] - new_tokens - 3 * batch
    # B: the longest request grows past 64 pages of 8 tokens
    lengths = [int(n) for n in np.linspace(6, 200 if name == "A" else min(longest, 64 * page - 60), batch)]
    prompts = [helpers.random_tokens(rng, n, sizes["vocab_size"]) for n in lengths]
    # the requests generate 310, 313, 316, ... tokens: the batch shrinks one by one at the end, each
    # size a captured step of its own
    counts = [new_tokens + 3 * i for i in range(batch)]
    pages = sum(-(-(n + c) // page) for n, c in zip(lengths, counts)) + 2
    engine = make_engine(model, EngineOptions(block_size=page, num_blocks=pages, max_sequences=batch, max_batch_tokens=2048,
                                              prefill_chunk_size=512, prefix_caching=False))
    for i, (prompt, count) in enumerate(zip(prompts, counts)):
        engine.add(f"r{i}", prompt, count, ignore_eos=True)
    while engine.pending:
        engine.step()
    results = [engine.result(f"r{i}") for i in range(batch)]
    graphs = engine.runner.graphs
    widths = {key[1] for key in graphs.graphs}
    assert graphs.keys_used >= 3, "the decode steps were never re-keyed"
    if name == "B":              # 64 pages of 8 tokens end at 512 tokens; A's 1,024 positions fit 64 pages of 16
        assert len(widths) >= 2 or graphs.evictions, f"the block tables never grew past one width ({widths})"
    assert all(g.graph is not None for g in graphs.graphs.values() if g.launches)
    for i, (prompt, result) in enumerate(zip(prompts, results)):
        assert len(result["output"]) == counts[i] and result["finishReason"] == "length"
        check_tokens(model_dirs[name], prompt, result["output"], dtype, f"{name}/{dtype}/batch {batch}/request {i}")
    engine.runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,batch", [("B", 3), ("A", 9), ("B", 18)])
def test_replayed_decode_steps_give_the_plain_logits(model_dirs, name, batch, dtype):
    """The logits inside the captured decode step, read after every replay, with the requests'
    tokens forced: at the tolerance of the step function's own tests, across plan and width
    changes."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    sizes, _, page = helpers.TINY[name]
    model = load_model(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(29)
    decode = 200 if batch > 3 else 330
    heads = [int(n) for n in np.linspace(5, min(64 * page - 150, sizes["max_position_embeddings"] - decode - 1), batch)]
    requests = {f"g{i}": helpers.random_tokens(rng, n + decode, sizes["vocab_size"]) for i, n in enumerate(heads)}
    want = {rid: helpers.plain_logits(model_dirs[name], toks) for rid, toks in requests.items()}
    pages = sum(-(-len(t) // page) for t in requests.values())
    runner = ModelRunner(model, num_pages=pages, page_tokens=page, max_requests=batch, prefix_caching=False)
    seqs = {}
    for (rid, toks), head in zip(requests.items(), heads):
        seqs[rid] = runner.new_sequence()
        assert runner.reserve(seqs[rid], head)
        runner.step([StepEntry(seqs[rid], toks[:head], [])])
    # the first request leaves after a third of the steps, the second after two thirds: three batch
    # sizes, each a captured step of its own; pages are taken as the requests grow, so B's tables
    # widen past 64 pages on the way
    leaves = {"g0": decode // 3, "g1": 2 * decode // 3}
    graphs_seen, widths, worst = set(), set(), 0.0
    for step in range(decode):
        live = [(rid, head) for rid, head in zip(requests, heads) if step < leaves.get(rid, decode)]
        for rid, _ in live:
            assert runner.reserve(seqs[rid], seqs[rid].length + 1)
        entries = [StepEntry(seqs[rid], [requests[rid][head + step]], [0]) for rid, head in live]
        sampled = runner.step_and_sample(entries, [0.0] * len(live), [0.0] * len(live))
        graph = runner.last_decode_graph
        graphs_seen.add(id(graph))
        widths.add(graph.table_pages)
        assert graph.requests == len(live)
        logits = graph.last_logits.float().cpu().numpy()
        for row, token, (rid, head) in zip(logits, sampled, live):
            ref = want[rid][head + step]
            err = float(np.abs(row - ref).max())
            worst = max(worst, err)
            assert err <= TOL[dtype], f"{name}/{dtype}: request {rid} position {head + step} differs by {err:.3e} in a replayed step"
            assert row[token] == row.max()
    assert len(graphs_seen) >= 3
    if name == "B":
        assert len(widths) >= 2      # the longest request crossed 64 pages
    runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,batch", [("A", 1), ("B", 8), ("A", 9), ("B", 16), ("A", 17), ("B", 64)])
def test_device_side_decode_loop_gives_the_schedulers_tokens(model_dirs, name, batch, dtype):
    """``DecodeLoop`` (the benchmark's device-side run of decode steps) against ``generate``: the
    same tokens in 32-bit, and in bfloat16 tokens that the plain implementation backs."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.generate import generate
    from sprout_lm_b200.engine.step import ModelRunner
    sizes, _, page = helpers.TINY[name]
    model = load_model(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(31 + batch)
    steps = 140 if batch <= 9 else 40 if batch > 17 else 80
    prompts = [helpers.random_tokens(rng, int(n), sizes["vocab_size"]) for n in rng.integers(3, 60, batch)]
    pages = sum(-(-(len(p) + steps + 2) // page) for p in prompts) + 1
    runner = ModelRunner(model, num_pages=pages, page_tokens=page, max_requests=batch, prefix_caching=False)
    seqs, first = [], []
    for prompt in prompts:
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(prompt))
        first += runner.step_and_sample([StepEntry(seq, prompt, [len(prompt) - 1])], [0.0], [0.0])
        seqs.append(seq)
    loop = runner.decode_loop([StepEntry(s, [t], [0]) for s, t in zip(seqs, first)], [0.0] * batch, [0.0] * batch,
                              max_steps=steps + 1)
    loop.run(steps - 1)                                    # the capture's own step comes on top
    history = loop.finish().numpy()
    runner.check_status()
    assert history.shape == (steps, batch) and loop.graph is not None
    outputs = [[first[i]] + [int(t) for t in history[:, i]] for i in range(batch)]
    for seq, prompt in zip(seqs, prompts):
        assert seq.length == len(prompt) + steps
    if dtype == "float32":
        results = generate(model, prompts, max_new_tokens=steps + 1, ignore_eos=True)
        assert [r["output"] for r in results] == outputs
    for i in range(0, batch, max(1, batch // 6)):
        check_tokens(model_dirs[name], prompts[i], outputs[i], dtype, f"loop/{name}/{dtype}/request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_mixed_step_with_sampling(model_dirs, dtype):
    """A step with prompt portions that also samples, replayed from its capture (``StepGraphs`` with
    sampling inside): the same tokens as the uncaptured step, greedy rows backed by the plain
    implementation, drawn rows equal for equal uniform numbers."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    name = "A"
    sizes, _, page = helpers.TINY[name]
    model = load_model(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(41)
    rounds = [[helpers.random_tokens(rng, 70, sizes["vocab_size"]), helpers.random_tokens(rng, 64, sizes["vocab_size"])]
              for _ in range(6)]
    temperatures, uniforms = [0.0, 0.8], [0.0, 0.37]

    def run(capture: bool):
        runner = ModelRunner(model, num_pages=16, page_tokens=page, max_requests=4, prefix_caching=False)
        runner.step_graphs.enabled = capture
        out = []
        for prompts in rounds:
            seqs = [runner.new_sequence() for _ in prompts]
            for seq, prompt in zip(seqs, prompts):
                assert runner.reserve(seq, len(prompt))
            out.append(runner.step_and_sample([StepEntry(s, p, [len(p) - 1]) for s, p in zip(seqs, prompts)],
                                              temperatures, uniforms))
            for seq in seqs:
                runner.release(seq)
        runner.check_status()
        return out, runner
    eager, _ = run(False)
    captured, runner = run(True)
    assert runner.step_graphs.replays >= 2 and any(key[4] for key in runner.step_graphs.captured)
    assert captured == eager
    for prompts, tokens in zip(rounds, captured):
        check_tokens(model_dirs[name], prompts[0], [tokens[0]], dtype, "captured mixed step")
        assert 0 <= tokens[1] < sizes["vocab_size"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_launched_ahead_give_the_same_tokens(model_dirs, dtype):
    """The scheduler has the next decode step launched behind the one in flight, its tokens fed on
    the device (``EngineOptions.launch_ahead``).  Same tokens as without, most steps taken from the
    launch, and a request added in the middle (which makes the launched step the wrong one) still
    gets, and leaves to the others, the plain implementation's tokens."""
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    name = "B"
    sizes, _, page = helpers.TINY[name]
    model = load_model(model_dirs[name], dtype=dtype)
    rng = np.random.default_rng(61)
    prompts = [helpers.random_tokens(rng, n, sizes["vocab_size"]) for n in (9, 30, 18, 5)]
    outputs = {}
    for ahead in (False, True):
        engine = make_engine(model, EngineOptions(block_size=page, num_blocks=64, max_sequences=4, max_batch_tokens=64,
                                                  prefill_chunk_size=16, prefix_caching=False, launch_ahead=ahead))
        for i, prompt in enumerate(prompts[:3]):
            # the second request draws its tokens (the draw's number for a token is fixed by seed, request and index)
            engine.add(f"r{i}", prompt, 40, ignore_eos=True, temperature=0.9 if i == 1 else 0.0, seed=11)
        steps = 0
        while engine.pending:
            engine.step()
            steps += 1
            if steps == 20:
                engine.add("r3", prompts[3], 12, ignore_eos=True)
        engine.runner.check_status()
        outputs[ahead] = [engine.result(f"r{i}")["output"] for i in range(4)]
        runner = engine.runner
        if ahead:
            assert runner.ahead_used >= 25 and runner.ahead_dropped >= 1
        else:
            assert runner.ahead_used == 0 and runner.ahead_dropped == 0
        assert runner.manager.free_pages() == 64
    if dtype == "float32":
        assert outputs[True] == outputs[False]
    for i, (prompt, output) in enumerate(zip(prompts, outputs[True])):
        if i != 1:
            check_tokens(model_dirs[name], prompt, output, dtype, f"launch ahead/{dtype}")
    assert outputs[True][1] != outputs[True][0] and len(set(outputs[True][1])) > 5      # the drawn tokens are no argmax run


def test_a_request_that_ends_drops_the_step_launched_behind_it(model_dirs, tmp_path):
    """Three requests decode with the step after always launched behind the step in flight; one of
    them meets its end-of-sequence token in the middle, which the host learns only after the next
    step is under way with that request in it.  That step is let go and run again without the
    request; everybody's tokens are the plain implementation's, and every page comes back."""
    import json
    import shutil
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    name = "B"
    sizes, _, page = helpers.TINY[name]
    rng = np.random.default_rng(67)
    prompts = [helpers.random_tokens(rng, n, sizes["vocab_size"]) for n in (11, 7, 20)]
    import plain_qwen2 as plain
    weights = plain.read_model_folder(model_dirs[name])
    wants = [plain.greedy(*weights, prompt, 30) for prompt in prompts]
    # an end-of-sequence token that the first request produces at some step after its tenth and the others never do
    others = set(wants[1]) | set(wants[2])
    at = next((i for i in range(10, 30) if wants[0][i] not in others and wants[0][i] not in wants[0][:i]), None)
    if at is None:
        pytest.skip("no token of the first request is its own")
    folder = tmp_path / "tiny_B_eos"
    shutil.copytree(model_dirs[name], folder)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": wants[0][at]}))
    model = load_model(folder, dtype="float32")
    engine = make_engine(model, EngineOptions(block_size=page, num_blocks=64, max_sequences=4, max_batch_tokens=64,
                                              prefill_chunk_size=32, prefix_caching=False))
    for i, prompt in enumerate(prompts):
        engine.add(f"r{i}", prompt, 30)
    while engine.pending:
        engine.step()
    engine.runner.check_status()
    assert engine.result("r0")["output"] == wants[0][:at + 1] and engine.result("r0")["finishReason"] == "eos"
    assert engine.result("r1")["output"] == wants[1] and engine.result("r2")["output"] == wants[2]
    assert engine.runner.ahead_dropped >= 1 and engine.runner.ahead_used >= 15
    assert engine.runner.manager.free_pages() == 64


def test_large_batch_decodes_with_resident_contexts(tmp_path):
    """A batch large enough for the attention kernel that keeps a request's whole context in one
    CTA's shared memory (head size 64, 48 requests of 2 key/value heads): the logits inside the
    replayed decode steps against the plain implementation, with prompts of many lengths so that
    pages end everywhere, and the plan checked to be the resident one."""
    from sprout_lm_b200 import kernels, load_model
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.weights import write_random_model
    sizes = dict(hidden_size=896, intermediate_size=512, num_hidden_layers=2, num_attention_heads=14, num_key_value_heads=2,
                 vocab_size=600, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1000000.0,
                 tie_word_embeddings=False, eos_token_id=599)
    folder = write_random_model(tmp_path / "wide", parse_config(helpers.raw_config(sizes)), seed=9)
    model = load_model(folder, dtype="bfloat16")
    batch, decode, page = 48, 12, 16
    rng = np.random.default_rng(67)
    heads = [int(n) for n in rng.integers(1, 300, batch)]
    heads[0], heads[1] = 255, 256                        # a context that fills its pages exactly, and one more
    requests = {f"w{i}": helpers.random_tokens(rng, n + decode, 600) for i, n in enumerate(heads)}
    want = {rid: helpers.plain_logits(folder, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(w).max()) for w in want.values())
    runner = ModelRunner(model, num_pages=sum(-(-len(t) // page) for t in requests.values()), page_tokens=page,
                         max_requests=batch, prefix_caching=False)
    seqs = {}
    for (rid, toks), head in zip(requests.items(), heads):
        seqs[rid] = runner.new_sequence()
        assert runner.reserve(seqs[rid], head)
        runner.step([StepEntry(seqs[rid], toks[:head], [])])
    for step in range(decode):
        for rid in requests:
            assert runner.reserve(seqs[rid], seqs[rid].length + 1)
        entries = [StepEntry(seqs[rid], [requests[rid][head + step]], [0]) for rid, head in zip(requests, heads)]
        runner.step_and_sample(entries, [0.0] * batch, [0.0] * batch)
        graph = runner.last_decode_graph
        plan = model.decode_plan(batch, graph.table_pages * page, graph.ctx.planned_context, page)
        assert plan[0][0] == "resident", plan[0]
        logits = graph.last_logits.float().cpu().numpy()
        for row, (rid, head) in zip(logits, zip(requests, heads)):
            err = float(np.abs(row - want[rid][head + step]).max())
            assert err <= 0.02 * scale, f"request {rid} position {head + step} differs by {err:.3e} (scale {scale:.3f})"
    runner.check_status()
