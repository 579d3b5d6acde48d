"""The engine's 32-bit path on the reference project's own fixture.

The fixture is a random 2-layer Qwen2 with head size 4, intermediate size 28 and hidden size 16:
sizes that the tensor-core kernels refuse and the 32-bit kernels take.  Its eight logit vectors
were computed by the reference's authors with an independent implementation; the reference holds
its own GPU path to 1e-5 on them (test/cuda-device.integration.ts:18-49), with a cache whose
pages are made non-contiguous by a second request that takes page 0 and gives it back
(test/qwen.test.ts:20-29).  The same here, through this engine's model, cache and step function.
"""
import json

import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def load(fixture_dir):
    from sprout_lm_b200.models import load_model
    return load_model(fixture_dir, dtype=torch.float32)


def test_engine_matches_the_reference_fixture_token_by_token(fixture_dir):
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    model = load(fixture_dir)
    record = json.loads((fixture_dir / "reference.json").read_text())
    worst = 0.0
    for case in record["cases"]:
        runner = ModelRunner(model, num_pages=12, page_tokens=2, max_requests=4, prefix_caching=False)
        blocker = runner.new_sequence()
        assert runner.reserve(blocker, 1) and blocker.blocks == [0]
        seq = runner.new_sequence()
        logits = None
        for token in case["tokens"]:
            assert runner.reserve(seq, seq.length + 1)
            logits = runner.step([StepEntry(seq, [int(token)], [0])])
            if seq.length == 2:
                runner.release(blocker)
        assert list(seq.blocks[:2]) == [1, 0]              # the request's pages are not contiguous
        for step, name in enumerate(case["logits"]):
            want = np.fromfile(fixture_dir / name, dtype="<f4")
            got = logits[0].cpu().numpy()
            err = float(np.abs(got - want).max())
            worst = max(worst, err)
            assert err < 1e-5, (name, err)
            assert int(np.argmax(got)) == case["output"][step]
            if step + 1 < len(case["output"]):
                assert runner.reserve(seq, seq.length + 1)
                logits = runner.step([StepEntry(seq, [int(case["output"][step])], [0])])
        runner.check_status()
        runner.release(seq)
        assert runner.manager.free_pages() == 12
    print(f"worst error against the reference's stored logits: {worst:.3e}")


def test_fixture_generates_the_reference_outputs(fixture_dir):
    """Greedy generation through the scheduler: the reference's recorded output ids."""
    from sprout_lm_b200 import EngineOptions, generate, make_engine
    model = load(fixture_dir)
    record = json.loads((fixture_dir / "reference.json").read_text())
    prompts = [case["tokens"] for case in record["cases"]]
    engine = make_engine(model, EngineOptions(block_size=2, num_blocks=16, max_sequences=4, max_batch_tokens=3,
                                              prefill_chunk_size=2))
    results = generate(model, prompts, max_new_tokens=4, ignore_eos=True, engine=engine)
    assert [r["output"] for r in results] == [case["output"] for case in record["cases"]]


def test_fixture_under_every_cutting(fixture_dir):
    """The fixture's model under the four cuttings, against the plain implementation at the
    reference's GPU tolerance, and bitwise equal between the cuttings."""
    from sprout_lm_b200.engine.step import ModelRunner
    model = load(fixture_dir)
    rng = np.random.default_rng(3)
    requests = {f"f{i}": helpers.random_tokens(rng, n, 32) for i, n in enumerate((4, 9, 33, 50, 64))}
    plans = {"whole": helpers.plan_whole(requests), "tail": helpers.plan_tail_decode(requests),
             "portions": helpers.plan_portions(requests),
             "mixed": helpers.plan_mixed(requests, np.random.default_rng(8))}
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = ModelRunner(model, num_pages=budget // 4, page_tokens=4, max_requests=8, prefix_caching=False)
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        helpers.compare_with_plain(fixture_dir, requests, got, 1e-5, f"fixture/{label}")
        assert runner.manager.free_pages() == budget // 4
    for label in ("tail", "portions", "mixed"):
        for place, row in results["whole"].items():
            assert np.array_equal(results[label][place], row), (label, place)


def test_fixture_sizes_are_refused_in_bfloat16_with_a_clear_error(fixture_dir):
    from sprout_lm_b200.models import load_model
    with pytest.raises(ValueError, match="bfloat16 path"):
        load_model(fixture_dir, dtype=torch.bfloat16)
