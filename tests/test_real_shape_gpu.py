"""The layer sizes of the 0.5B configuration (hidden 896, 14 query / 2 key-value heads of 64,
feed-forward 4864, vocabulary 151936, tied head), with two layers to keep the plain
implementation affordable: whole, in portions, decoded one by one (the captured decode graph),
in true 32-bit and in bfloat16.

Tolerance in 32-bit: the reference project's own bar for the real 0.5B model against an
independent float32 implementation, 1e-3 + 1e-4 |ref| (test/model.integration.ts:69)."""
import numpy as np
import pytest

import helpers

pytestmark = pytest.mark.gpu

SIZES = dict(hidden_size=896, intermediate_size=4864, num_hidden_layers=2, num_attention_heads=14,
             num_key_value_heads=2, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
             rope_theta=1000000.0, tie_word_embeddings=True, eos_token_id=151645)


SIZES_7B_LAYER = dict(hidden_size=3584, intermediate_size=18944, num_hidden_layers=1, num_attention_heads=28,
                      num_key_value_heads=4, vocab_size=1000, max_position_embeddings=4096, rms_norm_eps=1e-6,
                      rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=999)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_7b_layer_sizes(tmp_path, dtype):
    """One layer with the 7B configuration's sizes (head size 128, 28 / 4 heads, feed-forward
    18944; a small vocabulary keeps the plain implementation affordable): a portion, then tokens
    one by one."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m7", parse_config(helpers.raw_config(SIZES_7B_LAYER)), seed=3)
    rng = np.random.default_rng(0)
    requests = {"a": helpers.random_tokens(rng, 30, 1000), "b": helpers.random_tokens(rng, 19, 1000)}
    want = {rid: helpers.plain_logits(folder, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(w).max()) for w in want.values())
    model = load_model(folder, dtype=dtype)
    runner = ModelRunner(model, num_pages=8, page_tokens=16, max_requests=4, prefix_caching=False)
    got = helpers.run_plan_in_process(runner, helpers.plan_tail_decode(requests, tail=8))
    for rid, toks in requests.items():
        for pos in range(len(toks)):
            ref = want[rid][pos]
            err = np.abs(got[(rid, pos)] - ref)
            if dtype == "float32":
                assert (err <= 1e-3 + 1e-4 * np.abs(ref)).all(), (rid, pos, float(err.max()))
            else:
                assert float(err.max()) <= 0.02 * scale, (rid, pos, float(err.max()), scale)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model
    config = parse_config(helpers.raw_config(SIZES))
    return write_random_model(tmp_path_factory.mktemp("real") / "model", config, seed=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_under_all_cuttings(folder, dtype):
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    rng = np.random.default_rng(0)
    requests = {"a": helpers.random_tokens(rng, 40, SIZES["vocab_size"]), "b": helpers.random_tokens(rng, 23, SIZES["vocab_size"])}
    want = {rid: helpers.plain_logits(folder, toks) for rid, toks in requests.items()}
    model = load_model(folder, dtype=dtype)
    scale = max(float(np.abs(w).max()) for w in want.values())

    def check(got, label):
        for rid, toks in requests.items():
            for pos in range(len(toks)):
                if (rid, pos) not in got:
                    continue
                ref = want[rid][pos]
                err = np.abs(got[(rid, pos)] - ref)
                if dtype == "float32":
                    assert (err <= 1e-3 + 1e-4 * np.abs(ref)).all(), (label, rid, pos, float(err.max()))
                else:
                    assert float(err.max()) <= 0.02 * scale, (label, rid, pos, float(err.max()), scale)

    for label, plan in (("whole", helpers.plan_whole(requests)), ("portions", helpers.plan_portions(requests)),
                        ("mixed", helpers.plan_mixed(requests, np.random.default_rng(1)))):
        runner = ModelRunner(model, num_pages=8, page_tokens=16, max_requests=4, prefix_caching=False)
        check(helpers.run_plan_in_process(runner, plan), label)

    # the captured decode graph: prompts in one step each, then both requests decoded together with
    # their own tokens forced; the sampled token of every step must be the plain argmax
    runner = ModelRunner(model, num_pages=8, page_tokens=16, max_requests=4, prefix_caching=False)
    seqs = {rid: runner.new_sequence() for rid in requests}
    head = 12
    for rid, toks in requests.items():
        assert runner.reserve(seqs[rid], len(toks))
        runner.step([StepEntry(seqs[rid], toks[:head], [])])
    for at in range(head, 23):
        entries = [StepEntry(seqs[rid], [requests[rid][at]], [0]) for rid in requests]
        tokens = runner.step_and_sample(entries, [0.0, 0.0], [0.0, 0.0])
        for rid, token in zip(requests, tokens):
            row = want[rid][at]
            top2 = np.sort(row)[-2:]
            if dtype == "float32" or top2[1] - top2[0] > 0.04 * scale:
                assert token == int(np.argmax(row)), (rid, at)
    assert len(runner.graphs.graphs) == 1 and next(iter(runner.graphs.graphs.values())).graph is not None
    runner.check_status()


@pytest.fixture(scope="module")
def full_depth_folder(tmp_path_factory):
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model
    config = parse_config(helpers.raw_config({**SIZES, "num_hidden_layers": 24}))
    return write_random_model(tmp_path_factory.mktemp("full") / "model", config, seed=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_depth_0_5b_under_all_cuttings(full_depth_folder, dtype):
    """All 24 layers of the 0.5B configuration (random weights), two short requests, whole, in
    portions, mixed, and decoded by the device-side loop: against the plain implementation at
    every position.  The reference checks its real 0.5B model the same way, 18 positions of
    151,936 logits at 1e-3 + 1e-4 |ref| (test/model.integration.ts:21-69); that is the 32-bit bar
    here.  bfloat16 rounds activations, keys and values to 8 bits of mantissa (2^-9 relative) some
    six times a layer; over 24 layers these add up like a random walk to about 0.025 of the scale,
    and the bar is twice that: 0.05 of the largest logit."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    rng = np.random.default_rng(5)
    vocab = SIZES["vocab_size"]
    requests = {"a": helpers.random_tokens(rng, 24, vocab), "b": helpers.random_tokens(rng, 13, vocab)}
    want = {rid: helpers.plain_logits(full_depth_folder, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(w).max()) for w in want.values())
    model = load_model(full_depth_folder, dtype=dtype)
    assert len(model.blocks) == 24

    def check(got, label):
        assert got
        for (rid, pos), row in got.items():
            ref = want[rid][pos]
            err = np.abs(row - ref)
            if dtype == "float32":
                assert (err <= 1e-3 + 1e-4 * np.abs(ref)).all(), (label, rid, pos, float(err.max()))
            else:
                assert float(err.max()) <= 0.05 * scale, (label, rid, pos, float(err.max()), scale)

    for label, plan in (("whole", helpers.plan_whole(requests)), ("portions", helpers.plan_portions(requests)),
                        ("mixed", helpers.plan_mixed(requests, np.random.default_rng(2), max_live=2)),
                        ("tail", helpers.plan_tail_decode(requests, tail=6))):
        runner = ModelRunner(model, num_pages=8, page_tokens=16, max_requests=4, prefix_caching=False)
        check(helpers.run_plan_in_process(runner, plan), label)
        runner.check_status()
    # the device-side decode loop at these sizes: each token must be one that the plain logits back
    runner = ModelRunner(model, num_pages=8, page_tokens=16, max_requests=4, prefix_caching=False)
    seqs, first = [], []
    heads = {"a": 18, "b": 7}
    for rid, toks in requests.items():
        seq = runner.new_sequence()
        assert runner.reserve(seq, heads[rid])
        first += runner.step_and_sample([StepEntry(seq, toks[:heads[rid]], [heads[rid] - 1])], [0.0], [0.0])
        seqs.append(seq)
    for rid, token in zip(requests, first):
        row = want[rid][heads[rid] - 1]
        assert row[token] >= row.max() - (1e-3 if dtype == "float32" else 0.05 * scale)
    loop = runner.decode_loop([StepEntry(s, [t], [0]) for s, t in zip(seqs, first)], [0.0, 0.0], [0.0, 0.0], max_steps=5)
    loop.run(3)
    history = loop.finish().numpy()
    runner.check_status()
    import plain_qwen2 as plain
    cfg, w = plain.read_model_folder(full_depth_folder)
    assert history.shape == (4, 2)
    for i, rid in enumerate(requests):
        if rid != "b":
            continue                         # the shorter request keeps the plain implementation's head product small
        generated = [first[i]] + [int(t) for t in history[:, i]]
        rows = plain.logits(cfg, w, requests[rid][:heads[rid]] + generated)
        for j, token in enumerate(generated[1:]):
            row = rows[heads[rid] + j]
            assert row[token] >= row.max() - (1e-3 if dtype == "float32" else 0.05 * scale), (rid, j)


LONG_PREFILL = {
    # head size 64 as in the 0.5B configuration, 7 query heads per key/value head
    "hd64": dict(hidden_size=896, intermediate_size=512, num_hidden_layers=1, num_attention_heads=14,
                 num_key_value_heads=2, vocab_size=600, max_position_embeddings=2048, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=599),
    # head size 128 as in the 7B configuration
    "hd128": dict(hidden_size=1024, intermediate_size=512, num_hidden_layers=1, num_attention_heads=8,
                  num_key_value_heads=2, vocab_size=600, max_position_embeddings=2048, rms_norm_eps=1e-5,
                  rope_theta=10000.0, tie_word_embeddings=False, eos_token_id=599),
}


@pytest.mark.parametrize("name", ["hd64", "hd128"])
def test_long_prefill_on_the_tcgen05_attention(tmp_path, name):
    """Prompts of several key tiles through the tcgen05 prefill attention (bfloat16): whole (the
    longest pieces get two CTAs each), in large portions over a growing cache, and two requests
    in one step, against the plain implementation at every position.  The query and key
    projections are scaled up so that the softmax leans on particular keys; the bar is the one of
    the sharpened model in test_replay_gpu.py (0.03 of the largest logit: bfloat16 rounding of
    peaked scores; the mma.sync kernel lands at the same 0.017 and 0.022 on these two models)."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.weights import Checkpoint, write_random_model, write_safetensors
    sizes = LONG_PREFILL[name]
    folder = write_random_model(tmp_path / name, parse_config(helpers.raw_config(sizes)), seed=7)
    with Checkpoint(folder) as ck:
        tensors = {n: ck.tensor(n) for n in ck.inventory()}
    for n in tensors:
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            tensors[n] = (tensors[n].float() * 4.0).to(tensors[n].dtype)
    write_safetensors(folder / "model.safetensors", tensors)
    rng = np.random.default_rng(3)
    requests = {"a": helpers.random_tokens(rng, 700, sizes["vocab_size"]), "b": helpers.random_tokens(rng, 333, sizes["vocab_size"])}
    want = {rid: helpers.plain_logits(folder, toks) for rid, toks in requests.items()}
    scale = max(float(np.abs(w).max()) for w in want.values())
    model = load_model(folder, dtype="bfloat16")

    def portions(toks, rid, sizes_):
        steps, at = [], 0
        for n in sizes_:
            n = min(n, len(toks) - at)
            if n <= 0:
                break
            steps.append({"entries": [(rid, toks[at:at + n], list(range(n)))], "end": []})
            at += n
        assert at == len(toks)
        return steps

    plans = {
        "whole": helpers.plan_whole(requests),
        "portions": portions(requests["a"], "a", (300, 256, 144)) + portions(requests["b"], "b", (129, 204)),
        "together": [{"entries": [("a", requests["a"][:400], list(range(400))), ("b", requests["b"][:200], list(range(200)))], "end": []},
                     {"entries": [("a", requests["a"][400:], list(range(300))), ("b", requests["b"][200:], list(range(133)))], "end": []}],
    }
    for label, plan in plans.items():
        runner = ModelRunner(model, num_pages=80, page_tokens=16, max_requests=4, prefix_caching=False)
        got = helpers.run_plan_in_process(runner, plan)
        runner.check_status()
        for rid, toks in requests.items():
            for pos in range(len(toks)):
                err = float(np.abs(got[(rid, pos)] - want[rid][pos]).max())
                assert err <= 0.03 * scale, (label, rid, pos, err, scale)
