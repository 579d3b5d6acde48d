"""The engine against the plain implementation under every way of cutting the work.

Each request alone and whole; most of it in one step and the last 32 tokens one by one; in
portions of changing size; mixed, up to four live requests with so few pages that they are
used again.  In true 32-bit and in bfloat16, on both tiny configurations, through the step
function in process and through bin/trace_run.
"""
import json

import numpy as np
import pytest
import torch

import helpers
from helpers import TOL

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(base, name) for name in helpers.TINY}


def make_requests(name, seed, lengths):
    vocab = helpers.TINY[name][0]["vocab_size"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": helpers.random_tokens(rng, n, vocab) for i, n in enumerate(lengths)}


def make_runner(model_dir, dtype, pages, page_tokens):
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    model = load_model(model_dir, dtype=DTYPES[dtype])
    return ModelRunner(model, num_pages=pages, page_tokens=page_tokens, max_requests=8, prefix_caching=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_all_cuttings_in_process(model_dirs, name, dtype):
    page = helpers.TINY[name][2]
    requests = make_requests(name, 11, [5, 17, 33, 70, 129])
    rng = np.random.default_rng(5)
    plans = {
        "whole": helpers.plan_whole(requests),
        "tail": helpers.plan_tail_decode(requests),
        "portions": helpers.plan_portions(requests),
        "mixed": helpers.plan_mixed(requests, rng),
    }
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(model_dirs[name], dtype, budget // page, page)
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        assert len(got) == sum(len(t) for t in requests.values())
        helpers.compare_with_plain(model_dirs[name], requests, got, TOL[dtype], f"{name}/{dtype}/{label}")
        runner.manager.check_invariants()
        assert runner.manager.free_pages() == budget // page      # every page came back
    if dtype == "float32":
        # the 32-bit path adds every sum in an order that the cutting does not touch: not one bit differs
        for label in ("tail", "portions", "mixed"):
            for place, row in results["whole"].items():
                assert np.array_equal(results[label][place], row), f"{name}/{label}: {place} differs in some bit"


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuttings_with_weights_stored_in_32_bit(tmp_path, name):
    """The same with a folder whose matrices are stored in float32 (24 bits of mantissa, where the
    random-weights mode's default stores bfloat16 values): the 32-bit path keeps them as stored and
    multiplies full mantissas."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import Checkpoint, write_random_model
    sizes, seed, page = helpers.TINY[name]
    folder = write_random_model(tmp_path / f"full_{name}", parse_config(helpers.raw_config(sizes)), seed=seed + 10,
                                dtype="float32")
    with Checkpoint(folder) as ck:
        matrix = ck.tensor("model.layers.0.mlp.down_proj.weight")
    assert matrix.dtype == torch.float32 and not torch.equal(matrix, matrix.to(torch.bfloat16).float())
    requests = make_requests(name, 13, [5, 40, 70])
    plans = {"whole": helpers.plan_whole(requests), "tail": helpers.plan_tail_decode(requests),
             "portions": helpers.plan_portions(requests), "mixed": helpers.plan_mixed(requests, np.random.default_rng(6))}
    results = {}
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(folder, "float32", budget // page, page)
        assert runner.model.blocks[0].feed_forward.down.weight.dtype == torch.float32
        got = results[label] = helpers.run_plan_in_process(runner, plan)
        helpers.compare_with_plain(folder, requests, got, TOL["float32"], f"full-mantissa/{name}/{label}")
    for label in ("tail", "portions", "mixed"):
        for place, row in results["whole"].items():
            assert np.array_equal(results[label][place], row), (label, place)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_reuses_pages(model_dirs, dtype):
    """Seven requests through four live slots in a pool that holds four: pages of finished
    requests are handed to later ones, block tables become non-contiguous."""
    name = "B"
    page = helpers.TINY[name][2]
    requests = make_requests(name, 23, [40, 61, 24, 50, 33, 64, 47])
    plan = helpers.plan_mixed(requests, np.random.default_rng(9))
    budget = helpers.live_token_budget(plan, requests)
    assert budget < sum(-(-len(t) // 64) * 64 for t in requests.values())   # the pool cannot hold all at once
    runner = make_runner(model_dirs[name], dtype, budget // page, page)
    got = helpers.run_plan_in_process(runner, plan)
    helpers.compare_with_plain(model_dirs[name], requests, got, TOL[dtype], f"mixed-reuse/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, tmp_path, dtype):
    """bin/trace_run itself: whole, then tail decoding, then mixed, compared with the plain
    implementation and with each other."""
    name = "A"
    requests = make_requests(name, 31, [9, 40, 75, 66])
    results = {}
    for label, plan in (("whole", helpers.plan_whole(requests)),
                        ("tail", helpers.plan_tail_decode(requests)),
                        ("mixed", helpers.plan_mixed(requests, np.random.default_rng(2)))):
        budget = helpers.live_token_budget(plan, requests)
        got = helpers.run_plan_with_trace_run(model_dirs[name], dtype, plan, tmp_path / f"{label}_{dtype}", budget)
        helpers.compare_with_plain(model_dirs[name], requests, got, TOL[dtype], f"trace_run/{dtype}/{label}")
        results[label] = got
    # cutting changes nothing beyond rounding, and in 32-bit not even that
    for place, row in results["whole"].items():
        for other in ("tail", "mixed"):
            if dtype == "float32":
                assert np.array_equal(results[other][place], row), (other, place)
            else:
                assert np.abs(results[other][place] - row).max() <= 2 * TOL[dtype]
    # the index names every row of every file
    index = json.loads((tmp_path / f"whole_{dtype}" / "index.json").read_text())
    assert index["vocab"] == helpers.TINY[name][0]["vocab_size"]
    rows = [tuple(place) for places in index["files"].values() for place in places]
    assert sorted(rows) == sorted(results["whole"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """A short prompt, then several hundred tokens one by one across many page edges (in
    bfloat16 through the tensor-core decode attention, its splits and their merge)."""
    name = "A"
    requests = make_requests(name, 41, [400])
    toks = requests["r0"]
    plan = [{"entries": [("r0", toks[:6], list(range(6)))], "end": []}]
    plan += [{"entries": [("r0", [t], [0])], "end": []} for t in toks[6:]]
    runner = make_runner(model_dirs[name], dtype, 448 // 16, 16)
    got = helpers.run_plan_in_process(runner, plan)
    helpers.compare_with_plain(model_dirs[name], requests, got, TOL[dtype], "long-decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context(tmp_path, dtype):
    """2,500 tokens of history: the prompt in portions of 512 (prefill over a long cache), then
    tokens one by one with the keys of a request split over several passes per CTA and several
    CTAs, against the plain implementation at the last 24 positions."""
    folder = helpers.make_model_dir(tmp_path, "A", max_position_embeddings=4096)
    requests = make_requests("A", 91, [2524])
    toks = requests["r0"]
    want = helpers.plain_logits(folder, toks)
    plan, at = [], 0
    while at < 2500:
        n = min(512, 2500 - at)
        plan.append({"entries": [("r0", toks[at:at + n], [n - 1])], "end": []})
        at += n
    plan += [{"entries": [("r0", [t], [0])], "end": []} for t in toks[2500:]]
    runner = make_runner(folder, dtype, 2560 // 16, 16)
    got = helpers.run_plan_in_process(runner, plan)
    assert len(got) == 5 + 24
    for (rid, pos), row in got.items():
        err = float(np.abs(row - want[pos]).max())
        assert err <= TOL[dtype], (pos, err)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_shows_every_key(model_dirs, tmp_path, dtype, name):
    """Random weights make attention nearly uniform, which hides a lost or misplaced key under
    bfloat16 rounding.  Here the query and key projections are scaled up so that the softmax is
    peaked: each position leans on a few particular keys, near and far, and an engine that
    misses one of them (a page's edge, a reused page, the start of a portion) moves the logits
    far beyond the tolerance."""
    import plain_qwen2 as plain
    from sprout_lm_b200.weights import Checkpoint, write_safetensors
    import shutil
    page = helpers.TINY[name][2]
    folder = tmp_path / "sharp"
    shutil.copytree(model_dirs[name], folder)
    with Checkpoint(model_dirs[name]) as ck:
        tensors = {n: ck.tensor(n) for n in ck.inventory()}
    for n in tensors:
        if n.endswith("q_proj.weight") or n.endswith("k_proj.weight"):
            tensors[n] = (tensors[n].float() * 7.0).to(tensors[n].dtype)
    write_safetensors(folder / "model.safetensors", tensors)
    requests = make_requests(name, 77, [150, 97, 64, 120])
    cfg, w = plain.read_model_folder(folder)
    # the attention really is peaked: in the last layer's input the largest probability is far from uniform
    logits_ref = {rid: plain.logits(cfg, w, toks) for rid, toks in requests.items()}
    plans = {"whole": helpers.plan_whole(requests), "portions": helpers.plan_portions(requests),
             "mixed": helpers.plan_mixed(requests, np.random.default_rng(4)), "tail": helpers.plan_tail_decode(requests)}
    scale = max(float(np.abs(v).max()) for v in logits_ref.values())
    tol = 1e-4 if dtype == "float32" else 0.03 * scale
    for label, plan in plans.items():
        budget = helpers.live_token_budget(plan, requests)
        runner = make_runner(folder, dtype, budget // page, page)
        got = helpers.run_plan_in_process(runner, plan)
        for rid, toks in requests.items():
            for pos in range(len(toks)):
                err = float(np.abs(got[(rid, pos)] - logits_ref[rid][pos]).max())
                assert err <= tol, f"{label}/{dtype}: request {rid} position {pos} (% {page} = {pos % page}) differs by {err:.3e}"
    # and the test can fail: dropping one far key of one head changes the plain logits by more than the tolerance
    toks = requests["r0"]
    x = plain.hidden_states(cfg, w, toks, layers=0)
    heads, kv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["hidden_size"] // cfg["num_attention_heads"]
    h = plain.rms_norm(x, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    q = plain.rope_half_split(plain.linear(h, w["model.layers.0.self_attn.q_proj.weight"], w["model.layers.0.self_attn.q_proj.bias"]), range(len(toks)), hd, cfg["rope_theta"])
    k = plain.rope_half_split(plain.linear(h, w["model.layers.0.self_attn.k_proj.weight"], w["model.layers.0.self_attn.k_proj.bias"]), range(len(toks)), hd, cfg["rope_theta"])
    scores = (q[-1, :hd].astype(np.float64) @ k[:, :hd].astype(np.float64).T) / np.sqrt(hd)
    p = np.exp(scores - scores.max())
    p /= p.sum()
    assert p.max() > 10.0 / len(toks), "the attention of the sharpened model is not peaked"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(model_dirs, dtype):
    """Positions 0, 1, 2: a sequence of one token, and the first tokens one by one."""
    name = "B"
    requests = make_requests(name, 51, [1, 3])
    plan = [{"entries": [("r0", requests["r0"], [0])], "end": ["r0"]}]
    plan += [{"entries": [("r1", [t], [0])], "end": []} for t in requests["r1"]]
    runner = make_runner(model_dirs[name], dtype, 16, 8)
    got = helpers.run_plan_in_process(runner, plan)
    helpers.compare_with_plain(model_dirs[name], requests, got, TOL[dtype], "first-tokens")
