"""Generation through the Python entry point and the scheduler on the GPU, against the plain
implementation: greedy tokens, a pool so small that requests are preempted and recomputed,
prefix reuse, seeded temperature sampling that no batching changes, the command line."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_dir(base, name) for name in helpers.TINY}


def plain_greedy_with_margin(model_dir, prompt, count):
    """Greedy continuation of the plain implementation and the smallest gap between the best and
    the second-best logit on the way (a near-tie may legitimately fall the other way in
    bfloat16)."""
    cfg, w = plain.read_model_folder(model_dir)
    history, out, margin = list(prompt), [], np.inf
    for _ in range(count):
        row = plain.logits(cfg, w, history)[-1]
        top2 = np.sort(row)[-2:]
        margin = min(margin, float(top2[1] - top2[0]))
        out.append(int(np.argmax(row)))
        history.append(out[-1])
    return out, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(model_dirs, name, dtype):
    from sprout_lm_b200 import generate, load_model
    model = load_model(model_dirs[name], dtype=dtype)
    vocab = helpers.TINY[name][0]["vocab_size"]
    rng = np.random.default_rng(3)
    prompts = [helpers.random_tokens(rng, n, vocab) for n in (5, 17, 33)]
    results = generate(model, prompts, max_new_tokens=8, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        want, margin = plain_greedy_with_margin(model_dirs[name], prompt, 8)
        if dtype == "float32" or margin > 4 * helpers.TOL[dtype]:
            assert result["output"] == want
        assert result["finish_reason"] == "length" and len(result["output"]) == 8


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pressure_prefix_reuse_and_chunks_keep_the_tokens(model_dirs, dtype):
    """Tiny B's workload: prompts 3/24/40/61 sharing a 16-token prefix, portions of 7, page size 8,
    a pool that forces preemption and recomputation: same tokens as an unconstrained run."""
    from sprout_lm_b200 import EngineOptions, generate, load_model, make_engine
    model = load_model(model_dirs["B"], dtype=dtype)
    rng = np.random.default_rng(8)
    shared = helpers.random_tokens(rng, 16, 509)
    prompts = [shared[:3]] + [shared + helpers.random_tokens(rng, n - 16, 509) for n in (24, 40, 61)]
    roomy = generate(model, prompts, max_new_tokens=12, ignore_eos=True)
    tight = EngineOptions(block_size=8, num_blocks=14, max_sequences=4, max_batch_tokens=16, prefill_chunk_size=7)
    engine = make_engine(model, tight)
    squeezed = generate(model, prompts, max_new_tokens=12, ignore_eos=True, engine=engine)
    assert any(e["type"] == "preempted" for e in engine.trace)
    assert sum(r["prefix_hits"] for r in squeezed) > 0
    if dtype == "float32":
        assert [r["output"] for r in squeezed] == [r["output"] for r in roomy]
        for prompt, result in zip(prompts, squeezed):
            assert result["output"] == plain.greedy(*plain.read_model_folder(model_dirs["B"]), prompt, 12)
    engine.cache.clear_prefixes()
    assert engine.cache.snapshot()["freePages"] == 14
    engine.cache.check_invariants()


def test_temperature_sampling_is_seeded_and_independent_of_batching(model_dirs):
    from sprout_lm_b200 import EngineOptions, generate, load_model, make_engine
    model = load_model(model_dirs["B"], dtype="float32")
    rng = np.random.default_rng(12)
    prompts = [helpers.random_tokens(rng, n, 509) for n in (3, 24, 40)]
    runs = []
    for options in (None, EngineOptions(block_size=8, num_blocks=12, max_sequences=2, max_batch_tokens=9,
                                        prefill_chunk_size=7)):
        engine = make_engine(model, options) if options else None
        runs.append([r["output"] for r in generate(model, prompts, max_new_tokens=12, temperature=0.8, seed=4,
                                                   ignore_eos=True, engine=engine)])
    assert runs[0] == runs[1]
    other = [r["output"] for r in generate(model, prompts, max_new_tokens=12, temperature=0.8, seed=5, ignore_eos=True)]
    greedy = [r["output"] for r in generate(model, prompts, max_new_tokens=12, ignore_eos=True)]
    assert other != runs[0] and greedy != runs[0]


def test_eos_stops_generation(model_dirs):
    from sprout_lm_b200 import generate, load_model
    import shutil
    rng = np.random.default_rng(1)
    prompt = helpers.random_tokens(rng, 9, 256)
    want = plain.greedy(*plain.read_model_folder(model_dirs["A"]), prompt, 5)
    folder = model_dirs["A"].parent / "tiny_A_eos"
    shutil.copytree(model_dirs["A"], folder)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": want[2]}))
    model = load_model(folder, dtype="float32")
    result = generate(model, [prompt], max_new_tokens=5)[0]
    stop = want.index(want[2]) + 1
    assert result["output"] == want[:stop] and result["finish_reason"] == "eos"


def test_sharded_folder_generates_like_the_single_file(model_dirs, tmp_path):
    """A folder with an index of two shards against the single file it was split from
    (after the reference's test/weight-files.test.ts:12-29)."""
    from sprout_lm_b200 import generate, load_model
    from sprout_lm_b200.weights import Checkpoint, write_safetensors
    import shutil
    single = model_dirs["B"]
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    shutil.copy(single / "config.json", sharded / "config.json")
    with Checkpoint(single) as ck:
        tensors = {n: ck.tensor(n) for n in ck.inventory()}
    names = sorted(tensors)
    weight_map = {}
    for shard, members in (("model-00001-of-00002.safetensors", names[::2]), ("model-00002-of-00002.safetensors", names[1::2])):
        write_safetensors(sharded / shard, {n: tensors[n] for n in members})
        weight_map.update({n: shard for n in members})
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    rng = np.random.default_rng(6)
    prompts = [helpers.random_tokens(rng, n, 509) for n in (7, 30)]
    outs = [[r["output"] for r in generate(load_model(folder, dtype="float32"), prompts, max_new_tokens=6, ignore_eos=True)]
            for folder in (single, sharded)]
    assert outs[0] == outs[1]


def test_a_pool_larger_than_the_device_is_refused(model_dirs):
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    from sprout_lm_b200.cache.storage import CapacityError
    model = load_model(model_dirs["A"], dtype="float32")
    with pytest.raises(CapacityError, match="device memory"):
        make_engine(model, EngineOptions(block_size=16, num_blocks=2_000_000_000, max_sequences=2))


def test_command_line_demo_and_generate(model_dirs):
    root = helpers.ROOT
    done = subprocess.run([sys.executable, "-m", "sprout_lm_b200", "demo", "--json", "--pressure", "--dtype", "float32",
                           "--model", str(model_dirs["A"])], capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    report = json.loads(done.stdout)
    assert report["mode"] == "pressure" and [r["status"] for r in report["results"]] == ["finished"] * 3
    assert any(e["type"] == "preempted" for r in report["reports"] for e in r["events"])
    assert all(sum(w["tokens"] for w in r["work"]) <= 6 for r in report["reports"])
    done = subprocess.run([sys.executable, str(root / "bin" / "sprout-b200"), "demo", "--model", str(model_dirs["A"])],
                          capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    assert "logical → physical pages" in done.stdout and "Tick 1 | free pages" in done.stdout and "0→" in done.stdout
    assert "prefix tokens reused" in done.stdout
    done = subprocess.run([sys.executable, "-m", "sprout_lm_b200", "generate", "--model", str(model_dirs["A"]),
                           "--dtype", "float32", "--prompt", "1,2,3,4,5", "--max-new-tokens", "4", "--ignore-eos", "--json"],
                          capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    final = json.loads(done.stdout.strip().splitlines()[-1])
    want = plain.greedy(*plain.read_model_folder(model_dirs["A"]), [1, 2, 3, 4, 5], 4)
    assert final["report"]["results"][0]["output"] == want
    # a tiny random model written on the spot: the other configuration, and the refusal of both sources at once
    done = subprocess.run([sys.executable, "-m", "sprout_lm_b200", "demo", "--tiny", "B", "--seed", "3", "--json", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    report = json.loads(done.stdout)
    assert [r["status"] for r in report["results"]] == ["finished"] * 3
    assert all(0 <= t < 509 for r in report["results"] for t in r["output"])
    done = subprocess.run([sys.executable, "-m", "sprout_lm_b200", "demo", "--tiny", "B", "--model", str(model_dirs["A"])],
                          capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode != 0 and "not both" in done.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_step_shapes_replay(tmp_path, dtype):
    """Steps with prompt portions whose sizes come again (tokens, requests, wanted rows) are
    replayed from a capture.  Only the sizes are fixed in it: other requests, other splits of the
    tokens between the requests and other pages give the logits of a runner that never captures."""
    import numpy as np
    import helpers
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    folder = helpers.make_model_dir(tmp_path, "A", max_position_embeddings=1024)
    model = load_model(folder, dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
    vocab = helpers.TINY["A"][0]["vocab_size"]
    rng = np.random.default_rng(12)
    rounds = [(200, 56), (100, 156), (31, 225), (128, 128), (255, 1), (7, 249)]   # 256 tokens of two requests each time

    def run(capturing: bool):
        runner = ModelRunner(model, num_pages=200, page_tokens=16, max_requests=8, prefix_caching=False)
        runner.step_graphs.enabled = capturing
        out = []
        local = np.random.default_rng(5)
        for a, b in rounds:
            seqs = [runner.new_sequence(), runner.new_sequence()]
            history = [helpers.random_tokens(local, 40, vocab), helpers.random_tokens(local, 7, vocab)]
            for seq, tokens in zip(seqs, history):                          # some cache before the step of interest
                assert runner.reserve(seq, len(tokens))
                runner.step([StepEntry(seq, tokens, [])])
            entries = []
            for seq, n in zip(seqs, (a, b)):
                assert runner.reserve(seq, seq.length + n)
                entries.append(StepEntry(seq, helpers.random_tokens(local, n, vocab), [0, n - 1]))
            out.append(runner.step(entries).cpu().numpy())
            if len(out) == 4:
                runner.release(seqs[0])                                     # later rounds get other pages
            else:
                for seq in seqs:
                    runner.release(seq)
        runner.check_status()
        return out, runner.step_graphs.replays

    plain, none = run(False)
    replayed, count = run(True)
    assert none == 0 and count == len(rounds) - 3            # the fourth round and later replay the third's capture
    for want, got in zip(plain, replayed):
        assert np.abs(want - got).max() <= (1e-5 if dtype == "float32" else 2 * helpers.TOL["bfloat16"])
