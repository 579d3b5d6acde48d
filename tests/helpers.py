"""Shared pieces of the tests: the two tiny configurations, model folders, replay plans.

The two configurations differ in every size and option: layers, width, heads and groups
(grouped-query 4/2 against multi-query 3/1), head size, feed-forward width, vocabulary (one
is odd), rotary base, norm eps, tied against untied head, page size.
"""
from __future__ import annotations

import functools
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

import plain_qwen2 as plain

ROOT = Path(__file__).resolve().parents[1]

TINY_A = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=256, max_position_embeddings=1024, rms_norm_eps=1e-6,
              rope_theta=10000.0, tie_word_embeddings=True, eos_token_id=255)
TINY_B = dict(hidden_size=96, intermediate_size=320, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, vocab_size=509, max_position_embeddings=768, rms_norm_eps=1e-5,
              rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=[507, 508])
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8)}          # name -> (config, seed, page size)

# Absolute tolerances on logits against the plain implementation.  The tiny models' logits are
# of order 0.1 (weights are N(0, 0.02)).  float32: the reference project's bar for its GPU path on
# its tiny fixture (test/cuda-device.integration.ts:38).  bfloat16: activations, keys and values
# are rounded to 8 bits of mantissa at every layer; a wrong key, page or position moves logits
# by far more than this.
TOL = {"float32": 1e-5, "bfloat16": 6e-3}


def raw_config(sizes: dict) -> dict:
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", **sizes}


def make_model_dir(tmp_path, name: str, **overrides) -> Path:
    """Write a random-weights model folder for tiny configuration ``name`` with the package's
    random-weights mode."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.weights import write_random_model
    sizes, seed, _ = TINY[name]
    config = parse_config(raw_config({**sizes, **overrides}))
    return write_random_model(Path(tmp_path) / f"tiny_{name}", config, seed=seed)


@functools.lru_cache(maxsize=None)
def _plain_model(directory: str):
    return plain.read_model_folder(directory)


_logit_cache: dict = {}


def plain_logits(directory, tokens) -> np.ndarray:
    """Logits of the plain implementation at every position of ``tokens``."""
    key = (str(directory), tuple(tokens))
    if key not in _logit_cache:
        cfg, w = _plain_model(str(directory))
        _logit_cache[key] = plain.logits(cfg, w, list(tokens))
    return _logit_cache[key]


def random_tokens(rng, count, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=count)]


# ----------------------------------------------------------------------------- replay plans
# A plan is a list of steps; a step is {"entries": [(id, tokens, want)], "end": [ids]}.

def plan_whole(requests: dict) -> list:
    """Each request alone and whole: one step holds its entire sequence, logits everywhere."""
    return [{"entries": [(rid, toks, list(range(len(toks))))], "end": [rid]} for rid, toks in requests.items()]


def plan_tail_decode(requests: dict, tail: int = 32) -> list:
    """Most of the sequence in one step, then the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [(rid, toks[:head], list(range(head)))], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [(rid, [toks[i]], [0])], "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def plan_portions(requests: dict, sizes=(7, 2, 5, 3, 2, 11, 4, 2, 16, 1, 9)) -> list:
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    for rid, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append({"entries": [(rid, toks[at:at + n], list(range(n)))],
                          "end": [rid] if at + n == len(toks) else []})
            at += n
            k += 1
    return steps


def plan_mixed(requests: dict, rng, max_live: int = 4, portion=(2, 9), prefill_fraction: float = 0.6) -> list:
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others;
    a request sometimes sits a step out; finished requests give their pages back and later
    requests use them again."""
    waiting = list(requests.items())
    live: dict = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended = [], []
        for rid, state in list(live.items()):
            toks, at = state
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            boundary = int(len(toks) * prefill_fraction)
            n = int(rng.integers(portion[0], portion[1] + 1)) if at < boundary else 1
            n = min(n, len(toks) - at)
            entries.append((rid, toks[at:at + n], list(range(n))))
            state[1] = at + n
            if state[1] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": ended})
    return steps


def live_token_budget(plan, requests: dict) -> int:
    """The most tokens that live requests hold at any time, each rounded up to a multiple of 64."""
    held: dict = {}
    worst = 0
    for step in plan:
        for rid, toks, _ in step["entries"]:
            held[rid] = held.get(rid, 0) + len(toks)
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return worst


def run_plan_in_process(runner, plan) -> dict:
    """Drive a ModelRunner through a plan; {(request id, position): logits row}."""
    from sprout_lm_b200.engine.batch import StepEntry
    live, position, out = {}, {}, {}
    for step in plan:
        entries, places = [], []
        for rid, toks, want in step["entries"]:
            seq = live.get(rid)
            if seq is None:
                seq = live[rid] = runner.new_sequence()
                position[rid] = 0
            assert runner.reserve(seq, seq.length + len(toks)), "page pool too small for the plan"
            entries.append(StepEntry(seq, list(toks), list(want)))
            places += [(rid, position[rid] + w) for w in want]
            position[rid] += len(toks)
        logits = runner.step(entries)
        if logits is not None:
            rows = logits.float().cpu().numpy()
            for place, row in zip(places, rows):
                out[place] = row
        runner.check_status()
        for rid in step["end"]:
            runner.release(live.pop(rid))
    return out


def run_plan_with_trace_run(model_dir, dtype: str, plan, out_dir, max_tokens: int, page_tokens: int = 16,
                            extra_env=None) -> dict:
    """Drive bin/trace_run through a plan over its standard input; same result form."""
    import os
    lines, places_by_step, position = [], {}, {}
    for index, step in enumerate(plan):
        places = []
        for rid, toks, want in step["entries"]:
            position.setdefault(rid, 0)
            places += [(rid, position[rid] + w) for w in want]
            position[rid] += len(toks)
        places_by_step[index] = places
        lines.append(json.dumps({"step": index, "end": step["end"], "entries": [
            {"id": rid, "tokens": list(toks), "want": list(want)} for rid, toks, want in step["entries"]]}))
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), "--page-tokens", str(page_tokens)]
    done = subprocess.run(cmd, input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, timeout=900)
    assert done.returncode == 0, done.stderr[-4000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(plan))]
    _, w = _plain_model(str(model_dir))
    vocab = w["model.embed_tokens.weight"].shape[0]
    out = {}
    for index, places in places_by_step.items():
        if not places:
            continue
        rows = np.fromfile(Path(out_dir) / f"{index}.f32", dtype="<f4").reshape(len(places), vocab)
        for place, row in zip(places, rows):
            out[place] = row
    return out


def compare_with_plain(model_dir, requests: dict, got: dict, tol: float, label: str = ""):
    """Every wanted place against the plain implementation; on failure name the first wrong
    token and what is special about its place."""
    assert got, "no logits came back"
    worst = (0.0, None)
    for rid, toks in requests.items():
        want = plain_logits(model_dir, toks)
        for pos in range(len(toks)):
            if (rid, pos) not in got:
                continue
            err = float(np.abs(got[(rid, pos)] - want[pos]).max())
            if not np.isfinite(err) or err > tol:
                raise AssertionError(f"{label}: request {rid} position {pos} (of {len(toks)}; "
                                     f"position % 16 = {pos % 16}, % 8 = {pos % 8}) differs by {err:.3e} > {tol}")
            if err > worst[0]:
                worst = (err, (rid, pos))
    return worst
