"""Benchmark: decode tokens per second of the Qwen2.5-0.5B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step.  The default run has the layer sizes of the 0.5B configuration
(24 layers, hidden 896, 14/2 heads of 64, feed-forward 4864, vocabulary 151936, tied head)
with random weights in bfloat16, a batch of 8 requests with 512-token random prompts and a
4096-token context limit.  One JSON line is printed:

* ``value``: decoded tokens per second with the step running wholly on the device (sampled
  tokens fed back by a kernel, the step replayed as a CUDA graph), timed with CUDA events
  over exactly K steps after W warm-up steps;
* ``e2e``: the same through the Python entry point (``Engine.step``): every step copies the
  batch's arrays from pinned host memory to the device and reads the new token ids back;
* ``prefill``: one 2,048-token prompt in one step, tokens per second and the fraction of the
  bfloat16 tensor-core peak its floating-point work reaches;
* ``roofline``: bytes a decode step must read (every weight once, the cache of the live
  requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens per second at batch 1 and 64;
* ``clocks``: SM clock and throttle reasons sampled during the timed region.

Inputs are larger than the L2 cache (988 MB of weights are read every step), so no flush is
needed between timed iterations.  ``--gpus N`` with N > 1 is refused with exit code 2: this
engine runs on one GPU.  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIG_05B = dict(hidden_size=896, intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14,
                  num_key_value_heads=2, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, tie_word_embeddings=True, eos_token_id=151645)
# the 7B shape of the reference's second workload (continuous batching over mixed prompt lengths)
CONFIG_7B = dict(hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                 num_key_value_heads=4, vocab_size=152064, max_position_embeddings=4096, rms_norm_eps=1e-6,
                 rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=151645)
# the 14B shape of its third (a shared prefix, a pool too small for all requests)
CONFIG_14B = dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=48, num_attention_heads=40,
                  num_key_value_heads=8, vocab_size=152064, max_position_embeddings=8192, rms_norm_eps=1e-5,
                  rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=151645)
SHAPES = {"0.5b": CONFIG_05B, "7b": CONFIG_7B, "14b": CONFIG_14B}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
REFERENCE_UNAVAILABLE = ("the reference is a TypeScript program for Node >= 24 with a Node-API CUDA module; it has no "
                         "Python package to install (pip finds no setup.py or pyproject.toml) and node is not in this image")


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            found = {"source": "measured"}
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = raw.get(key)
                if isinstance(value, dict):
                    value = value.get("value")
                if isinstance(value, (int, float)):
                    found[key] = float(value)
            if "hbm_gbs" in found and "bf16_tflops" in found:
                return found
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                             "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        peak = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for s in self.samples for name, flag in zip(names, s[2:6]) if flag.lower().startswith("active")})
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(peak) if peak else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_folder(layers: int, shape: str = "0.5b", context: int = 0) -> Path:
    """The random-weights model folder of the benchmark shape (written once per temporary folder);
    ``context``: another context length than the shape's."""
    from sprout_lm_b200 import parse_config, write_random_model
    sizes = dict(SHAPES[shape], num_hidden_layers=layers)
    tag = "" if shape == "0.5b" else "_" + shape
    if context and context != sizes["max_position_embeddings"]:
        sizes["max_position_embeddings"] = context
        tag += f"_C{context}"
    folder = Path(tempfile.gettempdir()) / f"sprout_lm_b200_bench_{os.getuid()}{tag}_L{layers}"
    config = parse_config({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", **sizes})
    marker = folder / "complete"
    if not marker.exists():
        print(f"[bench] writing random weights to {folder}", file=sys.stderr, flush=True)
        write_random_model(folder, config, seed=0)
        marker.write_text("ok")
    return folder


def weight_bytes(model) -> int:
    """Bytes of every weight a decode step uses once (the tied head is the embedding matrix)."""
    seen, total = set(), 0

    def add(t):
        nonlocal total
        if t is not None and t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for block in model.blocks:
        for lin in (block.mixer.qkv, block.mixer.out, block.feed_forward.gate_up, block.feed_forward.down):
            add(lin.weight)
            add(lin.bias)
        for norm in block.norms:
            add(norm.gain)
    add(model.final_norm.gain)
    add(model.head.linear.weight)
    return total


def prefill_flops(cfg: dict, tokens: int) -> float:
    h, i, l = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    heads, kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = h // heads
    per_token = l * 2 * (h * (heads + 2 * kv) * hd + heads * hd * h + 2 * h * i + i * h)
    attention = l * 4 * heads * hd * tokens * (tokens + 1) / 2          # QK^T and PV over the causal half
    head = 2 * h * cfg["vocab_size"]                                     # logits at one place
    return per_token * tokens + attention + head


def timed_decode(runner, batch: int, prompt_len: int, steps: int, warmup: int, rng, sampler=None):
    """Prefill ``batch`` prompts, then time ``steps`` decode steps that run wholly on the device."""
    import torch
    from sprout_lm_b200.engine.batch import StepEntry
    vocab = runner.vocab_size
    seqs = []
    for _ in range(batch):
        seq = runner.new_sequence()
        assert runner.reserve(seq, prompt_len)
        seqs.append(seq)
    chunk = max(1, 4096 // prompt_len)
    first = []
    for at in range(0, batch, chunk):
        for begin in range(0, prompt_len, 4096):                 # long prompts in portions of 4,096 tokens
            n = min(4096, prompt_len - begin)
            last = begin + n == prompt_len
            entries = [StepEntry(s, [int(t) for t in rng.integers(0, vocab, n)], [n - 1] if last else [])
                       for s in seqs[at:at + chunk]]
            sampled = runner.step_and_sample(entries, [0.0] * len(entries) if last else [], [0.0] * len(entries) if last else [])
        first += sampled
    entries = [StepEntry(s, [t], [0]) for s, t in zip(seqs, first)]
    loop = runner.decode_loop(entries, [0.0] * batch, [0.0] * batch, max_steps=steps + warmup + 2)
    loop.run(max(warmup - 1, 0))                 # capture runs one more step
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    loop.run(steps)
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    ms = begin.elapsed_time(end)
    mean_context = prompt_len + warmup + steps / 2
    tokens = loop.finish()
    runner.check_status()
    assert tokens.shape[0] == steps + warmup and int(tokens.min()) >= 0
    for s in seqs:
        runner.release(s)
    return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1000), "launches_per_step": loop.launches_per_step,
            "mean_context": mean_context, "clocks": clocks}


def ablation(model, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """Marginal cost of each kind of kernel in the decode step: the step is captured and timed
    with one kind replaced by a no-op (its outputs are then garbage; only the time is used).
    Shows where the step's time goes under the real launch pipeline, warm caches included."""
    import numpy as np
    import torch
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    real = {name: getattr(kernels, name) for name in ("attention_decode", "attention_decode_fused", "attention_decode_resident",
                                                      "rmsnorm", "rope_append", "gemm_bf16", "gemm_bf16_unscaled", "sample",
                                                      "ffn_decode", "linear_decode")}
    linear = real["linear_decode"]
    gemm = real["gemm_bf16"]
    hidden, inter = model.spec.hidden_size, model.blocks[0].feed_forward.intermediate_size
    qkv_rows = model.blocks[0].mixer.qkv.out_features

    def gemm_without(skip):
        def call(a, w, out, status, **kw):
            return None if skip(w, kw) else gemm(a, w, out, status, **kw)
        return call

    variants = {
        "baseline": {},
        "attention": {"attention_decode": lambda *a, **k: None, "attention_decode_fused": lambda *a, **k: None,
                      "attention_decode_resident": lambda *a, **k: None},
        "rmsnorm": {"rmsnorm": lambda *a, **k: None},
        "rope_append": {"rope_append": lambda *a, **k: None},
        # (from 17 tokens the q/k/v product may be the one that takes the norm's input as it is)
        "gemm_qkv": {"gemm_bf16": gemm_without(lambda w, kw: w.shape[0] == qkv_rows), "gemm_bf16_unscaled": lambda *a, **k: None},
        "gemm_o": {"gemm_bf16": gemm_without(lambda w, kw: tuple(w.shape) == (hidden, hidden))},
        "gemm_gate_up": {"gemm_bf16": gemm_without(lambda w, kw: bool(kw.get("swiglu")))},
        "gemm_down": {"gemm_bf16": gemm_without(lambda w, kw: tuple(w.shape) == (hidden, inter))},
        "gemm_lm_head": {"gemm_bf16": gemm_without(lambda w, kw: w.shape[0] == model.spec.vocab_size)},
        "sample": {"sample": lambda *a, **k: None},
        # the small-batch kernels (they take the place of the norms and of every product but the head at up to 8 tokens)
        "ffn_decode": {"ffn_decode": lambda *a, **k: None},
        "linear_norm_qkv": {"linear_decode": lambda w, out, st, a=None, norm=None: None if norm is not None else linear(w, out, st, a=a)},
        "linear_o": {"linear_decode": lambda w, out, st, a=None, norm=None: None if a is not None else linear(w, out, st, norm=norm)},
        "all_gemms": {"gemm_bf16": lambda *a, **k: None, "gemm_bf16_unscaled": lambda *a, **k: None},
    }
    out = {}
    for label, patches in variants.items():
        rng = np.random.default_rng(0)
        runner = ModelRunner(model, num_pages=batch * (-(-(prompt_len + steps + warmup + 16) // 16)) + 16, page_tokens=16,
                             max_requests=max(batch, 1), prefix_caching=False)
        seqs = []
        for _ in range(batch):
            seq = runner.new_sequence()
            assert runner.reserve(seq, prompt_len)
            seqs.append(seq)
        first = []
        for at in range(0, batch, 8):
            entries = [StepEntry(s, [int(t) for t in rng.integers(0, 1000, prompt_len)], [prompt_len - 1]) for s in seqs[at:at + 8]]
            first += runner.step_and_sample(entries, [0.0] * len(entries), [0.0] * len(entries))
        for name, fn in patches.items():
            setattr(kernels, name, fn)
        try:
            loop = runner.decode_loop([StepEntry(s, [t], [0]) for s, t in zip(seqs, first)], [0.0] * batch, [0.0] * batch,
                                      max_steps=steps + warmup + 2)
            loop.run(warmup)
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            loop.run(steps)
            end.record()
            torch.cuda.synchronize()
        finally:
            for name, fn in real.items():
                setattr(kernels, name, fn)
        runner.runtime.status.zero_()
        out[label] = round(begin.elapsed_time(end) / steps * 1000, 1)
    base = out["baseline"]
    return {"us_per_step": base, "saved_us_without": {k: round(base - v, 1) for k, v in out.items() if k != "baseline"}}


def timed_e2e(model, batch: int, prompt_len: int, steps: int, warmup: int, rng):
    """The same workload through Engine.step: host token ids in, host token ids out, every step."""
    import torch
    from sprout_lm_b200 import EngineOptions, make_engine
    pages = batch * (-(-(prompt_len + steps + warmup + 8) // 16)) + 8
    engine = make_engine(model, EngineOptions(block_size=16, num_blocks=pages, max_sequences=max(batch, 1),
                                              max_batch_tokens=8192, prefill_chunk_size=2048, prefix_caching=False,
                                              record_trace=False))
    for i in range(batch):
        engine.add(f"r{i}", [int(t) for t in rng.integers(0, model.spec.vocab_size, prompt_len)],
                   steps + warmup + 4, ignore_eos=True)
    while any(w["phase"] != "decode" for w in engine.step()["work"]):
        pass
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    before = dict(engine.runner.stats)
    start = time.perf_counter()
    produced, marks = 0, [start]
    for _ in range(steps):
        report = engine.step()
        produced += sum(1 for e in report["events"] if e["type"] == "token")
        marks.append(time.perf_counter())       # the step's tokens are on the host here
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start
    per_step = sorted((b - a) * 1000 for a, b in zip(marks, marks[1:]))
    engine.runner.check_status()
    assert produced == batch * steps
    h2d = (engine.runner.stats["h2d_bytes"] - before["h2d_bytes"]) // steps
    d2h = (engine.runner.stats["d2h_bytes"] - before["d2h_bytes"]) // steps
    return {"value": produced / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": seconds * 1000 / steps, "p50_ms": per_step[len(per_step) // 2],
            "p95_ms": per_step[min(len(per_step) - 1, int(len(per_step) * 0.95))]}


def timed_prefill(runner, tokens: int, rng, repeats: int = 5):
    """A prompt of ``tokens`` tokens in one step through ``ModelRunner.step`` (what the scheduler
    calls): token ids from the host, the last position's logits on the device.  The same sizes
    come every time, so from the fourth step on the runner replays its capture of the step."""
    import numpy as np
    import torch
    from sprout_lm_b200.engine.batch import StepEntry
    times = []
    for _ in range(repeats + 4):
        seq = runner.new_sequence()
        assert runner.reserve(seq, tokens)
        entry = StepEntry(seq, rng.integers(0, runner.vocab_size, tokens).astype(np.int32), [tokens - 1])
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        logits = runner.step([entry])
        end.record()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(logits).all())
        times.append(begin.elapsed_time(end))
        runner.release(seq)
    return statistics.median(times[4:])


def timed_serving(shape: str, layers: int, requests: int, workload: str = "mixed", seed: int = 0) -> dict:
    """Continuous batching through ``Engine.step``, host tokens in and out every step.

    ``mixed``: ``requests`` requests with uniform-random prompt lengths in [128, 2048] arrive at
    once, prompts are prefilled in portions beside the decoding of the others, every request
    generates 128 tokens.  ``shared-prefix``: prompts of 4,096 tokens whose first 1,024 are the
    same, 256 generated tokens each, prefix reuse on, and a pool that holds 60 % of what all
    requests need at their longest, so that requests wait or are preempted and recomputed
    (requests are admitted when the pool can take them; SPROUT_REFERENCE_ADMISSION=1 admits
    as the reference does, whenever a sequence slot is free)."""
    import numpy as np
    import torch
    from sprout_lm_b200 import EngineOptions, load_model, make_engine
    sizes = SHAPES[shape]
    layers = layers or sizes["num_hidden_layers"]
    model = load_model(model_folder(layers, shape), dtype="bfloat16", device="cuda:0")
    rng = np.random.default_rng(seed)
    shared = workload == "shared-prefix"
    if shared:
        lengths, new_tokens = [4096] * requests, 256
        if 4096 + new_tokens - 1 > sizes["max_position_embeddings"]:
            raise SystemExit(f"bench.py: the shared-prefix workload needs a context of 4,351 positions; shape {shape} has "
                             f"{sizes['max_position_embeddings']}")
        pages = int(0.6 * requests * -(-(4096 + new_tokens) // 16))
    else:
        lengths, new_tokens = [int(n) for n in rng.integers(128, 2049, requests)], 128
        pages = sum(-(-(n + new_tokens) // 16) for n in lengths) + 64
    options = EngineOptions(block_size=16, num_blocks=pages, max_sequences=requests, max_batch_tokens=2048,
                            prefill_chunk_size=1024, prefix_caching=shared, record_trace=False,
                            admit_within_pool=shared and os.environ.get("SPROUT_REFERENCE_ADMISSION") != "1")
    engine = make_engine(model, options)                 # one engine for both rounds: the second finds the graphs captured

    def run_once(tag):
        prefix = [int(t) for t in rng.integers(0, model.spec.vocab_size, 1024)]     # a new one each round: no hits across rounds
        for i, n in enumerate(lengths):
            tokens = [int(t) for t in rng.integers(0, model.spec.vocab_size, n)]
            if shared:
                tokens[:1024] = prefix
            engine.add(f"{tag}{i}", tokens, new_tokens, ignore_eos=True)
        times, kinds, preempted = [], {"prefill": 0, "mixed": 0, "decode": 0}, 0
        # the prompts are millions of Python integers: a full collection walking them in the middle
        # of the run would cost hundreds of milliseconds; collect now and set them aside
        gc.collect()
        gc.freeze()
        torch.cuda.synchronize()
        begin = time.perf_counter()
        while engine.pending:
            t0 = time.perf_counter()
            report = engine.step()
            times.append((time.perf_counter() - t0) * 1000)
            phases = {w["phase"] for w in report["work"]}
            kinds["decode" if phases == {"decode"} else "prefill" if "decode" not in phases else "mixed"] += 1
            preempted += sum(1 for e in report["events"] if e["type"] == "preempted")
        torch.cuda.synchronize()
        seconds = time.perf_counter() - begin
        gc.unfreeze()
        engine.runner.check_status()
        results = [engine.result(f"{tag}{i}") for i in range(requests)]
        assert all(len(r["output"]) == new_tokens for r in results)
        return seconds, times, kinds, preempted, engine.runner.step_graphs.replays, sum(r["prefixHits"] for r in results)

    run_once("warm")                                     # first use: kernel set-up, graph captures
    seconds, times, kinds, preempted, replays, hits = run_once("r")
    times.sort()
    pick = lambda q: round(times[min(len(times) - 1, int(q * len(times)))], 3)
    return {"impl": "ours", "only": "serve", "workload": workload, "shape": shape, "layers": layers,
            "layers_of_model": sizes["num_hidden_layers"], "requests": requests, "pool_pages": pages, "prefix_hit_tokens": hits, "prompt_tokens": sum(lengths), "new_tokens": requests * new_tokens,
            "seconds": round(seconds, 4), "generated_tokens_per_s": round(requests * new_tokens / seconds, 1),
            "all_tokens_per_s": round((sum(lengths) + requests * new_tokens) / seconds, 1),
            "steps": len(times), "step_kinds": kinds, "step_ms": {"p50": pick(0.5), "p95": pick(0.95), "max": times[-1].__round__(3)},
            "preempted": preempted, "prefill_steps_replayed": replays,
            "decode_graphs": {"keys": engine.runner.graphs.keys_used, "held": len(engine.runner.graphs.graphs),
                              "dropped": engine.runner.graphs.evictions},
            "steps_launched_ahead": {"taken": engine.runner.ahead_used, "let_go": engine.runner.ahead_dropped}}


def timed_attention(tokens: int, shape: str = "0.5b", repeats: int = 20) -> dict:
    """The prefill attention kernels alone, at the model's head sizes, over a paged cache: one
    request of ``tokens`` tokens attending to itself (causal), both kernels."""
    import torch
    from sprout_lm_b200 import kernels
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    head_dim, page = SHAPES[shape]["hidden_size"] // heads, 16
    pages = -(-tokens // page)
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(pages + 1, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).reshape(1, pages)
    q = torch.randn(tokens, heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    q_start = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flops = 4.0 * heads * head_dim * tokens * (tokens + 1) / 2
    result = {"impl": "ours", "only": "attention", "shape": shape, "tokens": tokens, "heads": heads, "kv_heads": kv_heads,
              "head_dim": head_dim, "page_tokens": page}
    for variant in ("mma_sync", "tcgen05"):
        call = lambda: kernels.attention_prefill(q, k, v, table, q_start, positions, out, heads, kv_heads, head_dim,
                                                 status, variant=variant)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(repeats):
            call()
        end.record()
        torch.cuda.synchronize()
        us = begin.elapsed_time(end) * 1000 / repeats
        result[f"{variant}_us"] = round(us, 1)
        result[f"{variant}_tflops"] = round(flops / us / 1e6, 1)
    assert int(status.item()) == 0
    return result


def timed_decode_attention(shape: str, batch: int, context: int, repeats: int = 10) -> dict:
    """The decode attention kernel alone (one query token per request, ``context`` keys each, pages
    scattered over the pool, block tables as wide as a replayed decode graph's): with the split
    plan the engine would pick, and with other split sizes for comparison.  Bytes are the keys and
    values read."""
    import torch
    from sprout_lm_b200 import kernels
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    head_dim, page = SHAPES[shape]["hidden_size"] // heads, 16
    width = -(-(-(-context // page)) // 64) * 64
    total = batch * width
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(total, kv_heads, page, head_dim, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.randperm(total, device="cuda", generator=g).to(torch.int32).reshape(batch, width)
    lens = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    q = torch.randn(batch, heads * head_dim, device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    planned = -(-context // 128) * 128

    def replayed(split_keys):
        if split_keys == "resident":
            room = min(kernels.resident_cap(heads, kv_heads, head_dim, page), -(-context // 256) * 256)
            call = lambda: kernels.attention_decode_resident(k, v, table, lens, out, heads, kv_heads, head_dim, status, room, q=q)
        else:
            call = lambda: kernels.attention_decode(q, k, v, table, lens, out, heads, kv_heads, head_dim, status,
                                                    split_keys=split_keys, live_keys=planned)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(repeats):
                    call()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1000 / repeats)
        return statistics.median(times)

    megabytes = 2.0 * batch * context * kv_heads * head_dim * 2 / 1e6
    plan = kernels.decode_split_plan(batch, kv_heads, width * page, head_dim, planned)
    us = replayed(None)
    result = {"impl": "ours", "only": "decode-attention", "shape": shape, "batch": batch, "context": context,
              "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "table_keys": width * page,
              "plan": {"split_keys": plan[0], "splits": plan[1], "through_memory": plan[2]},
              "us": round(us, 1), "gbs": round(megabytes / us * 1e3), "mb": round(megabytes, 1), "other_splits_us": {}}
    for passes in (1, 2, 4, 8, 16, 32, width * page // 128):
        if passes * 128 <= width * page and width * page // (passes * 128) <= 256:
            result["other_splits_us"][str(passes * 128)] = round(replayed(passes * 128), 1)
    if context <= kernels.resident_cap(heads, kv_heads, head_dim, page):
        # the whole context of a (request, key/value head) in one CTA's shared memory, pages by TMA
        us = replayed("resident")
        result["resident_us"], result["resident_gbs"] = round(us, 1), round(megabytes / us * 1e3)
        result["engine_takes"] = kernels.decode_attention_plan(batch, heads, kv_heads, head_dim, page, width * page, planned)[0]
    assert int(status.item()) == 0
    return result


def timed_long_prompt(shape: str, layers: int, total: int, portion: int) -> dict:
    """One request of ``total`` tokens through ``ModelRunner.step`` in portions of ``portion``: the
    time of every step (CUDA events; the second of two runs), so that the attention over the cached
    keys shows as the increase from portion to portion (the products cost the same in each)."""
    import numpy as np
    import torch
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    base = SHAPES[shape]
    layers = layers or base["num_hidden_layers"]
    context = base["max_position_embeddings"]
    while context < total:
        context *= 2
    model = load_model(model_folder(layers, shape, context), dtype="bfloat16", device="cuda:0")
    runner = ModelRunner(model, num_pages=-(-total // 16) + 16, page_tokens=16, max_requests=2, prefix_caching=False)
    rng = np.random.default_rng(0)
    heads, head_dim = base["num_attention_heads"], base["hidden_size"] // base["num_attention_heads"]
    steps = []
    for run in range(2):
        seq = runner.new_sequence()
        assert runner.reserve(seq, total)
        steps = []
        for begin in range(0, total, portion):
            n = min(portion, total - begin)
            tokens = [int(t) for t in rng.integers(0, base["vocab_size"], n)]
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(seq, tokens, [n - 1])])
            end.record()
            torch.cuda.synchronize()
            steps.append({"context": begin, "tokens": n, "ms": round(start.elapsed_time(end), 3)})
        runner.check_status()
        runner.release(seq)
    whole = sum(s["ms"] for s in steps)
    out = {"impl": "ours", "only": "long-prompt", "shape": shape, "layers": layers, "tokens": total, "portion": portion,
           "context_limit": context, "ms": round(whole, 2), "tokens_per_s": round(total / whole * 1000, 1), "steps": steps}
    full = [s for s in steps if s["tokens"] == portion]
    if len(full) >= 3:
        # attention over one more portion's worth of cached keys: 4 * portion^2 * heads * head_dim flops a layer
        growth = (full[-1]["ms"] - full[1]["ms"]) / (len(full) - 2)
        out["ms_more_per_portion_of_context"] = round(growth, 3)
        out["attention_tflops_from_growth"] = round(4.0 * portion * portion * heads * head_dim * layers / (growth / 1000) / 1e12, 1)
    return out


def timed_gemms(tokens: int, shape: str = "0.5b", repeats: int = 20) -> dict:
    """The model's four projections at ``tokens`` tokens, each alone: 20 launches replayed from a
    CUDA graph (no host time between them), beside the library's plain bfloat16 product of the
    same shape for scale (it fuses nothing and is not on the engine's path).  Up to 256 tokens (the
    decode regime, where a product is a stream of weights) the launches cycle through copies of
    the weights that together exceed L2, as the layers of a model do, and the RMSNorm that
    precedes a product is timed the same way."""
    import torch
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.parts.linear import small_batch_split_k
    from sprout_lm_b200.parts.mlp import interleave_gate_up
    hidden, inter = SHAPES[shape]["hidden_size"], SHAPES[shape]["intermediate_size"]
    heads, kv_heads = SHAPES[shape]["num_attention_heads"], SHAPES[shape]["num_key_value_heads"]
    qkv = (heads + 2 * kv_heads) * (hidden // heads)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    rand = lambda *shape: (torch.randn(*shape, device="cuda", generator=g) * 0.05).to(torch.bfloat16)

    def replayed(call):
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for i in range(repeats):
                    call(i)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1000 / repeats

    result = {"impl": "ours", "only": "gemm", "shape": shape, "tokens": tokens}
    # up to 256 tokens the engine sums q/k/v in float32 over a split K range (bias and rotation follow in attention)
    cases = [("qkv", qkv, hidden, "bias" if tokens > 256 else "residual"), ("o", hidden, hidden, "residual"),
             ("gate_up", 2 * inter, hidden, "swiglu"), ("down", hidden, inter, "residual")]
    if tokens <= 256:
        x, gain, normed = torch.randn(tokens, hidden, device="cuda", generator=g), torch.ones(hidden, device="cuda"), rand(tokens, hidden)
        result["rmsnorm"] = {"shape": [tokens, hidden], "us": round(replayed(lambda i: kernels.rmsnorm(x, gain, normed, 1e-6)), 2)}
    for name, n, k, kind in cases:
        a, w = rand(tokens, k), rand(n, k)
        copies = min(repeats, -(-160_000_000 // (2 * n * k))) if tokens <= 256 else 1
        kw = {}
        if kind == "bias":
            out, kw = torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda"), {"bias": torch.zeros(n, device="cuda")}
        elif kind == "residual":
            out = torch.zeros(tokens, n, device="cuda")
            kw = {"residual": out, "split_k": small_batch_split_k(n, k, tokens, True, kernels.sm_count())}
        else:
            w = interleave_gate_up(w[:n // 2].contiguous(), w[n // 2:].contiguous())
            out, kw = torch.empty(tokens, n // 2, dtype=torch.bfloat16, device="cuda"), {"swiglu": True}
        ws = [w] + [w.clone() for _ in range(copies - 1)]
        us = replayed(lambda i: kernels.gemm_bf16(a, ws[i % copies], out, status, **kw))
        library = replayed(lambda i: torch.matmul(a, ws[i % copies].t()))
        result[name] = {"shape": [tokens, n, k], "epilogue": kind, "split_k": kw.get("split_k", 1), "weight_copies": copies, "us": round(us, 1),
                        "tflops": round(2.0 * tokens * n * k / us / 1e6), "weight_gbs": round(2.0 * n * k / us / 1e3),
                        "library_plain_us": round(library, 1)}
    assert int(status.item()) == 0
    return result


def run(args) -> dict:
    import numpy as np
    import torch
    from sprout_lm_b200 import kernels, load_model
    from sprout_lm_b200.cache.storage import cache_bytes_per_token
    from sprout_lm_b200.engine.step import ModelRunner
    kernels.load_library(verbose=True)
    if args.only == "attention":
        return timed_attention(args.tokens, args.shape)
    if args.only == "gemm":
        return timed_gemms(args.tokens, args.shape)
    if args.only == "decode-attention":
        return timed_decode_attention(args.shape, args.batch, args.tokens)
    if args.only == "serve":
        return timed_serving(args.shape, args.layers, args.requests, args.workload)
    if args.only == "long-prompt":
        return timed_long_prompt(args.shape, args.layers, args.tokens, args.portion)
    if args.only == "all" and args.shape != "0.5b":
        raise SystemExit("bench.py: the full line is measured at the 0.5b shape; give --only with another --shape")
    base = SHAPES[args.shape]
    layers = args.layers or base["num_hidden_layers"]
    batch, prompt_len, context = args.batch, 512, base["max_position_embeddings"]
    if args.prompt_len != 512:
        if args.only != "decode":
            raise SystemExit("bench.py: --prompt-len goes with --only decode (the full line is measured at 512-token prompts)")
        prompt_len = args.prompt_len
        need = prompt_len + args.warmup + args.steps + 8
        while context < need:                     # a longer context than the shape names: said in the line
            context *= 2
    folder = model_folder(layers, args.shape, context)
    model = load_model(folder, dtype="bfloat16", device="cuda:0")
    cfg = dict(base, num_hidden_layers=layers)
    peak = peaks()
    rng = np.random.default_rng(0)
    if prompt_len + args.warmup + args.steps + 8 > context:
        raise SystemExit(f"bench.py: {prompt_len}-token prompts and {args.warmup} + {args.steps} decode steps do not fit the "
                         f"{context}-token context of the benchmark configuration; use at most {context - prompt_len - args.warmup - 8} steps")
    slots = max(64, batch)
    pages = slots * (-(-(prompt_len + args.steps + args.warmup + 16) // 16)) + 2048 // 16 + 16
    runner = ModelRunner(model, num_pages=pages, page_tokens=16, max_requests=slots, prefix_caching=False)

    if args.only == "ablate":
        return {"impl": "ours", "only": "ablate", "shape": args.shape, "layers": layers, "batch": batch,
                **ablation(model, batch, prompt_len, min(args.steps, 60), args.warmup)}
    if args.only == "prefill":
        prefill_ms = timed_prefill(runner, 2048, rng, repeats=1)
        return {"impl": "ours", "only": "prefill", "shape": args.shape, "layers": layers, "ms": round(prefill_ms, 4),
                "frac": round(prefill_flops(cfg, 2048) / (prefill_ms / 1000) / (peak["bf16_tflops"] * 1e12), 4)}
    # the clocks are sampled over all timed sections together (a single section of a few
    # milliseconds is shorter than nvidia-smi's sampling period)
    sampler = ClockSampler()
    sampler.start()
    main = timed_decode(runner, batch, prompt_len, args.steps, args.warmup, rng)
    if args.only == "decode":
        sampler.stop()
        step_bytes = weight_bytes(model) + batch * main["mean_context"] * cache_bytes_per_token(model, torch.bfloat16)
        out = {"impl": "ours", "only": "decode", "shape": args.shape, "layers": layers, "batch": batch,
               "ms_per_step": round(main["ms_per_step"], 4), "launches_per_step": main["launches_per_step"],
               "gbs": round(step_bytes / (main["ms_per_step"] / 1000) / 1e9, 1)}
        if prompt_len != 512:
            out.update({"prompt_len": prompt_len, "context": context, "mb_per_step": round(step_bytes / 1e6, 1),
                        "hbm_frac": round(step_bytes / (main["ms_per_step"] / 1000) / 1e9 / peak["hbm_gbs"], 3)})
        phases = kernels.ffn_decode_phase_stamps()       # from a build with SPROUT_BUILD_FLAGS=-DFFN_STAMPS
        if phases:
            out["ffn_decode_phases_us"] = {k: {n: round(v, 2) for n, v in d.items()} for k, d in phases.items()}
        phases = kernels.attention_decode_phase_stamps() # from a build with SPROUT_BUILD_FLAGS=-DATTN_STAMPS
        if phases:
            out["attention_decode_phases_us"] = {n: round(v, 2) for n, v in phases.items()}
        timeline = kernels.decode_timeline()             # from a build with SPROUT_BUILD_FLAGS=-DSPROUT_TIMELINE
        if timeline:
            out["last_layer_timeline_us"] = {k: {n: round(v, 2) for n, v in d.items()} for k, d in timeline.items()}
        return out
    points = {}
    for b in (1, 64):
        points[f"decode_b{b}"] = round(timed_decode(runner, b, prompt_len, args.steps, args.warmup, rng)["tokens_per_s"], 1)
    prefill_ms = timed_prefill(runner, 2048, rng)
    flops = prefill_flops(cfg, 2048)
    e2e = timed_e2e(model, batch, prompt_len, args.steps, args.warmup, rng)
    clocks = sampler.stop()

    step_bytes = weight_bytes(model) + batch * main["mean_context"] * cache_bytes_per_token(model, torch.bfloat16)
    achieved = step_bytes / (main["ms_per_step"] / 1000) / 1e9
    return {
        "metric": "decode tokens/s, Qwen2.5-0.5B shape, batch 8 (also batch 1/64 and prefill of 2,048 tokens)",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "impl": "ours",
        "config": {"model": "Qwen2.5-0.5B shape", "layers": layers, "layers_of_model": CONFIG_05B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": 64, "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied_head": True, "global_batch": batch, "prompt_len": prompt_len, "seq_len": context,
                   "page_tokens": 16, "parallelism": "single GPU", "l2": "inputs larger than L2 (weights 988 MB per step)"},
        "e2e": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main["launches_per_step"] * args.steps),
        "prefill": {"value": round(2048 / (prefill_ms / 1000), 1), "tokens": 2048, "ms": round(prefill_ms, 4),
                    "frac": round(flops / (prefill_ms / 1000) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "peaks": peak["source"]},
        "points": points,
        "clocks": clocks,
    }


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--portion", type=int, default=4096, help="with --only long-prompt: tokens of a step (--tokens: of the whole prompt)")
    parser.add_argument("--prompt-len", type=int, default=512, help="with --only decode: tokens of every request's prompt (the context grows to hold it)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    parser.add_argument("--only", choices=["all", "decode", "prefill", "ablate", "attention", "decode-attention", "gemm", "serve", "long-prompt"], default="all",
                        help="measure one part only (for profiling captures); the JSON line then holds that part")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="0.5b", help="with --only: the model's sizes")
    parser.add_argument("--requests", type=int, default=64, help="with --only serve: requests of the workload")
    parser.add_argument("--workload", choices=["mixed", "shared-prefix"], default="mixed",
                        help="with --only serve: mixed prompt lengths, or long prompts that share a prefix in a pool too small for all")
    parser.add_argument("--tokens", type=int, default=2048, help="with --only attention or gemm: tokens of the one request; with decode-attention: the context of each request")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    result = run(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
