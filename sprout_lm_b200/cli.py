"""Command line in the manner of the reference's demo (src/demo.ts) and smoke script
(scripts/smoke-cuda.ts).

    python -m sprout_lm_b200 demo [--model DIR | --tiny A|B] [--seed S] [--json] [--pressure] [--dtype bfloat16|float32]
    python -m sprout_lm_b200 generate (--model DIR | --tiny A|B) --prompt 1,2,3 [--max-new-tokens N]
                                      [--temperature T] [--seed S] [--ignore-eos] [--json]
    python -m sprout_lm_b200 random-model --out DIR --config CONFIG.json [--seed S]

``demo`` runs the reference demo's scenario on a model: requests A and B at the start, C
(sharing a prefix with A) after two ticks, with ``blockSize 4``, ``numBlocks 18`` (5 with
``--pressure``), ``maxSequences 3``, ``maxBatchTokens 6``, ``prefillChunkSize 4``; every tick
it prints free and cached pages, a table of the work done (request, phase, position, tokens,
logical -> physical pages) and the events; at the end the results.  ``--json`` prints
``{mode, reports, results}`` instead.  Without ``--model`` it writes a tiny random model (``--tiny``,
A if not given, weights from ``--seed``) to a temporary folder first.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time

# Two tiny random models that differ in every size and option (--tiny A|B; A is the default of demo)
TINY = {
    "A": dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6,
              rope_theta=10000.0, tie_word_embeddings=True, eos_token_id=255),
    "B": dict(hidden_size=96, intermediate_size=320, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, vocab_size=509, max_position_embeddings=256, rms_norm_eps=1e-5,
              rope_theta=1000000.0, tie_word_embeddings=False, eos_token_id=[507, 508]),
}
DEMO_TINY = TINY["A"]


def _table(rows: list[dict]) -> str:
    if not rows:
        return "  (no work)"
    columns = list(rows[0])
    widths = [max(len(str(c)), *(len(str(r[c])) for r in rows)) for c in columns]
    line = lambda cells: "  " + " | ".join(str(c).ljust(w) for c, w in zip(cells, widths))
    return "\n".join([line(columns), "  " + "-+-".join("-" * w for w in widths), *(line([r[c] for c in columns]) for r in rows)])


def _load(args):
    from . import load_model, parse_config, write_random_model
    if args.model and getattr(args, "tiny", None):
        raise SystemExit("give --model DIR or --tiny A|B, not both")
    if args.model:
        return load_model(args.model, dtype=args.dtype), None
    tmp = tempfile.TemporaryDirectory()
    sizes = TINY[getattr(args, "tiny", None) or "A"]
    config = parse_config({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu", **sizes})
    write_random_model(tmp.name, config, seed=args.seed)
    return load_model(tmp.name, dtype=args.dtype), tmp


def run_demo(args) -> int:
    import numpy as np
    from . import EngineOptions, make_engine
    model, tmp = _load(args)
    options = EngineOptions(block_size=args.block_size, num_blocks=5 if args.pressure else 18, max_sequences=3,
                            max_batch_tokens=6, prefill_chunk_size=4)
    engine = make_engine(model, options)
    rng = np.random.default_rng(args.seed)
    vocab = model.spec.vocab_size
    draw = lambda n: [int(t) for t in rng.integers(0, vocab, size=n)]
    shared = draw(8)
    prompts = {"A": shared + draw(2), "B": draw(5), "C": shared + draw(3)}
    if not args.json:
        print(f"sprout_lm_b200 · {model.spec.architecture} on {model.runtime.device} ({args.dtype}), random token prompts")
        print("Token IDs demonstrate scheduling and numerical correctness, not language quality.\n")
    engine.add("A", prompts["A"], 7, ignore_eos=True)
    engine.add("B", prompts["B"], 4, ignore_eos=True)
    reports, iterations = [], 0
    while engine.pending:
        if iterations == 2:
            engine.add("C", prompts["C"], 3, ignore_eos=True)   # arrives while A and B run
        iterations += 1
        if iterations > 2000:
            raise RuntimeError("Demo did not converge.")
        report = engine.step().resolve()      # take the page snapshot now, before the next tick changes it
        reports.append(report)
        if not args.json:
            memory = report["memory"]
            print(f"Tick {report['tick']} | free pages {memory['freePages']}/{memory['totalPages']} | cached {memory['cachedPages']}")
            print(_table([{"request": w["id"], "phase": w["phase"], "position": w["from"], "tokens": w["tokens"],
                           "logical → physical pages": " ".join(f"{i}→{p}" for i, p in enumerate(w["blockTable"]))}
                          for w in report["work"]]))
            for event in report["events"]:
                print(f"  {event['id']} {event['type']}: {event['detail']}")
            print()
    engine.runner.check_status()
    results = [engine.result(name) for name in ("A", "B", "C")]
    if args.json:
        print(json.dumps({"mode": "pressure" if args.pressure else "normal", "reports": reports, "results": results}, indent=2))
    else:
        print("Results:")
        print(_table([{"request": r["id"], "status": r["status"], "prefix tokens reused": r["prefixHits"],
                       "output": ", ".join(map(str, r["output"]))} for r in results]))
        print("Cached pages may remain after requests finish; their activeRefs are zero.")
    if tmp:
        tmp.cleanup()
    return 0


def run_generate(args) -> int:
    from . import EngineOptions, make_engine
    from .engine.generate import default_options
    started = time.perf_counter()
    model, tmp = _load(args)
    load_ms = (time.perf_counter() - started) * 1000
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt]
    options = default_options(prompts, args.max_new_tokens)
    engine = make_engine(model, options)
    for i, prompt in enumerate(prompts):
        engine.add(f"request-{i}", prompt, args.max_new_tokens, temperature=args.temperature, seed=args.seed,
                   ignore_eos=args.ignore_eos)
    rounds, first_token_ms = [], None
    begun = time.perf_counter()
    while engine.pending:
        before = time.perf_counter()
        report = engine.step()
        tokens = [e["token"] for e in report["events"] if e["type"] == "token"]
        if tokens and first_token_ms is None:
            first_token_ms = (time.perf_counter() - begun) * 1000
        phase = report["work"][0]["phase"] if report["work"] else "none"
        rounds.append({"round": len(rounds) + 1, "ms": (time.perf_counter() - before) * 1000, "phase": phase, "tokens": tokens})
        if args.json:
            print(json.dumps(rounds[-1]))
    engine.runner.check_status()
    decode = [r for r in rounds if r["phase"] == "decode"]
    decode_ms = sum(r["ms"] for r in decode)
    summary = {"loadMs": load_ms, "firstTokenMs": first_token_ms, "generationMs": (time.perf_counter() - begun) * 1000,
               "decodeSummary": {"steps": len(decode), "totalMs": decode_ms,
                                 "meanMs": decode_ms / len(decode) if decode else None,
                                 "stepsPerSecond": len(decode) * 1000 / decode_ms if decode_ms else None},
               "results": [engine.result(f"request-{i}") for i in range(len(prompts))],
               "kv": {k: v for k, v in engine.cache.snapshot().items() if k != "pages"}}
    if args.json:
        print(json.dumps({"phase": "finished", "report": summary}))
    else:
        for r in summary["results"]:
            print(f"{r['id']}: {r['finishReason']}: {', '.join(map(str, r['output']))}")
        d = summary["decodeSummary"]
        print(f"first token {first_token_ms:.1f} ms; {d['steps']} decode steps, mean "
              f"{(d['meanMs'] or 0):.3f} ms")
    if tmp:
        tmp.cleanup()
    return 0


def run_random_model(args) -> int:
    from . import parse_config, write_random_model
    with open(args.config) as handle:
        config = parse_config(json.load(handle))
    path = write_random_model(args.out, config, seed=args.seed, dtype=args.store)
    print(path)
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="sprout_lm_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    demo = sub.add_parser("demo", help="the reference demo's scenario, tick by tick")
    demo.add_argument("--json", action="store_true")
    demo.add_argument("--pressure", action="store_true", help="5 pages instead of 18: forces preemption")
    demo.add_argument("--block-size", type=int, default=4)
    gen = sub.add_parser("generate", help="generate from token-id prompts")
    gen.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeatable")
    gen.add_argument("--max-new-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--json", action="store_true")
    for p in (demo, gen):
        p.add_argument("--model", help="folder with config.json and model.safetensors")
        p.add_argument("--tiny", choices=sorted(TINY), help="instead of --model: a tiny random model (A: 2 layers, hidden 64, "
                       "4/2 heads of 16, tied head; B: 3 layers, hidden 96, 3/1 heads of 32, untied head), written with --seed")
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
        p.add_argument("--seed", type=int, default=0)
    rnd = sub.add_parser("random-model", help="write config.json and model.safetensors with random weights")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--config", required=True, help="a config.json of a registered architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--store", choices=["bfloat16", "float32"], default="bfloat16")
    args = parser.parse_args(argv)
    return {"demo": run_demo, "generate": run_generate, "random-model": run_random_model}[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
