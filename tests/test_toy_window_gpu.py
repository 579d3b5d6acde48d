"""A toy mixer that keeps only a window of keys, defined here and not in the package.

The framework's own architecture keeps every key.  This toy architecture has one layer of the
built-in attention (a group of pages that keeps every position) and one layer of a mixer that
attends over the last ``window`` positions only and encodes position as a penalty on the
distance, so the engine runs two page groups with pools of different sizes: the window group's
pages are given back while a request is still running and are used again, by the same request
and by others.  The mixer is plain tensor code (gathers through the block table): what is under
test is the cache manager's window group, the step's block tables of two groups, the captured
decode step's table rewrite, and that none of it needs a change to the framework's files.

The mixer writes NaN where a key that it has to read lies in a page that was given back, so a
page trimmed too early fails the comparison instead of reading whatever the page holds now.
"""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


def register_window_parts():
    from sprout_lm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture
    from sprout_lm_b200.parts import CacheSpec, Part, TensorDecl, register_part

    @register_part("mixer", "toy_window_attention")
    class WindowAttention(Part):
        """Each query sees the keys at most ``window - 1`` positions before it; a head's score falls
        by ``slope * (head + 1)`` per position of distance."""

        def __init__(self, prefix, hidden_size, heads, head_dim, window, slope):
            self.hidden, self.heads, self.head_dim, self.window, self.slope = hidden_size, heads, head_dim, window, slope
            self.prefix = prefix

        def cache_spec(self):
            return CacheSpec(kv_heads=1, head_dim=self.head_dim, kind="window", window=self.window)

        def state_spec(self):
            return None

        def tensor_decls(self):
            p, width = self.prefix, self.heads * self.head_dim
            return [TensorDecl(p + "wq.weight", (width, self.hidden)), TensorDecl(p + "wk.weight", (self.head_dim, self.hidden)),
                    TensorDecl(p + "wv.weight", (self.head_dim, self.hidden)), TensorDecl(p + "wo.weight", (self.hidden, width))]

        def load(self, source):
            dev = source.runtime.device
            self.wq, self.wk, self.wv, self.wo = (source.raw(self.prefix + n + ".weight").float().to(dev)
                                                  for n in ("wq", "wk", "wv", "wo"))

        def forward(self, h, x, ctx, cache, state):
            h32 = h.float()
            T, P = h32.shape[0], cache.page_tokens
            q = (h32 @ self.wq.T).view(T, self.heads, self.head_dim)
            k, v = h32 @ self.wk.T, h32 @ self.wv.T
            pos, seq = ctx.positions.long(), ctx.seq_of_token.long()
            table = cache.block_table.long()
            if cache.write:
                pages = table[seq, pos // P]
                cache.k[pages, 0, pos % P] = k.to(cache.k.dtype)
                cache.v[pages, 0, pos % P] = v.to(cache.v.dtype)
            back = torch.arange(self.window, device=h.device)
            key_pos = pos[:, None] - back[None, :]                               # [T, window]
            seen = key_pos >= 0
            key_pos = key_pos.clamp(min=0)
            pages = table[seq[:, None], key_pos // P]
            lost = seen & (pages < 0)                                            # a key in a page given back
            pages = pages.clamp(min=0)
            keys = cache.k[pages, 0, key_pos % P].float()                        # [T, window, head_dim]
            values = cache.v[pages, 0, key_pos % P].float()
            scores = torch.einsum("thd,twd->thw", q, keys) / self.head_dim ** 0.5
            heads = torch.arange(1, self.heads + 1, device=h.device, dtype=torch.float32)
            scores = scores - self.slope * heads[None, :, None] * back[None, None, :].float()
            scores = scores.masked_fill(~seen[:, None, :], float("-inf"))
            out = torch.einsum("thw,twd->thd", torch.softmax(scores, -1), values).reshape(T, -1)
            out = torch.where(lost.any(-1, keepdim=True), torch.full_like(out, float("nan")), out)
            x += out @ self.wo.T

    @dataclass
    class WindowConfig:
        hidden_size: int = 40
        heads: int = 5
        window: int = 12
        slope: float = 0.07
        intermediate_size: int = 56
        vocab_size: int = 97
        max_positions: int = 512
        eps: float = 1e-6
        eos_token_ids: tuple = (96,)
        architecture = "ToyWindowForCausalLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in raw.items()
                          if k in cls.__dataclass_fields__})

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": "toy_window",
                    **{k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}}

        def with_eos(self, ids):
            return self

        def model_spec(self):
            head_dim = 16
            norm = lambda name: PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps, "name": name})
            mlp = PartSpec("swiglu_mlp", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size})
            full = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "heads": 2, "kv_heads": 1, "head_dim": head_dim,
                "position": PartSpec("rope_half_split", {"head_dim": head_dim, "theta": 10000.0, "max_positions": self.max_positions})})
            window = PartSpec("toy_window_attention", {"hidden_size": self.hidden_size, "heads": self.heads,
                                                       "head_dim": head_dim, "window": self.window, "slope": self.slope})
            layers = (LayerSpec("pre_norm", "layers.0.", full, mlp, (norm("ln1"), norm("ln2"))),
                      LayerSpec("pre_norm", "layers.1.", window, mlp, (norm("ln1"), norm("ln2"))))
            return ModelSpec(
                architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                max_positions=self.max_positions,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                                       "name": "embed"}),
                layers=layers, order=(LayerCall(0, 0), LayerCall(1, 1)), final_norm=norm("final_ln"),
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                          "tied_to": None, "name": "head"}),
                eos_token_ids=self.eos_token_ids)

    register_architecture("ToyWindowForCausalLM", WindowConfig, model_types=("toy_window",))
    return WindowConfig


def window_plain_logits(cfg, w, tokens):
    """The toy model in the plain manner: whole sequence, no cache, float64 sums."""
    T, hd = len(tokens), 16
    x = plain.embed(w["embed.weight"], tokens)

    def feed_forward(x, p):
        h2 = plain.rms_norm(x, w[p + "ln2.weight"], cfg.eps)
        t = plain.swiglu(plain.linear(h2, w[p + "gate_proj.weight"]), plain.linear(h2, w[p + "up_proj.weight"]))
        return plain.residual_add(x, plain.linear(t, w[p + "down_proj.weight"]))

    p = "layers.0."
    h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps)
    q = plain.rope_half_split(plain.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]), range(T), hd, 10000.0)
    k = plain.rope_half_split(plain.linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]), range(T), hd, 10000.0)
    v = plain.linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"])
    x = plain.residual_add(x, plain.linear(plain.causal_gqa_attention(q, k, v, 2, 1, hd), w[p + "o_proj.weight"]))
    x = feed_forward(x, p)

    p = "layers.1."
    h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps).astype(np.float64)
    q = (h @ w[p + "wq.weight"].astype(np.float64).T).reshape(T, cfg.heads, hd)
    k = h @ w[p + "wk.weight"].astype(np.float64).T
    v = h @ w[p + "wv.weight"].astype(np.float64).T
    out = np.zeros((T, cfg.heads, hd))
    for t in range(T):
        first = max(0, t - cfg.window + 1)
        distance = (t - np.arange(first, t + 1)).astype(np.float64)
        for head in range(cfg.heads):
            scores = k[first:t + 1] @ q[t, head] / np.sqrt(hd) - cfg.slope * (head + 1) * distance
            weights = np.exp(scores - scores.max())
            out[t, head] = (weights / weights.sum()) @ v[first:t + 1]
    mixed = (out.reshape(T, -1) @ w[p + "wo.weight"].astype(np.float64).T).astype(np.float32)
    x = feed_forward(plain.residual_add(x, mixed), p)
    return plain.linear(plain.rms_norm(x, w["final_ln.weight"], cfg.eps), w["head.weight"])


@pytest.fixture(scope="module")
def window_toy(tmp_path_factory):
    from sprout_lm_b200 import write_random_model
    config = register_window_parts()()
    folder = write_random_model(tmp_path_factory.mktemp("toy_window") / "model", config, seed=11)
    return config, folder


PAGE = 8


def test_window_group_gives_pages_back_while_requests_run_and_uses_them_again(window_toy):
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    config, folder = window_toy
    _, weights = plain.read_model_folder(folder)
    model = load_model(folder, dtype="float32")
    specs = model.cache_specs()
    assert specs[0].kind == "full" and (specs[1].kind, specs[1].window) == ("window", config.window)
    rng = np.random.default_rng(2)
    requests = {f"w{i}": helpers.random_tokens(rng, n, config.vocab_size) for i, n in enumerate((90, 61, 33, 75))}
    want = {rid: window_plain_logits(config, weights, toks) for rid, toks in requests.items()}
    all_pages = sum(-(-len(t) // PAGE) for t in requests.values())
    # the window group gets fewer pages than one long request has positions for: a step of at most 16
    # tokens needs the pages of window + 16 positions, and three requests are live at a time
    window_pool = 3 * (-(-(config.window + 16) // PAGE) + 1)
    assert window_pool < all_pages
    for label, plan in (("tail", [s for rid, toks in requests.items() for s in tail_in_portions(rid, toks)]),
                        ("portions", helpers.plan_portions(requests)),
                        ("mixed", helpers.plan_mixed(requests, np.random.default_rng(5), max_live=3, portion=(2, 16)))):
        runner = ModelRunner(model, num_pages=[all_pages, window_pool], page_tokens=PAGE, max_requests=4)
        groups = runner.manager.groups
        assert [g.kind for g in groups] == ["full", "window"] and not runner.manager.prefix_caching
        got = helpers.run_plan_in_process(runner, plan)
        for rid, toks in requests.items():
            for pos in range(len(toks)):
                err = float(np.abs(got[(rid, pos)] - want[rid][pos]).max())
                assert err <= 2e-5, (label, rid, pos, err)          # NaN (a key in a page given back) fails too
        assert runner.manager.free_pages(0) == all_pages and runner.manager.free_pages(1) == window_pool
        runner.manager.check_invariants()


def tail_in_portions(rid, toks, tail=32, portion=16):
    """Portions of ``portion`` tokens, then the last ``tail`` tokens one by one."""
    head = len(toks) - tail
    steps = [{"entries": [(rid, toks[a:min(a + portion, head)], list(range(min(a + portion, head) - a)))], "end": []}
             for a in range(0, head, portion)]
    steps += [{"entries": [(rid, [toks[i]], [0])], "end": []} for i in range(head, len(toks))]
    steps[-1]["end"] = [rid]
    return steps


def test_window_group_trims_as_the_cache_manager_says(window_toy):
    """After every step a request holds, in the window group, exactly the pages that a later query
    can still see."""
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    config, folder = window_toy
    model = load_model(folder, dtype="float32")
    runner = ModelRunner(model, num_pages=[16, 5], page_tokens=PAGE, max_requests=2)
    seq = runner.new_sequence()
    tokens = helpers.random_tokens(np.random.default_rng(1), 70, config.vocab_size)
    at = 0
    for n in (5, 11, 2, 16, 1, 1, 9, 1, 13, 1, 1, 1, 8):
        assert runner.reserve(seq, at + n)
        runner.step([StepEntry(seq, tokens[at:at + n], [n - 1])])
        runner.check_status()
        at += n
        first_needed = max(0, at - config.window + 1)
        held = [i for i, page in enumerate(seq.tables[1]) if page >= 0]
        assert held == list(range(first_needed // PAGE, -(-at // PAGE))), (at, seq.tables[1])
        assert all(page >= 0 for page in seq.tables[0]) and len(seq.tables[0]) == -(-at // PAGE)
    runner.release(seq)
    assert runner.manager.free_pages(1) == 5


def test_window_toy_generates_through_the_scheduler_and_captured_decode_steps(window_toy):
    """Greedy generation through the entry point: decode steps are captured and replayed, their
    tables of the window group rewritten as pages are given back, steps are launched behind one
    another, and a pool too small for everyone preempts."""
    from sprout_lm_b200 import EngineOptions, generate, load_model, make_engine
    config, folder = window_toy
    _, weights = plain.read_model_folder(folder)
    model = load_model(folder, dtype="float32")
    rng = np.random.default_rng(8)
    prompts = [helpers.random_tokens(rng, n, config.vocab_size) for n in (7, 30, 18)]
    engine = make_engine(model, EngineOptions(block_size=PAGE, num_blocks=9, max_sequences=3, max_batch_tokens=16,
                                              prefill_chunk_size=8))
    results = generate(model, prompts, max_new_tokens=40, ignore_eos=True, engine=engine)
    assert any(e["type"] == "preempted" for e in engine.trace)
    for prompt, result in zip(prompts, results):
        assert len(result["output"]) == 40
        history = list(prompt)
        for token in result["output"]:
            row = window_plain_logits(config, weights, history)[-1]
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 1e-4:
                assert token == int(np.argmax(row)), (len(history), token)
            history.append(token)
    snapshot = engine.cache.snapshot()
    assert json.dumps(snapshot)                     # the snapshot names both groups and serialises
    assert engine.cache.free_pages(0) == 9 and engine.cache.free_pages(1) == 9
