"""Parts alone, and the framework's generality shown with toy parts.

First each built-in part is run by itself against the plain implementation's function for
it.  Then a toy architecture is defined *here*, not in the package: a mixer that keeps state of
its own per request (a running mean of what it has seen), a feed-forward with routing (top-1
of four experts), another position encoding (rotary with a linear frequency law), layers that
differ from one another, and a run order that names a layer twice, the second time reading the
cache the first call filled.  It is registered, written as a random model folder, loaded,
stepped whole, in portions and token by token, and scheduled, with no change to the
framework's files.
"""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ------------------------------------------------------------------------------------ helpers
class FakeSeq:
    def __init__(self, pages, length, slot=-1):
        self.tables, self.length, self.state_slot = [list(pages)], length, slot


def stage(entries, page_tokens, groups=1):
    from sprout_lm_b200.engine.batch import BatchStager
    return BatchStager(torch.device(DEV), groups).stage(entries, page_tokens)


def source_for(tensors, dtype):
    from sprout_lm_b200.parts import Runtime, WeightSource
    runtime = Runtime(DEV, dtype)
    return WeightSource(lambda name: tensors[name], runtime), runtime


# ------------------------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.parts import build_part
    part = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 1e-5, "name": "ln"}), "layer.")
    assert [d.name for d in part.tensor_decls()] == ["layer.ln.weight"] and part.tensor_decls()[0].init == "gain"
    gain = 1 + 0.1 * torch.randn(72)
    source, _ = source_for({"layer.ln.weight": gain}, dtype)
    part.load(source)
    x = torch.randn(5, 72) * 3
    out = part.forward(x.to(DEV))
    want = plain.rms_norm(x.numpy(), gain.numpy(), 1e-5)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    assert np.abs(out.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    assert out.dtype == dtype


def test_rotary_part_tables_match_plain_angles():
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.parts import Runtime, build_part
    part = build_part("position", PartSpec("rope_half_split", {"head_dim": 32, "theta": 1e6, "max_positions": 300}))
    cos, sin = part.rotary_tables(Runtime(DEV, torch.float32))
    unit = np.zeros((1, 32), np.float32)
    unit[0, 3] = 1
    for pos in (0, 1, 17, 299):
        rotated = plain.rope_half_split(unit, [pos], 32, 1e6)[0]
        assert abs(rotated[3] - float(cos[pos, 3])) < 1e-7 and abs(rotated[19] - float(sin[pos, 3])) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_mlp_part(dtype):
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.parts import build_part
    part = build_part("feed_forward", PartSpec("swiglu_mlp", {"hidden_size": 72, "intermediate_size": 200}), "l.")
    tensors = {d.name: (torch.randn(*d.shape) * 0.1).to(torch.bfloat16).float() for d in part.tensor_decls()}
    source, _ = source_for(tensors, dtype)
    part.load(source)
    h = torch.randn(6, 72).to(torch.bfloat16).float()
    x = torch.randn(6, 72)
    got = x.clone().to(DEV)
    part.forward(h.to(dtype).to(DEV), got, None)
    t = plain.swiglu(plain.linear(h.numpy(), tensors["l.gate_proj.weight"].numpy()),
                     plain.linear(h.numpy(), tensors["l.up_proj.weight"].numpy()))
    want = plain.residual_add(x.numpy(), plain.linear(t, tensors["l.down_proj.weight"].numpy()))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert np.abs(got.cpu().numpy() - want).max() <= tol
    # an intermediate size that is no multiple of 8: the 32-bit path takes it, the tensor-core path refuses it at load
    odd = build_part("feed_forward", PartSpec("swiglu_mlp", {"hidden_size": 72, "intermediate_size": 28}), "l.")
    tensors = {d.name: (torch.randn(*d.shape) * 0.1).to(torch.bfloat16).float() for d in odd.tensor_decls()}
    source, _ = source_for(tensors, dtype)
    if dtype == torch.bfloat16:
        with pytest.raises(ValueError, match="multiple of 8"):
            odd.load(source)
    else:
        odd.load(source)
        got = x.clone().to(DEV)
        odd.forward(h.to(DEV), got, None)
        t = plain.swiglu(plain.linear(h.numpy(), tensors["l.gate_proj.weight"].numpy()),
                         plain.linear(h.numpy(), tensors["l.up_proj.weight"].numpy()))
        want = plain.residual_add(x.numpy(), plain.linear(t, tensors["l.down_proj.weight"].numpy()))
        assert np.abs(got.cpu().numpy() - want).max() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(4, 2, 16, 8), (3, 1, 32, 16)])
def test_attention_part_whole_then_token_by_token(dtype, heads, kv_heads, head_dim, page):
    """The mixer alone over a paged cache: a portion of 13 tokens, then 4 single tokens, against
    the plain functions (projection, rotation, causal grouped attention, output projection)."""
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.parts import CacheView, build_part
    hidden = heads * head_dim
    spec = PartSpec("gqa_attention", {"hidden_size": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
                                      "position": PartSpec("rope_half_split", {"head_dim": head_dim, "theta": 1e4,
                                                                               "max_positions": 64})})
    part = build_part("mixer", spec, "a.")
    tensors = {d.name: (torch.randn(*d.shape) * 0.2).to(torch.bfloat16).float() for d in part.tensor_decls()}
    source, runtime = source_for(tensors, dtype)
    part.load(source)
    assert part.cache_spec().kv_heads == kv_heads and part.state_spec() is None
    total = 17
    h_all = torch.randn(total, hidden).to(torch.bfloat16).float()
    pages = [5, 2, 7]
    k_cache = torch.zeros(9, kv_heads, page, head_dim, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    seq = FakeSeq(pages, 0)
    got = torch.zeros(total, hidden, device=DEV)
    for count in (13, 1, 1, 1, 1):
        entry = StepEntry(seq, [0] * count, [])
        ctx = stage([entry], page)
        view = CacheView(k_cache, v_cache, ctx.block_tables[0], page, True)
        x = torch.zeros(count, hidden, device=DEV)
        part.forward(h_all[seq.length:seq.length + count].to(dtype).to(DEV), x, ctx, view, None)
        got[seq.length:seq.length + count] = x
        seq.length += count
    n = tensors
    q = plain.linear(h_all.numpy(), n["a.q_proj.weight"].numpy(), n["a.q_proj.bias"].numpy())
    k = plain.linear(h_all.numpy(), n["a.k_proj.weight"].numpy(), n["a.k_proj.bias"].numpy())
    v = plain.linear(h_all.numpy(), n["a.v_proj.weight"].numpy(), n["a.v_proj.bias"].numpy())
    q, k = (plain.rope_half_split(t, range(total), head_dim, 1e4) for t in (q, k))
    want = plain.linear(plain.causal_gqa_attention(q, k, v, heads, kv_heads, head_dim), n["a.o_proj.weight"].numpy())
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    assert np.abs(got.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
    assert int(runtime.status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_toy_position_part_of_interleaved_pairs_over_half_the_head(dtype):
    """Another position encoding is another registered part, not an edit of a kernel: this one,
    defined here, turns only the first half of every head, in neighbouring pairs (2d, 2d + 1), by
    angles that grow linearly with the pair's index.  The attention part hands its tables, their
    width and the pairing to the kernels as launch parameters.  A portion of 20 tokens (the
    rotary kernel from float32 sums in bfloat16), then single tokens (in bfloat16 the decode
    attention kernel that rotates and appends by itself), against the same rotation in numpy."""
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.parts import CacheView, Part, build_part, register_part
    heads, kv_heads, head_dim, page, max_positions = 4, 2, 32, 8, 64
    rotary_dim = head_dim // 2

    def angles():
        d = np.arange(rotary_dim // 2, dtype=np.float64)
        return np.arange(max_positions, dtype=np.float64)[:, None] * (0.07 * (d[None, :] + 1))

    @register_part("position", "toy_interleaved_half")
    class InterleavedHalf(Part):
        interleaved = True

        def __init__(self, prefix, **_):
            pass

        def rotary_tables(self, runtime):
            a = angles()
            return (torch.from_numpy(np.cos(a).astype(np.float32)).to(runtime.device),
                    torch.from_numpy(np.sin(a).astype(np.float32)).to(runtime.device))

    def rotate(t, positions):
        n = t.shape[1] // head_dim
        ts = t.astype(np.float64).reshape(len(positions), n, head_dim).copy()
        a = angles()[list(positions)]
        c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
        even, odd = ts[..., 0:rotary_dim:2].copy(), ts[..., 1:rotary_dim:2].copy()
        ts[..., 0:rotary_dim:2] = even * c - odd * s
        ts[..., 1:rotary_dim:2] = odd * c + even * s
        return ts.reshape(len(positions), n * head_dim).astype(np.float32)

    hidden = heads * head_dim
    spec = PartSpec("gqa_attention", {"hidden_size": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
                                      "position": PartSpec("toy_interleaved_half", {})})
    part = build_part("mixer", spec, "a.")
    tensors = {d.name: (torch.randn(*d.shape, generator=torch.Generator().manual_seed(5)) * 0.2).to(torch.bfloat16).float()
               for d in part.tensor_decls()}
    source, runtime = source_for(tensors, dtype)
    part.load(source)
    assert part.interleaved and part.tables[0].shape == (max_positions, rotary_dim // 2)
    total = 25
    h_all = torch.randn(total, hidden, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).float()
    k_cache = torch.zeros(9, kv_heads, page, head_dim, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    seq = FakeSeq([5, 2, 7, 0], 0)
    got = torch.zeros(total, hidden, device=DEV)
    for count in (20, 1, 1, 1, 1, 1):
        ctx = stage([StepEntry(seq, [0] * count, [])], page)
        view = CacheView(k_cache, v_cache, ctx.block_tables[0], page, True)
        x = torch.zeros(count, hidden, device=DEV)
        part.forward(h_all[seq.length:seq.length + count].to(dtype).to(DEV), x, ctx, view, None)
        got[seq.length:seq.length + count] = x
        seq.length += count
    n = tensors
    q = plain.linear(h_all.numpy(), n["a.q_proj.weight"].numpy(), n["a.q_proj.bias"].numpy())
    k = plain.linear(h_all.numpy(), n["a.k_proj.weight"].numpy(), n["a.k_proj.bias"].numpy())
    v = plain.linear(h_all.numpy(), n["a.v_proj.weight"].numpy(), n["a.v_proj.bias"].numpy())
    q, k = rotate(q, range(total)), rotate(k, range(total))
    want = plain.linear(plain.causal_gqa_attention(q, k, v, heads, kv_heads, head_dim), n["a.o_proj.weight"].numpy())
    tol = 2e-5 if dtype == torch.float32 else 5e-2
    assert np.abs(got.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
    # and the test can fail: half-split pairs over the whole head give something else
    wrong = plain.linear(plain.causal_gqa_attention(plain.rope_half_split(q, range(total), head_dim, 1e4), k, v, heads, kv_heads,
                                                    head_dim), n["a.o_proj.weight"].numpy())
    assert np.abs(wrong - want).max() > 0.05 * np.abs(want).max()
    assert int(runtime.status.item()) == 0


def test_a_flagged_step_leaves_no_sums_behind():
    """The accumulation workspaces belong to the model's runtime; when the status word is read and
    found set they are zeroed, so that whatever a refused token left there cannot reach the next
    step."""
    from sprout_lm_b200.engine.step import ModelRunner, StepError
    from sprout_lm_b200.parts import Runtime
    runtime = Runtime(DEV, torch.bfloat16)
    a = runtime.workspace(("qkv_sums", 96), (4, 96))
    assert runtime.workspace(("qkv_sums", 96), (4, 96)) is a and float(a.abs().max()) == 0.0
    other = Runtime(DEV, torch.bfloat16)
    assert other.workspace(("qkv_sums", 96), (4, 96)) is not a        # two models never share sums
    a += 5.0
    runtime.status.fill_(16)
    fake = ModelRunner.__new__(ModelRunner)
    fake.runtime, fake._ahead = runtime, None
    with pytest.raises(StepError, match="position outside the rotary table"):
        fake.check_status()
    assert float(a.abs().max()) == 0.0 and int(runtime.status.item()) == 0


def test_weights_beyond_the_budget_are_refused_before_any_copy(tmp_path):
    from sprout_lm_b200.models import load_model
    from sprout_lm_b200.models.decoder import WeightCapacityError
    folder = helpers.make_model_dir(tmp_path, "A")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    with pytest.raises(WeightCapacityError, match="Resident weight budget exceeded"):
        load_model(folder, dtype=torch.bfloat16, weight_budget_bytes=10_000)
    assert torch.cuda.memory_allocated() - before <= 4096      # the status word at most: no tensor went up
    model = load_model(folder, dtype=torch.bfloat16, weight_budget_bytes=10_000_000)
    assert model.weight_bytes(torch.bfloat16) <= 10_000_000 and model.weight_bytes(torch.float32) > model.weight_bytes(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head_parts(dtype, tied):
    from sprout_lm_b200.config import PartSpec
    from sprout_lm_b200.parts import build_part
    vocab, hidden = 509, 72
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden, "name": "emb"}))
    head = build_part("head", PartSpec("lm_head", {"vocab_size": vocab, "hidden_size": hidden,
                                                  "tied_to": "emb" if tied else None, "name": "out"}))
    assert [d.name for d in head.tensor_decls()] == ([] if tied else ["out.weight"])
    tensors = {"emb.weight": (torch.randn(vocab, hidden) * 0.1).to(torch.bfloat16).float(),
               "out.weight": (torch.randn(vocab, hidden) * 0.1).to(torch.bfloat16).float()}
    source, runtime = source_for(tensors, dtype)
    emb.load(source)
    head.load(source)
    if tied:
        assert head.linear.weight.data_ptr() == emb.table.data_ptr()      # the same matrix, not a copy
    tokens = torch.tensor([0, 508, 17, 17], dtype=torch.int32, device=DEV)
    x = emb.forward(tokens)
    assert x.dtype == torch.float32
    np.testing.assert_array_equal(x.cpu().numpy(), plain.embed(tensors["emb.weight"].numpy(), tokens.cpu().numpy()))
    h = torch.randn(3, hidden).to(torch.bfloat16).float()
    logits = head.forward(h.to(dtype).to(DEV))
    want = plain.linear(h.numpy(), tensors["emb.weight" if tied else "out.weight"].numpy())
    assert logits.dtype == torch.float32 and logits.shape == (3, vocab)
    assert np.abs(logits.cpu().numpy() - want).max() <= 1e-5
    assert int(runtime.status.item()) == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_small_batches_take_the_light_kernels_and_agree_with_the_separate_ones(tmp_path, monkeypatch, name):
    """Up to 16 tokens a small bfloat16 layer runs as four launches (norm + q/k/v, attention, output
    projection, feed-forward with its norm); the same model loaded with SPROUT_SMALL_BATCH=0 runs
    the separate norms and tensor-core products.  Both must give the plain implementation's logits,
    and the launch counts must show that the light kernels really ran."""
    from sprout_lm_b200 import kernels
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.engine.step import ModelRunner
    from sprout_lm_b200.models import load_model
    folder = helpers.make_model_dir(tmp_path, name)
    sizes, _, page = helpers.TINY[name]
    tokens = helpers.random_tokens(np.random.default_rng(3), 46, sizes["vocab_size"])
    want = helpers.plain_logits(folder, tokens)
    results, launches = {}, {}
    for mode in ("1", "0"):
        monkeypatch.setenv("SPROUT_SMALL_BATCH", mode)
        model = load_model(folder, dtype=torch.bfloat16)
        light = mode == "1"
        assert (model.blocks[0].feed_forward._fused_tokens == 16) == light
        assert (model.blocks[0].mixer.qkv.small_tokens == 16) == light
        runner = ModelRunner(model, num_pages=12, page_tokens=page, max_requests=2, prefix_caching=False)
        runner.graphs.enabled = runner.step_graphs.enabled = False
        seq = runner.new_sequence()
        assert runner.reserve(seq, len(tokens))
        rows, at = [], 0
        for count in (8, 5, 1, 1, 3, 2, 16, 9, 1):                # portions of up to 16 tokens, and single tokens
            before = kernels.LAUNCHES
            rows.append(runner.step([StepEntry(seq, tokens[at:at + count], list(range(count)))]).float().cpu().numpy())
            launches[mode] = kernels.LAUNCHES - before
            at += count
        runner.check_status()
        results[mode] = np.concatenate(rows)
        assert np.abs(results[mode] - want).max() <= helpers.TOL["bfloat16"]
    layers = sizes["num_hidden_layers"]
    # the feed-forward's norm and one of its products fewer per layer (the norm before attention costs neither form
    # a launch in a decode step: its scale is applied inside the attention kernel)
    assert launches["0"] - launches["1"] >= 2 * layers
    assert np.abs(results["1"] - results["0"]).max() <= helpers.TOL["bfloat16"]


def test_pre_norm_block_arranges_its_parts():
    """A whole block (norm, attention, norm, feed-forward with both residuals) against the plain
    layer function, on a fresh cache."""
    from sprout_lm_b200.config import parse_config
    from sprout_lm_b200.engine.batch import StepEntry
    from sprout_lm_b200.parts import CacheView, build_block
    config = parse_config(helpers.raw_config(helpers.TINY_B))
    layer = config.model_spec().layers[1]
    block = build_block(layer)
    tensors = {d.name: ((1 if d.init == "gain" else 0) + torch.randn(*d.shape) * 0.05).to(torch.bfloat16).float()
               for d in block.tensor_decls()}
    source, runtime = source_for(tensors, torch.float32)
    block.load(source)
    tokens, page = 21, 8
    x0 = torch.randn(tokens, config.hidden_size)
    seq = FakeSeq([3, 0, 5], 0)
    ctx = stage([StepEntry(seq, [0] * tokens, [])], page)
    k_cache = torch.zeros(6, config.num_key_value_heads, page, config.head_dim, device=DEV)
    cache = CacheView(k_cache, torch.zeros_like(k_cache), ctx.block_tables[0], page, True)
    x = x0.clone().to(DEV)
    block.forward(x, ctx, cache, None)
    raw = helpers.raw_config(helpers.TINY_B)
    want = plain.decoder_layer(x0.numpy(), {n: t.numpy() for n, t in tensors.items()}, layer.prefix, raw, np.arange(tokens))
    assert np.abs(x.cpu().numpy() - want).max() <= 2e-5
    assert int(runtime.status.item()) == 0


# ------------------------------------------------------------------------------------ the toy architecture
def toy_angles(head_dim, max_positions):
    d = np.arange(head_dim // 2, dtype=np.float64)
    return np.arange(max_positions, dtype=np.float64)[:, None] * (0.05 * (d[None, :] + 1))


def register_toy_parts():
    from sprout_lm_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture
    from sprout_lm_b200.parts import Part, StateSpec, TensorDecl, register_part

    @register_part("position", "toy_linear_rotary")
    class LinearRotary(Part):
        def __init__(self, prefix, head_dim, max_positions):
            self.head_dim, self.max_positions = head_dim, max_positions

        def rotary_tables(self, runtime):
            angle = toy_angles(self.head_dim, self.max_positions)
            return (torch.from_numpy(np.cos(angle).astype(np.float32)).to(runtime.device),
                    torch.from_numpy(np.sin(angle).astype(np.float32)).to(runtime.device))

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Part):
        """out_t = W mean(h_0..h_t): keeps the sum and the count of what it has seen per request."""

        def __init__(self, prefix, hidden_size):
            self.hidden, self.name = hidden_size, prefix + "mean_proj.weight"

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec(shape=(self.hidden + 1,), dtype=torch.float32)

        def tensor_decls(self):
            return [TensorDecl(self.name, (self.hidden, self.hidden))]

        def load(self, source):
            self.weight = source.raw(self.name).float().to(source.runtime.device)

        def forward(self, h, x, ctx, cache, state):
            h32 = h.float()
            slots = state.slots.long()
            if ctx.max_q_len == 1:                          # one token per request: no host round trip
                state.buffer[slots, :self.hidden] += h32
                state.buffer[slots, self.hidden] += 1
                mean = state.buffer[slots, :self.hidden] / state.buffer[slots, self.hidden:self.hidden + 1]
            else:
                starts = ctx.q_start.tolist()
                mean = torch.empty_like(h32)
                for r in range(ctx.num_seqs):
                    a, b = starts[r], starts[r + 1]
                    slot = int(slots[r])
                    sums = state.buffer[slot, :self.hidden] + torch.cumsum(h32[a:b], 0)
                    counts = state.buffer[slot, self.hidden] + torch.arange(1, b - a + 1, device=h.device)
                    mean[a:b] = sums / counts[:, None]
                    state.buffer[slot, :self.hidden] = sums[-1]
                    state.buffer[slot, self.hidden] = counts[-1]
            x += mean @ self.weight.T

    @register_part("feed_forward", "toy_routed")
    class Routed(Part):
        """Top-1 of `experts` square experts, router logits in float32."""

        def __init__(self, prefix, hidden_size, experts):
            self.hidden, self.experts, self.prefix = hidden_size, experts, prefix

        def tensor_decls(self):
            decls = [TensorDecl(self.prefix + "router.weight", (self.experts, self.hidden))]
            decls += [TensorDecl(f"{self.prefix}experts.{e}.weight", (self.hidden, self.hidden)) for e in range(self.experts)]
            return decls

        def load(self, source):
            device = source.runtime.device
            self.router = source.raw(self.prefix + "router.weight").float().to(device)
            self.stack = torch.stack([source.raw(f"{self.prefix}experts.{e}.weight").float()
                                      for e in range(self.experts)]).to(device)

        def forward(self, h, x, ctx):
            h32 = h.float()
            choice = (h32 @ self.router.T).argmax(-1)
            x += torch.bmm(self.stack[choice], h32.unsqueeze(-1)).squeeze(-1)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden_size: int = 48
        heads: int = 3
        kv_heads: int = 1
        intermediate_size: int = 64
        vocab_size: int = 101
        max_positions: int = 256
        eps: float = 1e-5
        experts: int = 4
        eos_token_ids: tuple = (100,)
        architecture = "ToyForCausalLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(**{k: (tuple(v) if isinstance(v, list) else v) for k, v in raw.items()
                          if k in cls.__dataclass_fields__})

        def to_dict(self):
            return {"architectures": [self.architecture], "model_type": "toy",
                    **{k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}}

        def with_eos(self, ids):
            return self

        def model_spec(self):
            head_dim = self.hidden_size // self.heads
            norm = lambda name: PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.eps, "name": name})
            attention = PartSpec("gqa_attention", {
                "hidden_size": self.hidden_size, "heads": self.heads, "kv_heads": self.kv_heads, "head_dim": head_dim,
                "position": PartSpec("toy_linear_rotary", {"head_dim": head_dim, "max_positions": self.max_positions})})
            layers = (
                LayerSpec("pre_norm", "layers.0.", attention,
                          PartSpec("toy_routed", {"hidden_size": self.hidden_size, "experts": self.experts}),
                          (norm("ln1"), norm("ln2"))),
                LayerSpec("pre_norm", "layers.1.", PartSpec("toy_running_mean", {"hidden_size": self.hidden_size}),
                          PartSpec("swiglu_mlp", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}),
                          (norm("ln1"), norm("ln2"))),
                LayerSpec("pre_norm", "layers.2.", attention,
                          PartSpec("swiglu_mlp", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}),
                          (norm("ln1"), norm("ln2"))),
            )
            # layer 0 runs twice; its second run reads the keys and values its first run cached; layer 2 (weights
            # of its own) has no cache: its queries attend over what layer 0 cached
            order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 0, writes_cache=False), LayerCall(2, 0, writes_cache=False))
            return ModelSpec(
                architecture=self.architecture, hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                max_positions=self.max_positions,
                embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                                       "name": "embed"}),
                layers=layers, order=order, final_norm=norm("final_ln"),
                head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                          "tied_to": None, "name": "head"}),
                eos_token_ids=self.eos_token_ids)

    register_architecture("ToyForCausalLM", ToyConfig, model_types=("toy",))
    return ToyConfig


def toy_plain_logits(cfg, w, tokens):
    """The toy model in the plain manner: whole sequence, no cache, float64 sums."""
    T, H = len(tokens), cfg.hidden_size
    heads, kv, hd = cfg.heads, cfg.kv_heads, cfg.hidden_size // cfg.heads
    x = plain.embed(w["embed.weight"], tokens)

    def rotate(t):
        angle = toy_angles(hd, cfg.max_positions)[:T]
        n = t.shape[1] // hd
        ts = t.astype(np.float64).reshape(T, n, hd)
        a, b = ts[..., :hd // 2], ts[..., hd // 2:]
        c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
        return np.concatenate([a * c - b * s, b * c + a * s], -1).reshape(T, n * hd).astype(np.float32)

    def layer0(x):
        p = "layers.0."
        h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps)
        q = rotate(plain.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]))
        k = rotate(plain.linear(h, w[p + "k_proj.weight"], w[p + "k_proj.bias"]))
        v = plain.linear(h, w[p + "v_proj.weight"], w[p + "v_proj.bias"])
        return x, h, q, k, v

    def finish0(x, q, k, v):
        p = "layers.0."
        x = plain.residual_add(x, plain.linear(plain.causal_gqa_attention(q, k, v, heads, kv, hd), w[p + "o_proj.weight"]))
        h2 = plain.rms_norm(x, w[p + "ln2.weight"], cfg.eps)
        choice = np.argmax(plain.linear(h2, w[p + "router.weight"]), -1)
        out = np.stack([w[f"{p}experts.{e}.weight"].astype(np.float64) @ h2[t].astype(np.float64)
                        for t, e in enumerate(choice)]).astype(np.float32)
        return plain.residual_add(x, out)

    x, _, q, k0, v0 = layer0(x)
    x = finish0(x, q, k0, v0)
    p = "layers.1."
    h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps)
    mean = (np.cumsum(h.astype(np.float64), 0) / np.arange(1, T + 1)[:, None]).astype(np.float32)
    x = plain.residual_add(x, plain.linear(mean, w[p + "mean_proj.weight"]))
    h2 = plain.rms_norm(x, w[p + "ln2.weight"], cfg.eps)
    t = plain.swiglu(plain.linear(h2, w[p + "gate_proj.weight"]), plain.linear(h2, w[p + "up_proj.weight"]))
    x = plain.residual_add(x, plain.linear(t, w[p + "down_proj.weight"]))
    # layer 0 again: new queries from the current stream, but the keys and values cached by its first run
    x, _, q, _, _ = layer0(x)
    x = finish0(x, q, k0, v0)
    # layer 2: its own weights, its queries over layer 0's cached keys and values, a dense feed-forward
    p = "layers.2."
    h = plain.rms_norm(x, w[p + "ln1.weight"], cfg.eps)
    q = rotate(plain.linear(h, w[p + "q_proj.weight"], w[p + "q_proj.bias"]))
    x = plain.residual_add(x, plain.linear(plain.causal_gqa_attention(q, k0, v0, heads, kv, hd), w[p + "o_proj.weight"]))
    h2 = plain.rms_norm(x, w[p + "ln2.weight"], cfg.eps)
    t = plain.swiglu(plain.linear(h2, w[p + "gate_proj.weight"]), plain.linear(h2, w[p + "up_proj.weight"]))
    x = plain.residual_add(x, plain.linear(t, w[p + "down_proj.weight"]))
    return plain.linear(plain.rms_norm(x, w["final_ln.weight"], cfg.eps), w["head.weight"])


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from sprout_lm_b200 import write_random_model
    config_class = register_toy_parts()
    config = config_class()
    folder = write_random_model(tmp_path_factory.mktemp("toy") / "model", config, seed=5)
    return config, folder


def test_toy_architecture_is_registered_built_and_stepped(toy):
    from sprout_lm_b200 import load_model
    from sprout_lm_b200.engine.step import ModelRunner
    config, folder = toy
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyForCausalLM"]
    _, weights = plain.read_model_folder(folder)
    assert "layers.0.experts.3.weight" in weights and "layers.1.mean_proj.weight" in weights
    model = load_model(folder, dtype="float32")
    assert [type(b.mixer).__name__ for b in model.blocks] == ["PagedGQAttention", "RunningMean", "PagedGQAttention"]
    assert model.cache_specs()[1] is None and model.state_specs()[1].shape == (49,)
    rng = np.random.default_rng(0)
    requests = {f"t{i}": helpers.random_tokens(rng, n, config.vocab_size) for i, n in enumerate((9, 40, 23))}
    want = {rid: toy_plain_logits(config, weights, toks) for rid, toks in requests.items()}
    for label, plan in (("whole", helpers.plan_whole(requests)),
                        ("tail", helpers.plan_tail_decode(requests, tail=6)),
                        ("portions", helpers.plan_portions(requests)),
                        ("mixed", helpers.plan_mixed(requests, np.random.default_rng(3), max_live=3))):
        runner = ModelRunner(model, num_pages=16, page_tokens=8, max_requests=4)
        assert not runner.manager.prefix_caching and runner.manager.state_slot_count == 4
        got = helpers.run_plan_in_process(runner, plan)
        for rid, toks in requests.items():
            for pos in range(len(toks)):
                err = float(np.abs(got[(rid, pos)] - want[rid][pos]).max())
                assert err <= 2e-5, (label, rid, pos, err)
        assert runner.manager.snapshot()["stateSlots"]["free"] == 4 and runner.manager.free_pages() == 16


def test_toy_architecture_generates_through_the_scheduler(toy):
    """State slots, preemption and recomputation with a mixer whose state must be rebuilt."""
    from sprout_lm_b200 import EngineOptions, generate, load_model, make_engine
    config, folder = toy
    _, weights = plain.read_model_folder(folder)
    model = load_model(folder, dtype="float32")
    rng = np.random.default_rng(4)
    prompts = [helpers.random_tokens(rng, n, config.vocab_size) for n in (5, 21, 12)]
    engine = make_engine(model, EngineOptions(block_size=8, num_blocks=6, max_sequences=3, max_batch_tokens=12,
                                              prefill_chunk_size=5))
    results = generate(model, prompts, max_new_tokens=10, ignore_eos=True, engine=engine)
    assert any(e["type"] == "preempted" for e in engine.trace)
    for prompt, result in zip(prompts, results):
        history = list(prompt)
        for token in result["output"]:
            row = toy_plain_logits(config, weights, history)[-1]
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 1e-4:
                assert token == int(np.argmax(row))
            history.append(token)
        assert result["prefix_hits"] == 0
    assert engine.cache.snapshot()["stateSlots"]["free"] == 3
