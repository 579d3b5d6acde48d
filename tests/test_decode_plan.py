"""How decode attention divides a request's keys among CTAs (no GPU needed: the plan is host
arithmetic), and that a captured decode step is keyed by it."""
import pytest

from sprout_lm_b200 import kernels


@pytest.mark.parametrize("head_dim,kv_heads", [(16, 1), (64, 2), (128, 4), (128, 8)])
@pytest.mark.parametrize("requests", [1, 3, 8, 33, 64, 200])
def test_plan_covers_every_key(head_dim, kv_heads, requests):
    for max_keys in (16, 128, 640, 1000, 4096, 33000):
        for live in (None, 1, max_keys // 2, max_keys, 10 * max_keys):
            split_keys, splits, through_memory = kernels.decode_split_plan(requests, kv_heads, max_keys, head_dim, live)
            assert split_keys % 128 == 0 and split_keys >= 128
            assert split_keys * splits >= max_keys                  # every key has a split
            assert split_keys * (splits - 1) < max(max_keys, 128)   # and no split is wholly beyond the table
            assert through_memory or splits <= 8                    # a cluster holds at most 8 CTAs
            assert not (through_memory and splits == 1)             # nothing to merge


def test_plan_counts_the_ctas_an_sm_really_holds():
    """The plan's waves follow how many CTAs an SM holds, through memory and in clusters (whose CTAs
    hold more shared memory); a launch of many waves goes through memory even where its splits
    would fit a cluster."""
    # without a device the counts are what shared memory and the kernel's register bounds give on a B200
    counts = kernels.decode_ctas_per_sm.__wrapped__
    assert (counts(64), counts(64, True), counts(128), counts(128, True)) == (5, 4, 3, 2)
    assert counts(80) == 4 and counts(16) == 5
    # 64 requests x 4 key/value heads of 128 over 8,192 keys: more CTAs than places, splits through memory
    split_keys, splits, through_memory = kernels._decode_split_plan(256, 64, 64, 128, 148, 3, 2)
    assert through_memory and splits <= 8 and split_keys * splits >= 8192
    # the same pairs with 640 keys each: one split per pair, all resident at once, nothing to merge
    assert kernels._decode_split_plan(256, 5, 5, 128, 148, 3, 2) == (640, 1, False)
    # fewer places per SM: another plan for a launch that no longer fits one wave
    assert kernels._decode_split_plan(128, 65, 65, 64, 148, 5, 4) != kernels._decode_split_plan(128, 65, 65, 64, 148, 3, 2)


def test_plan_keeps_the_picks_that_were_measured():
    """The cost model's picks for the cases that were timed on a B200 against every other split size
    (0.5B and 7B head shapes, 148 SMs, 5 / 4 and 3 / 2 CTAs per SM through memory / in clusters):
    each was the fastest or within 2 % of it.  (pairs, table passes, passes with keys, head size) ->
    (keys per split, splits, through memory)."""
    plan = kernels._decode_split_plan
    measured = {
        (128, 16, 16, 64): (512, 4, True),        # 64 requests x 2,048 keys: 13.5 us
        (128, 64, 64, 64): (1664, 5, True),       # x 8,192: 48.6 us, 5.5 TB/s
        (128, 256, 256, 64): (2048, 16, True),    # x 32,768: 167 us, 6.4 TB/s
        (16, 256, 256, 64): (768, 43, True),      # 8 requests x 32,768: 30.5 us
        (16, 8, 5, 64): (128, 8, False),          # 8 requests x 600 keys in tables of 1,024: a cluster of 8
        (2, 8, 5, 64): (128, 8, False),
        (256, 16, 16, 128): (256, 8, True),       # 7B heads, 64 requests x 2,048: 56 us
        (256, 64, 64, 128): (1664, 5, True),      # x 8,192: 166 us, 6.5 TB/s
        (32, 256, 256, 128): (2560, 13, True),    # 8 requests x 32,768: 89 us
        (256, 256, 256, 128): (1280, 26, True),   # 64 x 32,768: 639 us, 6.7 TB/s
        (256, 8, 5, 128): (1024, 1, False),       # 64 requests x 600 keys: one CTA per pair, no merge
        (32, 8, 5, 128): (256, 4, False),
    }
    for (pairs, total, live, head_dim), want in measured.items():
        per_sm = (5, 4) if head_dim == 64 else (3, 2)
        assert plan(pairs, total, live, head_dim, 148, *per_sm) == want, (pairs, total, live, head_dim)


def test_plan_follows_the_batch_and_the_context():
    # a small batch with a short context: many short splits (latency)
    assert kernels.decode_split_plan(8, 2, 640, 64)[0] == 128
    # a large batch of wide heads: one CTA per (request, head) takes the whole context, no merge
    assert kernels.decode_split_plan(64, 4, 640, 128) == (640, 1, False)
    # one request with a long context: many splits, merged through memory
    split_keys, splits, through_memory = kernels.decode_split_plan(1, 2, 32768, 64)
    assert through_memory and 16 <= splits <= 128
    # a wide table with short contexts is planned for the contexts
    assert kernels.decode_split_plan(64, 4, 4096, 128, 600) == kernels.decode_split_plan(64, 4, 4096, 128, 640)
    assert kernels.decode_split_plan(64, 4, 4096, 128, 600) != kernels.decode_split_plan(64, 4, 4096, 128, 4096)


def test_attention_plan_keeps_short_contexts_resident():
    """Contexts that fit one CTA's shared memory run the resident kernel, with room in steps of 256
    keys (a captured step is keyed by the room); longer ones, other head sizes and other page sizes
    are divided among CTAs."""
    plan = kernels.decode_attention_plan
    assert plan(64, 14, 2, 64, 16, 1024, 520) == ("resident", 768)
    assert plan(64, 14, 2, 64, 16, 1024, 512) == ("resident", 512)
    assert plan(64, 14, 2, 64, 16, 1024, 100) == ("resident", 256)
    assert plan(32, 28, 4, 128, 16, 4096, 300) == ("resident", 384)          # the room's limit at head size 128
    assert plan(64, 28, 4, 128, 16, 4096, 300)[0] == "split"                 # head size 128: more of them than SMs
    assert plan(8, 14, 2, 64, 16, 1024, 520)[0] == "split"                   # too few CTAs to keep the SMs' copies busy
    assert plan(256, 14, 2, 64, 16, 1024, 520)[0] == "split"                 # more CTAs than fit the SMs at once
    assert plan(64, 14, 2, 64, 16, 1024, 769)[0] == "split"
    assert plan(64, 14, 2, 64, 16, 4096)[0] == "split"                       # no context given: the tables' width counts
    assert plan(64, 4, 2, 32, 16, 256, 100)[0] == "split"                    # head size 32
    assert plan(64, 14, 2, 64, 24, 240, 100)[0] == "split"                   # pages of 24 tokens
    assert plan(64, 14, 2, 64, 16, 1024, 769)[1:] == kernels.decode_split_plan(64, 2, 1024, 64, 769)


def test_captured_decode_steps_are_keyed_by_the_parts_plans(monkeypatch):
    """A graph is reused while the parts lay their launches out alike, and only then."""
    from types import SimpleNamespace
    from sprout_lm_b200.engine import graphs

    made = []

    class FakeGraph:
        def __init__(self, runner, requests, table_pages, planned_context=0):
            made.append((requests, table_pages, planned_context))

    monkeypatch.setattr(graphs, "DecodeGraph", FakeGraph)
    asked = []

    def decode_plan(requests, max_keys, planned, page_tokens):
        asked.append((requests, max_keys, planned))
        return ("short",) if planned <= 256 else ("long",)

    runner = SimpleNamespace(page_tokens=16, model=SimpleNamespace(decode_plan=decode_plan))
    cache = graphs.GraphCache(runner, page_multiple=64)
    entry = lambda length: SimpleNamespace(seq=SimpleNamespace(length=length, tables=[[0] * (-(-(length + 1) // 16))]))
    first = cache.get([entry(100), entry(40)])
    assert cache.get([entry(101), entry(41)]) is first            # same plan: same graph
    assert asked[0] == (2, 1024, 128) and asked[1] == (2, 1024, 128)
    assert cache.get([entry(200), entry(41)]) is first            # planned for 256 keys: still the short plan
    other = cache.get([entry(300), entry(41)])
    assert other is not first and made == [(2, 64, 128), (2, 64, 384)]
    assert cache.get([entry(100), entry(40), entry(7)]) is not first      # another number of requests
    assert cache.get([entry(1030), entry(40)]) not in (first, other)      # a wider table


def test_captured_decode_steps_are_bounded(monkeypatch):
    """A serving loop with changing batch sizes and growing contexts asks for ever new keys: the
    cache keeps at most ``limit`` captures and drops the least recently used one."""
    from types import SimpleNamespace
    from sprout_lm_b200.engine import graphs

    alive = []

    class FakeGraph:
        def __init__(self, runner, requests, table_pages, planned_context=0):
            self.key = (requests, table_pages, planned_context)
            alive.append(self.key)

        def __del__(self):
            alive.remove(self.key)

    monkeypatch.setattr(graphs, "DecodeGraph", FakeGraph)
    runner = SimpleNamespace(page_tokens=16, model=SimpleNamespace(decode_plan=lambda requests, max_keys, planned, page_tokens: (planned // 128,)))
    cache = graphs.GraphCache(runner, page_multiple=64, limit=5)
    entry = lambda length: SimpleNamespace(seq=SimpleNamespace(length=length, tables=[[0] * (-(-(length + 1) // 16))]))
    for batch in range(1, 65):
        for length in (50, 300, 700, 1500):
            cache.get([entry(length)] * batch)
            assert len(cache.graphs) <= 5 and len(alive) <= 5
    assert cache.keys_used == 64 * 4 and cache.evictions == 64 * 4 - 5
    # a budget of bytes bounds it as well: captures of 10 units each, room for 35
    class SizedGraph(FakeGraph):
        nbytes = 10
    monkeypatch.setattr(graphs, "DecodeGraph", SizedGraph)
    sized = graphs.GraphCache(runner, page_multiple=64, limit=100, budget_bytes=35)
    for batch in range(1, 10):
        sized.get([entry(50)] * batch)
        assert sized.held_bytes() <= 35 and len(sized.graphs) <= 3
    assert sized.evictions == 6
    del sized
    # use keeps a capture: the one touched again outlives newer ones
    kept = cache.get([entry(50)] * 64)
    for length in (300, 700, 1500, 2100):
        cache.get([entry(length)] * 3)
        assert cache.get([entry(50)] * 64) is kept
    assert len(cache.graphs) == 5


def test_prefill_step_captures_do_not_take_turns_evicting_one_another(monkeypatch):
    """Six step shapes coming round and round with room for four captures: four are captured once
    and replayed from then on; the other two run eagerly instead of capturing over them."""
    import contextlib
    from types import SimpleNamespace
    from sprout_lm_b200.engine import graphs

    captures = []

    class FakeCudaGraph:
        def replay(self):
            pass

    monkeypatch.setattr(graphs.torch.cuda, "CUDAGraph", FakeCudaGraph)
    monkeypatch.setattr(graphs, "guarded_capture", lambda graph: contextlib.nullcontext())
    runner = SimpleNamespace(stager=SimpleNamespace(device_buffer=object()), forward=lambda ctx: None)
    steps = graphs.StepGraphs(runner, limit=4, after=3)
    original = steps._forward
    eager = []

    def forward(ctx, sample):
        eager.append(ctx)
        return original(ctx, sample)

    steps._forward = forward
    for round_ in range(30):
        for shape in range(6):
            before = len(steps.captured)
            steps.run(("shape", shape), shape, False)
            if len(steps.captured) > before:
                captures.append(shape)
    assert sorted(captures) == [0, 1, 2, 3]                     # each captured once, nothing captured over
    assert steps.replays == 4 * (30 - 3)
    # a shape that comes far more often than a captured one does take its place
    for _ in range(200):
        steps.run(("shape", 5), 5, False)
    assert ("shape", 5) in steps.captured and len(steps.captured) == 4


def test_small_batch_kernels_say_what_they_take():
    """The small-batch kernels' size rules are host arithmetic in the kernel library: up to 16 tokens,
    sizes in steps of 16, and a layer small enough for the SMs' shared memory.  What they refuse
    runs on the tensor-core products (the parts ask before they choose)."""
    # the 0.5B layer sizes and the tests' tiny ones fit
    for hidden, inter in [(896, 4864), (64, 128), (96, 320), (1024, 2816)]:
        assert kernels.ffn_decode_supported(8, hidden, inter) and kernels.ffn_decode_supported(1, hidden, inter)
        assert kernels.ffn_decode_supported(9, hidden, inter) and kernels.ffn_decode_supported(16, hidden, inter)
    assert kernels.linear_decode_supported(8, 1152, 896) and kernels.linear_decode_supported(3, 896, 896)
    assert kernels.linear_decode_supported(16, 1152, 896) and kernels.linear_decode_supported(9, 896, 896)
    # more tokens than the instruction has columns, sizes off the 16-step, layers too large
    assert not kernels.ffn_decode_supported(17, 896, 4864)
    assert not kernels.ffn_decode_supported(8, 904, 4864) and not kernels.ffn_decode_supported(8, 896, 4872)
    assert not kernels.ffn_decode_supported(8, 3584, 18944) and not kernels.ffn_decode_supported(8, 5120, 13824)
    assert not kernels.linear_decode_supported(17, 896, 896) and not kernels.linear_decode_supported(8, 900, 896)
    assert not kernels.linear_decode_supported(8, 3584, 3584)


def _share(n, part, parts):
    return n * part // parts


SMEM_LIMIT = 227 * 1024


@pytest.mark.parametrize("ctas,cluster", [(148, 1), (148, 2), (148, 4), (144, 8), (132, 4), (40, 8)])
def test_feed_forward_plan_covers_the_matrices_and_fits(ctas, cluster):
    """The launch layout of the one-kernel feed-forward for many sizes (host arithmetic of the kernel
    library): every gate/up tile has exactly one CTA; the activation columns a cluster produces are
    the K range its CTAs work on, and those CTAs share the down matrix's rows; the TMA boxes respect
    their limits (256 rows, starts on 1024 bytes, columns in steps of 8 elements); what shares a
    room fits in it, and the whole fits the SM's shared memory; sizes it cannot lay out are refused."""
    taken = 0
    for hidden in list(range(16, 513, 48)) + [896, 1024, 1536, 2048]:
        for inter in [16, 128, 320, 1008, 2816, 4864, 8192]:
            p = kernels.small_batch_plan("ffn", 8, hidden, inter, ctas, cluster)
            if p is None:
                continue
            taken += 1
            assert p["ctas"] == ctas and p["cluster"] == cluster and ctas % cluster == 0
            assert p["tiles1"] * 8 == inter and p["tiles2"] * 16 == hidden
            # gate/up: contiguous shares of base or base + 1 tiles
            shares = [_share(p["tiles1"], c + 1, ctas) - _share(p["tiles1"], c, ctas) for c in range(ctas)]
            assert sum(shares) == p["tiles1"] and set(shares) <= {p["base_tiles1"], p["base_tiles1"] + 1}
            assert max(shares) == p["max_tiles1"] <= 8 and p["base_tiles1"] * 16 <= 256
            assert p["boxes1"] * 64 >= hidden and p["box1_bytes"] == p["max_tiles1"] * 2048
            # down: a cluster's K range is what its CTAs produce; its ranks share the rows
            ranges = [sum(shares[c:c + cluster]) for c in range(0, ctas, cluster)]
            assert sum(ranges) == p["tiles1"] and max(ranges) == p["max_ktiles"]
            assert p["max_ksteps"] * 2 >= p["max_ktiles"] and p["col_boxes2"] * 4 >= p["max_ksteps"]
            rows = [_share(p["tiles2"], r + 1, cluster) - _share(p["tiles2"], r, cluster) for r in range(cluster)]
            assert sum(rows) == p["tiles2"] and max(rows) == p["max_tiles2"]
            assert p["box_rows2"] % 16 == 0 and p["box_rows2"] <= 256 and p["box_rows2"] * p["row_boxes2"] >= p["max_tiles2"] * 16
            assert p["box2_bytes"] == p["box_rows2"] * 128
            # rooms: the down rows where the gate/up tiles were; the operand rows; the exchanged activation
            weights = p["off_act"] - p["off_w2"]
            assert p["off_w2"] == 0 and weights >= p["boxes1"] * p["box1_bytes"]
            assert weights >= p["row_boxes2"] * p["col_boxes2"] * p["box2_bytes"]
            assert p["stride1"] == 2 * hidden + 16 and p["off_xchg"] - p["off_act"] >= 8 * p["stride1"]
            assert p["stride_x"] == p["max_ksteps"] * 32 + 16 and p["off_bar"] - p["off_xchg"] >= 8 * p["stride_x"]
            assert p["box1_bytes"] % 1024 == 0 and p["box2_bytes"] % 1024 == 0 and p["off_act"] % 16 == 0
            assert p["off_xchg"] % 16 == 0 and p["off_bar"] % 8 == 0
            assert p["smem_bytes"] >= p["off_bar"] + 16 + 1023 and p["smem_bytes"] <= SMEM_LIMIT - 1024
            assert p["boxes1"] * p["max_tiles1"] * 2048 < (1 << 20) and p["row_boxes2"] * p["col_boxes2"] * p["box2_bytes"] < (1 << 20)   # an mbarrier's byte count
    assert taken >= 20
    assert kernels.small_batch_plan("ffn", 8, 896, 4864, ctas, cluster) is not None or ctas < 100
    assert kernels.small_batch_plan("ffn", 8, 896, 4864, 148, 3) is None and kernels.small_batch_plan("ffn", 8, 896, 4864, 150, 4) is None


@pytest.mark.parametrize("ctas", [148, 132, 40])
def test_linear_plan_covers_the_matrix_and_fits(ctas):
    taken = 0
    for n in [16, 48, 128, 160, 896, 1152, 2048, 4096]:
        for k in [16, 64, 96, 896, 1536, 4864]:
            p = kernels.small_batch_plan("linear", 8, n, k, ctas)
            if p is None:
                continue
            taken += 1
            assert p["tiles"] * 16 == n and p["ksteps"] * 16 == k
            assert 1 <= p["row_groups"] <= p["tiles"] and 1 <= p["k_splits"] <= p["ksteps"] and p["row_groups"] * p["k_splits"] <= ctas
            rows = [_share(p["tiles"], g + 1, p["row_groups"]) - _share(p["tiles"], g, p["row_groups"]) for g in range(p["row_groups"])]
            steps = [_share(p["ksteps"], s + 1, p["k_splits"]) - _share(p["ksteps"], s, p["k_splits"]) for s in range(p["k_splits"])]
            assert sum(rows) == p["tiles"] and sum(steps) == p["ksteps"] and min(rows) >= 1 and min(steps) >= 1
            assert max(rows) == p["max_tiles"] <= 16 and max(steps) == p["max_ksteps"]
            assert p["boxes"] * 4 >= p["max_ksteps"] and p["box_bytes"] == p["max_tiles"] * 2048
            assert p["off_act"] >= p["boxes"] * p["box_bytes"]
            assert p["off_gain"] - p["off_act"] >= 8 * (p["max_ksteps"] * 32 + 16)
            assert p["off_stage"] - p["off_gain"] >= p["max_ksteps"] * 64 and p["off_bar"] - p["off_stage"] >= 8 * p["max_ksteps"] * 64
            assert p["off_act"] % 16 == 0 and p["off_gain"] % 16 == 0 and p["off_stage"] % 16 == 0 and p["off_bar"] % 8 == 0
            assert p["off_bar"] + 16 + 1023 <= p["smem_bytes"] <= 96 * 1024
    assert taken >= 20
    if ctas == 148:
        # the eight warps of a CTA share its tiles: a piece is eight tiles high and a few K steps long,
        # not one tile with many steps (q/k/v and output projection of the 0.5B sizes)
        qkv, o = kernels.small_batch_plan("linear", 8, 1152, 896), kernels.small_batch_plan("linear", 8, 896, 896)
        assert (qkv["row_groups"], qkv["k_splits"], qkv["max_tiles"], qkv["max_ksteps"]) == (9, 16, 8, 4)
        assert (o["row_groups"], o["k_splits"], o["max_tiles"], o["max_ksteps"]) == (7, 21, 8, 3)
