"""The cache manager on the host: pages, block tables, prefix reuse, eviction, windows, state
slots.  Scenarios after the reference's own (test/engine.test.ts:25-43,61-123), plus random
orders of requests with the invariants checked after every operation: no page lost, none held
twice, none freed twice."""
import random

import pytest

from sprout_lm_b200.cache import CacheError, CacheManager, GroupSpec

FULL = [GroupSpec("full", "full", None, (0, 1))]


def fill(manager, seq, tokens):
    for _ in range(tokens):
        assert manager.reserve(seq, seq.length + 1)
        seq.length += 1


def test_lowest_page_first_and_last_freed_first_reused():
    m = CacheManager(FULL, 6, 2)
    seq, blocker = m.create(), m.create()
    assert m.reserve(blocker, 1)                       # physical page 0 is taken
    for p in range(4):
        assert m.reserve(seq, seq.length + 1)
        seq.length += 1
        if p == 1:
            m.release(blocker)                         # the next logical page lands on physical page 0
    assert seq.blocks[:2] == [1, 0]
    m.release(seq)
    assert m.free_pages() == 6
    m.check_invariants()


def test_reserve_is_needed_only_at_page_edges_and_fails_when_empty():
    m = CacheManager(FULL, 2, 4)
    seq = m.create()
    fill(m, seq, 8)
    assert len(seq.blocks) == 2 and m.free_pages() == 0
    assert m.reserve(seq, 8) is True                  # still inside its pages
    assert m.reserve(seq, 9) is False                 # nothing left and nothing to evict
    m.release(seq)
    with pytest.raises(CacheError):
        m.reserve(seq, 1)                             # released
    m.release(seq)                                    # releasing again is a no-op, not a double free
    assert m.free_pages() == 2


def test_double_free_is_caught():
    m = CacheManager(FULL, 2, 4)
    seq = m.create()
    fill(m, seq, 1)
    page = seq.blocks[0]
    m.pools[0].release(page)
    with pytest.raises(CacheError, match="underflow"):
        m.pools[0].release(page)


def test_prefix_reuse_shares_pages_and_leaves_the_last_token():
    m = CacheManager(FULL, 8, 2)
    prompt = [5, 6, 7, 8]                              # exactly two pages
    a = m.create()
    fill(m, a, 4)
    m.publish(prompt, a)
    b = m.reuse_prefix(prompt)
    assert b.length == 2 and b.blocks == a.blocks[:1]  # never the whole prompt: one token is left to compute
    snap = m.snapshot()
    assert snap["pages"][a.blocks[0]]["activeRefs"] == 2 and snap["pages"][a.blocks[0]]["cached"]
    c = m.reuse_prefix(prompt + [9])
    assert c.length == 4 and c.blocks == a.blocks
    for seq in (a, b, c):
        m.release(seq)
    assert all(p["activeRefs"] == 0 for p in m.snapshot()["pages"])
    assert m.snapshot()["cachedPages"] == 2 and m.free_pages() == 6
    m.clear_prefixes()
    assert m.free_pages() == 8
    m.check_invariants()


def test_same_suffix_after_other_context_does_not_hit():
    m = CacheManager(FULL, 8, 2)
    a = m.create()
    fill(m, a, 4)
    m.publish([1, 2, 3, 4], a)
    assert m.reuse_prefix([9, 8, 3, 4, 5]).length == 0
    assert m.reuse_prefix([1, 2, 9, 9, 9]).length == 2
    assert m.reuse_prefix([1, 2, 3, 4, 5]).length == 4


def test_only_prompt_pages_that_are_full_are_published():
    m = CacheManager(FULL, 8, 4)
    a = m.create()
    fill(m, a, 7)
    m.publish([1, 2, 3, 4, 5, 6], a)                   # the prompt covers one full page only
    assert m.snapshot()["cachedPages"] == 1
    fill(m, a, 1)
    m.publish([1, 2, 3, 4, 5, 6], a)
    assert m.snapshot()["cachedPages"] == 1


def test_lru_eviction_spares_pages_with_live_users():
    m = CacheManager(FULL, 3, 2)
    a = m.create()
    fill(m, a, 5)
    m.publish([1, 2, 3, 4, 5], a)
    m.release(a)                                       # two cached pages stay, one page is free
    reused = m.reuse_prefix([1, 2, 9])
    protected = reused.blocks[0]
    other = m.create()
    fill(m, other, 4)                                  # takes the free page, then evicts the unused cached one
    assert m.evictions > 0
    assert m.snapshot()["pages"][protected]["activeRefs"] == 1
    assert protected not in other.blocks
    assert m.reserve(other, other.length + 1) is False
    m.release(other)
    m.release(reused)
    m.clear_prefixes()
    assert m.free_pages() == 3
    m.check_invariants()


def test_prefix_caching_off():
    m = CacheManager(FULL, 4, 2, prefix_caching=False)
    a = m.create()
    fill(m, a, 4)
    m.publish([1, 2, 3, 4], a)
    assert m.snapshot()["cachedPages"] == 0 and m.reuse_prefix([1, 2, 3, 4, 5]).length == 0


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    groups = [GroupSpec("full", "full", None, (0,)), GroupSpec("window6", "window", 6, (1,))]
    m = CacheManager(groups, [8, 3], 4)
    assert not m.prefix_caching                        # reuse would skip positions a window still needs
    seq = m.create()
    for _ in range(20):
        assert m.reserve(seq, seq.length + 1), seq.length
        seq.length += 1
        m.trim(seq)
        m.check_invariants()
    assert len(seq.tables[0]) == 5 and all(p >= 0 for p in seq.tables[0])
    # after 20 tokens the next query (position 20) sees keys 15..19: pages 0..2 are gone, 3 and 4 live
    assert [p >= 0 for p in seq.tables[1]] == [False, False, False, True, True]
    assert m.free_pages(1) == 1 and m.free_pages(0) == 3
    m.release(seq)
    assert m.free_pages(0) == 8 and m.free_pages(1) == 3
    # a window pool smaller than the sequence is enough; a full pool of that size is not
    m2 = CacheManager([GroupSpec("full", "full", None, (0,))], 3, 4)
    s2 = m2.create()
    assert all(m2.reserve(s2, n + 1) for n in range(12)) and not m2.reserve(s2, 13)


def test_state_slots_are_taken_and_given_back():
    m = CacheManager(FULL, 4, 2, state_slots=2)
    assert not m.prefix_caching                        # state is not rebuilt by skipping a prefix
    a, b = m.create(), m.create()
    assert {a.state_slot, b.state_slot} == {0, 1} and not m.can_create()
    with pytest.raises(CacheError, match="state slot"):
        m.create()
    m.release(a)
    c = m.create()
    assert c.state_slot == a.state_slot or c.state_slot in (0, 1)
    assert m.snapshot()["stateSlots"] == {"total": 2, "free": 0}
    m.release(b)
    m.release(c)
    m.check_invariants()
    assert m.snapshot()["stateSlots"]["free"] == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    page_tokens = rng.choice([1, 2, 4])
    m = CacheManager(FULL, rng.randint(4, 12), page_tokens)
    prompts = [[rng.randrange(3) for _ in range(rng.randint(1, 12))] for _ in range(5)]
    live = []
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 6:
            prompt = rng.choice(prompts)
            seq = m.reuse_prefix(prompt)
            live.append((seq, prompt))
        elif action < 0.75 and live:
            seq, prompt = rng.choice(live)
            if m.reserve(seq, seq.length + 1):
                seq.length += 1
                m.publish(prompt, seq)
        elif live:
            seq, _ = live.pop(rng.randrange(len(live)))
            m.release(seq)
        m.check_invariants()
        pool = m.pools[0]
        held = {}
        for seq, _ in live:
            assert len(set(seq.blocks)) == len(seq.blocks)            # no page twice in one table
            assert len(seq.blocks) * page_tokens >= seq.length
            for page in seq.blocks:
                held[page] = held.get(page, 0) + 1
        snap = m.snapshot()
        for page in snap["pages"]:
            assert page["activeRefs"] == held.get(page["id"], 0)       # held exactly as often as tables say
            if page["activeRefs"] > 1:
                assert page["cached"]                                  # only published pages are shared
        assert snap["freePages"] + sum(1 for p in snap["pages"] if p["refs"] > 0) == pool.num_pages
    for seq, _ in live:
        m.release(seq)
    m.clear_prefixes()
    assert m.free_pages() == m.pools[0].num_pages
    m.check_invariants()


@pytest.mark.parametrize("seed", range(4))
def test_prefix_entries_hold_a_page_of_every_group(seed):
    """Two groups that keep every key, with pools of different sizes: a published prefix holds one
    page of each, is found by any of them, and is counted and evicted as one.  Random orders of
    requests; every page of both pools stays accounted for."""
    rng = random.Random(100 + seed)
    page_tokens = rng.choice([2, 4])
    groups = [GroupSpec("a", "full", None, (0,)), GroupSpec("b", "full", None, (1,))]
    sizes = (rng.randint(6, 10), rng.randint(11, 16))
    m = CacheManager(groups, sizes, page_tokens)
    assert m.prefix_caching
    prompts = [[rng.randrange(3) for _ in range(rng.randint(3, 14))] for _ in range(5)]
    live = []
    hits = 0
    for _ in range(500):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            prompt = rng.choice(prompts)
            seq = m.reuse_prefix(prompt)
            hits += seq.length
            live.append((seq, prompt))
        elif action < 0.75 and live:
            seq, prompt = rng.choice(live)
            if m.reserve(seq, seq.length + 1):
                seq.length += 1
                m.publish(prompt, seq)
        elif live:
            seq, _ = live.pop(rng.randrange(len(live)))
            m.release(seq)
        m.check_invariants()
        snap = m.snapshot()
        for group, pool in enumerate(m.pools):
            held = {}
            for seq, _ in live:
                table = seq.tables[group]
                assert len(table) == len(seq.tables[0]) and len(set(table)) == len(table)
                for page in table:
                    held[page] = held.get(page, 0) + 1
            for page in snap["groups"][group]["pages"]:
                assert page["activeRefs"] == held.get(page["id"], 0)
            assert m.available_pages(group) == len(pool.free) + m._cached_only <= pool.num_pages
        assert len(m._entry_of_page) == 2 * len(m._prefixes)
    assert hits > 0 and m.evictions > 0
    for seq, _ in live:
        m.release(seq)
    m.clear_prefixes()
    assert [m.free_pages(g) for g in range(2)] == list(sizes)
    m.check_invariants()


def test_eviction_takes_the_least_recently_used_leaf_and_a_parent_only_after_its_children():
    """Three published chains; pages are asked for until the map has to give way.  The order of
    eviction: least recently used first, and within a chain the last page before the first."""
    manager = CacheManager([GroupSpec("full", "full", None, (0,))], 8, 2)
    chains = {"a": [1, 2, 3, 4], "b": [5, 6], "c": [7, 8, 9, 10]}
    for tokens in chains.values():                      # a: 2 pages, b: 1 page, c: 2 pages
        seq = manager.create()
        for upto in range(2, len(tokens) + 1, 2):
            assert manager.reserve(seq, upto)
        seq.length = len(tokens)
        manager.publish(tokens, seq)
        manager.release(seq)
    assert manager.free_pages() == 3 and manager.available_pages() == 8
    hit = manager.reuse_prefix(chains["a"] + [0])       # a is used again: now the most recent
    assert hit.length == 4
    manager.release(hit)
    manager.check_invariants()
    taker = manager.create()
    for upto in range(2, 7, 2):                         # the three free pages
        assert manager.reserve(taker, upto)
    assert manager.evictions == 0

    def cached(tokens):
        probe = manager.reuse_prefix(tokens + [0])
        length = probe.length
        manager.release(probe)
        return length

    assert manager.reserve(taker, 8) and manager.evictions == 1
    assert cached(chains["b"]) == 0 and cached(chains["c"]) == 4 and cached(chains["a"]) == 4     # b was used least recently
    manager.check_invariants()
    # the probes above made c then a the most recent; c's second page goes before its first
    assert manager.reserve(taker, 10) and manager.evictions == 2
    assert cached(chains["c"]) == 2
    # that probe used c's first page again; the least recently used leaf is now a's second page
    assert manager.reserve(taker, 12) and manager.evictions == 3
    assert cached(chains["a"]) == 2 and cached(chains["c"]) == 2
    manager.check_invariants()
    assert manager.available_pages() == 2
