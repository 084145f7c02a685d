"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; windowed groups give pages back early; slots."""
import random

import pytest

from tiny_llm_infer_b200.cache import CacheError, CacheManager, OutOfPages, OutOfSlots, PagePool
from tiny_llm_infer_b200.parts.spec import CacheSpec, StateSpec

FULL = {0: (CacheSpec.keys_and_values(2, 16, None), None), 1: (CacheSpec.keys_and_values(2, 16, None), None)}
MIXED = {0: (CacheSpec.keys_and_values(2, 16, 24), None), 1: (CacheSpec.keys_and_values(2, 16, None), None), 2: (CacheSpec.keys_and_values(2, 16, 24), None)}


def test_pool_lowest_first_and_double_free():
    p = PagePool(4)
    assert [p.alloc() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(2)
    p.free(0)
    assert p.alloc() == 0 and p.alloc() == 2
    p.free(1)
    with pytest.raises(CacheError):
        p.free(1)
    with pytest.raises(CacheError):
        p.free(17)
    p.audit()


def test_reserve_commit_release_and_reuse():
    m = CacheManager(FULL, page_size=8, num_pages=6, max_slots=3, max_seq_len=64)
    assert list(m.groups) == [None] and m.groups[None].cache_ids == [0, 1]
    s = m.admit("a")
    assert s == 0 and m.pages_needed("a", 17) == {None: 3}
    m.reserve("a", 17)
    assert m.pages_of("a") == {None: [0, 1, 2]}
    m.reserve("a", 20)                                   # same pages cover it
    assert m.free_pages() == {None: 3}
    m.commit("a", 17)
    with pytest.raises(CacheError):
        m.commit("a", 40)                                # more than was reserved
    m.admit("b")
    assert not m.can_reserve("b", 33) and m.can_reserve("b", 24)
    with pytest.raises(OutOfPages):
        m.reserve("b", 33)
    assert m.pages_of("b") == {None: []}                 # a failed reserve changes nothing
    m.reserve("b", 24)
    m.release("a")
    m.admit("c")
    m.reserve("c", 9)
    assert m.pages_of("c") == {None: [0, 1]}             # a's pages, used again
    assert m.slot_of("c") == 0                           # and its slot
    m.audit()
    assert not m.can_reserve("c", 65)                    # beyond max_seq_len
    with pytest.raises(CacheError):
        m.admit("c")


def test_slots_run_out():
    m = CacheManager(FULL, 8, 6, max_slots=2, max_seq_len=64)
    m.admit(1), m.admit(2)
    with pytest.raises(OutOfSlots):
        m.admit(3)
    m.release(1)
    assert m.admit(3) == 0


def test_window_group_gives_pages_back_early():
    m = CacheManager(MIXED, page_size=8, num_pages=16, max_slots=2, max_seq_len=128)
    assert set(m.groups) == {24, None} and m.groups[24].cache_ids == [0, 2]
    m.admit("a")
    m.reserve("a", 80)                                   # a whole prompt in one step: all pages needed
    assert m.free_pages() == {24: 6, None: 6}
    m.commit("a", 80)
    # the next query (position 80) reads keys 57..80 in the windowed group: pages 0..6 are dead
    assert m.free_pages() == {24: 13, None: 6}
    assert m.groups[24].table[0, :8].tolist()[:7] == [-1] * 7
    for n in range(81, 100):
        m.reserve("a", n)
        m.commit("a", n)
        m.audit()
        held = len(m.pages_of("a")[24])
        assert held <= 4                                 # window 24 over pages of 8
    m.release("a")
    assert m.free_pages() == {24: 16, None: 16}
    m.audit()


@pytest.mark.parametrize("needs", [FULL, MIXED])
@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_invariant(needs, seed):
    rng = random.Random(seed)
    m = CacheManager(needs, page_size=4, num_pages=40, max_slots=5, max_seq_len=96)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            new_len = min(96, live[rid] + rng.choice([1, 1, 1, 2, 7, 30]))
            if new_len > live[rid]:
                if m.can_reserve(rid, new_len):
                    m.reserve(rid, new_len)
                    m.commit(rid, new_len)
                    live[rid] = new_len
                    for key, pages in m.pages_of(rid).items():
                        first_needed = 0 if key is None else max(0, new_len - key + 1) // 4
                        assert len(pages) == -(-new_len // 4) - first_needed
                else:
                    with pytest.raises(OutOfPages):
                        m.reserve(rid, new_len)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.audit()
    for rid in list(live):
        m.release(rid)
    m.audit()
    assert all(v == 40 for v in m.free_pages().values()) and m.free_slots == 5


def test_state_slots_are_zeroed_at_admission():
    import torch
    needs = {0: (None, StateSpec((3, 2), "float32")), 1: (CacheSpec.keys_and_values(1, 16, None), None)}
    m = CacheManager(needs, 8, 4, max_slots=2, max_seq_len=32, dtype=torch.float32, device="cpu")
    assert m.state[0].shape == (2, 3, 2) and m.kv[1].shape == (4, 2, 1, 8, 16)
    slot = m.admit("a")
    m.view(0).state[slot] += 5
    m.release("a")
    assert m.admit("b") == slot and float(m.view(0).state[slot].abs().sum()) == 0.0
    assert m.view(0).kv is None and m.view(1).state is None


# ---------------------------------------------------------------------------- prefix cache
def prefix_manager(pages=12, slots=4, page=4):
    return CacheManager(FULL, page_size=page, num_pages=pages, max_slots=slots, max_seq_len=64, prefix_cache=True)


def run_request(m, rid, tokens):
    """Admit with the tokens, compute what is not shared in one step; returns what was shared."""
    m.admit(rid, tokens)
    shared = m.computed(rid)
    m.reserve(rid, len(tokens))
    m.commit(rid, len(tokens), tokens[shared:])
    m.audit()
    return shared


def test_prefix_pages_are_shared_counted_and_freed_by_the_last_user():
    m = prefix_manager()
    a = list(range(100, 111))                       # 11 tokens: two full pages and a part
    assert run_request(m, "a", a) == 0              # nothing to share yet
    b = a[:9] + [7, 7, 7]
    assert run_request(m, "b", b) == 8              # both full pages of the common beginning
    pa, pb = m.pages_of("a")[None], m.pages_of("b")[None]
    assert pa[:2] == pb[:2] and pa[2] != pb[2]
    assert m.free_pages() == {None: 12 - 4}
    c = a[:8]                                       # ends on a page edge: its last page is computed
    assert run_request(m, "c", c) == 4
    assert m.pages_of("c")[None][0] == pa[0] and m.pages_of("c")[None][1] not in pa + pb
    m.release("a")
    assert m.free_pages() == {None: 12 - 5 + 1}     # only a's own third page came back
    m.release("b")
    m.release("c")
    m.audit()
    assert m.free_pages() == {None: 12}
    # freed pages keep their hash until they are handed out again: the prompt comes back for free
    assert run_request(m, "d", a) == 8
    assert m.pages_of("d")[None][:2] == pa[:2]
    assert m.prefix_hit_pages == 2 + 1 + 2


def test_prefix_differs_in_the_first_page_or_in_tokens_behind_an_equal_page():
    m = prefix_manager(pages=16)
    a = list(range(20))
    run_request(m, "a", a)
    assert run_request(m, "b", [99] + a[1:]) == 0           # a later page alone never matches: the chain differs
    assert run_request(m, "c", a[:4] + [98] + a[5:]) == 4
    m.audit()


def test_prefix_hash_is_dropped_when_the_page_is_handed_out_again():
    """Freed pages that the prefix cache still knows are handed out last, the one freed
    longest ago first; a page that is handed out again no longer stands for its old tokens."""
    m = prefix_manager(pages=4)
    a = list(range(13))                                     # pages 0-2 full (hashed), page 3 part
    run_request(m, "a", a)
    m.release("a")                                          # freed in the order 3, 2, 1, 0
    other = list(range(50, 59))
    assert run_request(m, "x", other) == 0
    assert m.pages_of("x")[None] == [3, 2, 1]               # the unhashed page first, then the oldest
    m.release("x")
    assert run_request(m, "b", a) == 4                      # page 0 still holds a's beginning
    assert m.pages_of("b")[None][0] == 0
    m.release("b")
    assert run_request(m, "c", list(range(70, 83))) == 0    # takes all four pages
    m.release("c")
    assert run_request(m, "d", a) == 0 and m.computed("d") == 13
    m.audit()


def test_prefix_needs_tokens_and_full_caches_without_state():
    m = prefix_manager()
    m.admit("a")                                            # no tokens told: never hashed, never shares
    m.reserve("a", 9)
    m.commit("a", 9)
    assert run_request(m, "b", list(range(9))) == 0
    m.admit("c", list(range(30, 39)))
    m.reserve("c", 9)
    m.commit("c", 5)                                        # tokens not told for this step: hashing stops
    m.commit("c", 9, list(range(35, 39)))
    assert run_request(m, "d", list(range(30, 39))) == 0
    assert not CacheManager(MIXED, 4, 8, 2, 64, prefix_cache=True).prefix_active
    with_state = {0: (CacheSpec.keys_and_values(2, 16, None), StateSpec((3,), "float32"))}
    assert not CacheManager(with_state, 4, 8, 2, 64, prefix_cache=True).prefix_active


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_with_shared_prefixes_keep_every_invariant(seed):
    rng = random.Random(100 + seed)
    m = CacheManager(FULL, page_size=4, num_pages=30, max_slots=5, max_seq_len=64, prefix_cache=True)
    stems = [[rng.randrange(50) for _ in range(40)] for _ in range(3)]
    live, next_id, shared_total = {}, 0, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.3 and m.free_slots:
            stem = rng.choice(stems)
            cut = rng.randrange(1, 40)
            tokens = stem[:cut] + [rng.randrange(50, 60) for _ in range(rng.randrange(0, 9))]
            m.admit(next_id, tokens)
            done = m.computed(next_id)
            assert done % 4 == 0 and done < len(tokens)
            # what is shared holds the request's own tokens
            for i, page in enumerate(m.pages_of(next_id)[None]):
                assert m.groups[None].tokens_of[page] == tuple(tokens[4 * i:4 * i + 4])
            shared_total += done
            live[next_id] = (tokens, done)
            next_id += 1
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            tokens, done = live[rid]
            if done == len(tokens):
                tokens = tokens + [rng.randrange(60)]           # decoding
            new_len = min(len(tokens), done + rng.choice([1, 2, 5, 16]))
            if m.can_reserve(rid, new_len):
                m.reserve(rid, new_len)
                m.commit(rid, new_len, tokens[done:new_len])
                live[rid] = (tokens, new_len)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.audit()
    for rid in list(live):
        m.release(rid)
    m.audit()
    assert m.free_pages() == {None: 30} and m.free_slots == 5 and shared_total > 0


def test_try_reserve_is_reserve_or_nothing():
    m = CacheManager(MIXED, page_size=4, num_pages=3, max_slots=2, max_seq_len=64)
    m.admit("a")
    assert m.try_reserve("a", 9) and m.pages_of("a")[None] == [0, 1, 2]
    assert m.try_reserve("a", 12)                       # the pages are there already
    before = m.free_pages()
    assert not m.try_reserve("a", 13) and m.free_pages() == before and m.pages_of("a")[None] == [0, 1, 2]
    assert not m.try_reserve("a", 65)                   # beyond the longest sequence
    m.commit("a", 12)
    m.audit()


def test_a_page_with_a_token_still_to_be_told_waits_for_its_hash():
    """commit() with a negative token (computed on the device, not yet known on the host): the
    page is not hashed, so nobody can share it; fill_token() tells it, and the chain goes on
    through every page that was waiting behind it."""
    cm = prefix_manager(pages=16)
    stem = [5, 6, 7, 8, 9, 10, 11]
    cm.admit("a", stem)
    cm.reserve("a", 7)
    cm.commit("a", 7, stem)                               # one full page hashed, three tokens of the next
    cm.reserve("a", 9)
    cm.commit("a", 9, [-1, 13])                           # position 7 unknown: page 1 is full but waits
    cm.admit("b", stem + [12, 13, 1])
    assert cm.computed("b") == 4                          # only page 0 is found
    cm.release("b")
    cm.reserve("a", 12)
    cm.commit("a", 12, [14, 15, 16])                      # page 2 is full too, behind the waiting one
    cm.fill_token("a", 7, 12)
    cm.admit("c", stem + [12, 13, 14, 15, 16, 2])
    assert cm.computed("c") == 12                         # pages 0, 1 and 2
    cm.fill_token("a", 7, 99)                             # told once: a second telling changes nothing
    cm.fill_token("gone", 0, 1)                           # nor does one for a request that is not there
    cm.audit()
    for r in ("a", "c"):
        cm.release(r)
    cm.audit()
    assert cm.free_pages() == {None: 16}
