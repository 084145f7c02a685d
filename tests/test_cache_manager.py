"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; windowed groups give pages back early; slots."""
import random

import pytest

from tiny_llm_infer_b200.cache import CacheError, CacheManager, OutOfPages, OutOfSlots, PagePool
from tiny_llm_infer_b200.parts.spec import CacheSpec, StateSpec

FULL = {0: (CacheSpec(2, 16, None), None), 1: (CacheSpec(2, 16, None), None)}
MIXED = {0: (CacheSpec(2, 16, 24), None), 1: (CacheSpec(2, 16, None), None), 2: (CacheSpec(2, 16, 24), None)}


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
    needs = {0: (None, StateSpec((3, 2), "float32")), 1: (CacheSpec(1, 16, None), None)}
    m = CacheManager(needs, 8, 4, max_slots=2, max_seq_len=32, dtype=torch.float32, device="cpu")
    assert m.state[0].shape == (2, 3, 2) and m.kv[1].shape == (4, 2, 1, 8, 16)
    slot = m.admit("a")
    m.view(0).state[slot] += 5
    m.release("a")
    assert m.admit("b") == slot and float(m.view(0).state[slot].abs().sum()) == 0.0
    assert m.view(0).kv is None and m.view(1).state is None
