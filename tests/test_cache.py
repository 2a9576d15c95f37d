"""The cache manager: page states, prefix hits, windows, and that under random orders of
requests no page is lost, held twice or freed twice."""

from __future__ import annotations

import random

import pytest

from mercury_b200.cache import CacheManager, OutOfPages, PagePool, extend_hashes, page_hashes


# ------------------------------------------------------------------------------ hashing

def test_only_full_pages_are_hashed_and_the_chain_sees_everything_before():
    tokens = list(range(40))
    assert len(page_hashes(tokens, 16)) == 2
    assert len(page_hashes(tokens[:15], 16)) == 0
    changed = [99] + tokens[1:]
    a, b = page_hashes(tokens, 16), page_hashes(changed, 16)
    assert a[0] != b[0] and a[1] != b[1]
    assert page_hashes(tokens, 16, cryptographic=True) != a


def test_extending_equals_recomputing():
    tokens = [random.Random(1).randrange(1000) for _ in range(100)]
    grown: list[int] = []
    for n in (5, 16, 17, 48, 100):
        extend_hashes(grown, tokens[:n], 16)
        assert grown == page_hashes(tokens[:n], 16)


# ------------------------------------------------------------------------------ the pool

def test_pool_states_and_lru():
    pool = PagePool(4, 16)
    pages = [pool.take() for _ in range(4)]
    assert pool.take() is None and pool.num_available() == 0
    pool.commit(pages[0], 111)
    pool.commit(pages[1], 222)
    pool.commit(pages[2], 111)                       # duplicate content stays private
    assert pool.hash_of[pages[2]] is None
    pool.release(pages[1])
    pool.release(pages[0])
    pool.release(pages[3])
    pool.check_invariants()
    assert pool.take() == pages[3]                   # free pages before cached ones
    assert pool.take() == pages[1]                   # then the least recently released
    assert pool.lookup(222) is None and pool.lookup(111) == pages[0]
    assert pool.evictions == 1
    pool.hold(pages[0])
    assert pool.ref[pages[0]] == 1 and pool.num_available() == 0
    pool.check_invariants()


def test_double_free_is_caught():
    pool = PagePool(2, 16)
    page = pool.take()
    pool.release(page)
    with pytest.raises(AssertionError, match="twice"):
        pool.release(page)


# ------------------------------------------------------------------------------ the manager

def finish_prompt(cache, seq, tokens):
    cache.advance(seq, len(tokens), page_hashes(tokens, cache.page_size))


def test_a_hit_always_leaves_a_token_to_compute():
    cache = CacheManager([0], 16, 16, 4)
    tokens = list(range(32))
    a = cache.open("a")
    assert cache.admit(a, page_hashes(tokens, 16), 32) and a.num_computed == 0
    finish_prompt(cache, a, tokens)
    cache.close(a)
    b = cache.open("b")
    assert cache.admit(b, page_hashes(tokens, 16), 32)
    assert b.num_computed == 16                       # not 32: the last token must run
    c = cache.open("c")
    assert cache.admit(c, page_hashes(tokens + [7], 16), 33) and c.num_computed == 32
    assert c.tables[0][:1] == b.tables[0][:1]         # the shared head is the same page
    cache.check_invariants()


def test_failed_admission_changes_nothing():
    cache = CacheManager([0], 4, 16, 4)
    a = cache.open("a")
    assert cache.admit(a, [], 48)
    b = cache.open("b")
    before = cache.num_available()
    assert not cache.admit(b, [], 32)
    assert cache.num_available() == before and b.tables == [[]]
    cache.close(b)
    cache.check_invariants()


def test_hits_are_pinned_before_new_pages_are_taken():
    cache = CacheManager([0], 3, 16, 4)
    tokens = list(range(33))
    a = cache.open("a")
    cache.admit(a, page_hashes(tokens, 16), 33)
    finish_prompt(cache, a, tokens)
    cache.close(a)                                    # 2 cached pages + 1 free
    b = cache.open("b")
    # needs 3 pages, 2 of them cached hits: only 1 new page may be taken, and it must not
    # evict the hits
    assert cache.admit(b, page_hashes(tokens, 16), 33) and b.num_computed == 32
    cache.check_invariants()


def test_window_group_gives_pages_back_and_full_group_keeps_them():
    cache = CacheManager([0, 24], 16, 16, 2)
    s = cache.open("s")
    assert cache.ensure(s, 100)
    cache.advance(s, 100)
    assert all(p >= 0 for p in s.tables[0])
    # next query at 100 sees keys > 76: pages 0..3 (positions < 64) are behind the window
    assert s.tables[1][:4] == [-1] * 4 and all(p >= 0 for p in s.tables[1][4:])
    assert cache.num_available() == [16 - 7, 16 - 3]
    cache.close(s)
    assert cache.num_available() == [16, 16]
    cache.check_invariants()


def test_slots_run_out_and_come_back():
    cache = CacheManager([0], 8, 16, 2)
    a, b = cache.open("a"), cache.open("b")
    assert a.slot != b.slot and not cache.has_slot()
    with pytest.raises(OutOfPages):
        cache.open("c")
    cache.close(a)
    assert cache.open("c").slot == a.slot
    with pytest.raises(AssertionError):
        cache.close(a)


@pytest.mark.parametrize("windows", [[0], [0, 40], [24]])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_orders_keep_every_invariant(windows, seed):
    """Requests arrive, grow by portions and single tokens, share prefixes, finish or are
    dropped half-way, in random order, on a pool too small for all of them."""
    rng = random.Random(seed)
    page = 8
    cache = CacheManager(windows, 40, page, 6)
    prefixes = [[rng.randrange(50) for _ in range(rng.choice((16, 24, 40)))] for _ in range(3)]
    live: dict[str, tuple] = {}
    counter = 0
    for _ in range(1500):
        action = rng.random()
        if action < 0.25 and cache.has_slot():
            tokens = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(rng.randrange(1, 60))]
            seq = cache.open(f"r{counter}")
            counter += 1
            if cache.admit(seq, page_hashes(tokens, page), len(tokens)):
                live[seq.seq_id] = (seq, tokens)
            else:
                cache.close(seq)
        elif action < 0.85 and live:
            seq, tokens = live[rng.choice(list(live))]
            if seq.num_computed < len(tokens):
                upto = min(len(tokens), seq.num_computed + rng.choice((1, 2, 7, 16, 33)))
            else:
                tokens.append(rng.randrange(50))
                upto = len(tokens)
            if cache.ensure(seq, upto):
                cache.advance(seq, upto, page_hashes(tokens[:upto], page))
            else:
                cache.close(seq)                      # preempted
                del live[seq.seq_id]
        elif live:
            seq, _tokens = live.pop(rng.choice(list(live)))
            cache.close(seq)
        cache.check_invariants()
        for seq, _tokens in live.values():
            for group, table in enumerate(seq.tables):
                first = cache._first_needed(group, seq.num_computed)
                assert all(p >= 0 for p in table[first:]), "a page still in sight was given back"
    for seq, _tokens in list(live.values()):
        cache.close(seq)
    cache.check_invariants()
    assert cache.leaked_pages() == 0
    assert cache.num_available() == [40] * len(windows)
