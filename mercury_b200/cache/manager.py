"""The cache manager: block tables of live sequences over one page pool per layer group,
and slots for per-request state of fixed size.

A *group* is a set of cache layers with the same need: all keys (`window` 0) or the last
`window` keys. Each group has pages of its own (a `PagePool`) and each sequence has one
block table per group; the layers of a group share that table (page p of the group is
row p of every layer's tensor, as in mercury/runner.py:71-79). Pages go back to the pool
when the sequence closes or when a window has passed them, and are used again.

The rules of mercury/allocator.py are kept: a prefix hit always leaves one token to
compute (:64-73), hits are pinned before new pages are taken (:84-90), a failed admission
changes nothing (:78-83), pages are released last-first (:110-121).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence as Seq

from .pages import PagePool


class OutOfPages(RuntimeError):
    """A step was asked to run tokens whose pages could not be provided."""


@dataclass
class Sequence:
    """What one live request holds: a state slot and one block table per group.
    `tables[g][i]` is the page of tokens [i*page_size, (i+1)*page_size), or -1 once the
    group's window has passed it. `num_computed` tokens have keys in the cache."""

    seq_id: str
    slot: int
    tables: list[list[int]]
    num_computed: int = 0
    committed: list[int] = field(default_factory=list)
    closed: bool = False


class CacheManager:
    def __init__(self, group_windows: Seq[int], num_pages: int | Seq[int], page_size: int,
                 num_slots: int):
        if page_size <= 0 or page_size & (page_size - 1):
            raise ValueError("page_size must be a positive power of two")
        self.page_size = page_size
        self.windows = [int(w) for w in group_windows]
        counts = [num_pages] * len(self.windows) if isinstance(num_pages, int) else list(num_pages)
        self.pools = [PagePool(n, page_size) for n in counts]
        self.num_slots = num_slots
        self._free_slots = list(range(num_slots - 1, -1, -1))
        self.fresh_slots: list[int] = []
        self.live: dict[str, Sequence] = {}
        self.stats = {"hit_tokens": 0, "query_tokens": 0, "admissions": 0,
                      "allocation_failures": 0}

    # ------------------------------------------------------------------ sequences

    def has_slot(self) -> bool:
        return bool(self._free_slots)

    def open(self, seq_id: str) -> Sequence:
        if seq_id in self.live:
            raise KeyError(f"sequence {seq_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.num_slots} state slots are taken")
        slot = self._free_slots.pop()
        self.fresh_slots.append(slot)
        seq = Sequence(seq_id, slot, [[] for _ in self.pools], 0, [0] * len(self.pools))
        self.live[seq_id] = seq
        return seq

    def close(self, seq: Sequence) -> None:
        """Give back every page and the slot; hashed pages stay cached."""
        if seq.closed:
            raise AssertionError(f"sequence {seq.seq_id!r} was closed twice")
        for pool, table in zip(self.pools, seq.tables):
            pool.release_all(table)
            table.clear()
        seq.closed = True
        seq.num_computed = 0
        del self.live[seq.seq_id]
        self._free_slots.append(seq.slot)

    # ------------------------------------------------------------------ geometry

    def _first_needed(self, group: int, next_position: int) -> int:
        """Index of the first page that a query at `next_position` can still see."""
        window = self.windows[group]
        if window <= 0:
            return 0
        return max(0, next_position - window + 1) // self.page_size

    def _pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    # ------------------------------------------------------------------ prefix cache

    def _match(self, hashes: Seq[int], limit: int) -> int:
        """The longest n <= limit such that every group still has the pages that a query at
        position n*page_size would read: all n of them in a group that keeps every key, the
        ones inside the window in a windowed group."""
        for group, pool in enumerate(self.pools):
            if self.windows[group] <= 0:
                limit = min(limit, len(pool.cached_prefix(hashes[:limit])))
        for n in range(limit, 0, -1):
            ok = True
            for group, pool in enumerate(self.pools):
                if self.windows[group] <= 0:
                    continue
                first = self._first_needed(group, n * self.page_size)
                if any(pool.lookup(hashes[i]) is None for i in range(first, n)):
                    ok = False
                    break
            if ok:
                return n
        return 0

    def match_prefix(self, hashes: Seq[int], num_tokens: int) -> int:
        """How many leading pages of a prompt of `num_tokens` can be taken from the cache;
        at least one token is always left to compute, or the prompt's last position would
        yield no logits (mercury/allocator.py:64-73)."""
        return self._match(hashes, min(len(hashes), (num_tokens - 1) // self.page_size))

    def cached_prefix_tokens(self, hashes: Seq[int]) -> int:
        """Tokens of a prompt that are cached now: the scheduler's prefix-match score
        (mercury/scheduler.py:113)."""
        return self._match(hashes, len(hashes)) * self.page_size

    def admit(self, seq: Sequence, hashes: Seq[int], num_tokens: int) -> bool:
        """Pages for a whole prompt of `num_tokens`, reusing cached ones; on success
        `seq.num_computed` is the number of tokens already in the cache. False, with
        nothing changed, if some group cannot provide them."""
        if seq.num_computed or any(seq.tables):
            raise AssertionError("admit() wants a sequence that holds nothing")
        hit = self.match_prefix(hashes, num_tokens) if hashes else 0
        total = self._pages_for(num_tokens)
        plans = []
        for group, pool in enumerate(self.pools):
            first = self._first_needed(group, hit * self.page_size) if hit else 0
            reused = [pool.lookup(hashes[i]) for i in range(first, hit)]
            pinned = sum(1 for p in reused if pool.ref[p] == 0)
            need_new = total - hit
            if need_new > pool.num_available() - pinned:
                self.stats["allocation_failures"] += 1
                return False
            plans.append((first, reused, need_new))
        for group, (first, reused, need_new) in enumerate(plans):
            pool = self.pools[group]
            for page in reused:
                pool.hold(page)
            table = [-1] * first + reused + [pool.take() for _ in range(need_new)]
            seq.tables[group] = table
            seq.committed[group] = hit
        seq.num_computed = hit * self.page_size
        self.stats["hit_tokens"] += seq.num_computed
        self.stats["query_tokens"] += num_tokens
        self.stats["admissions"] += 1
        return True

    # ------------------------------------------------------------------ growth

    def pages_short(self, seq: Sequence, length: int) -> list[int]:
        """Per group, how many pages are missing for the tokens up to `length`."""
        total = self._pages_for(length)
        return [max(0, total - len(table)) for table in seq.tables]

    def ensure(self, seq: Sequence, length: int) -> bool:
        """Make pages exist for every position below `length`. All or nothing."""
        short = self.pages_short(seq, length)
        if any(n > pool.num_available() for n, pool in zip(short, self.pools)):
            return False
        for n, pool, table in zip(short, self.pools, seq.tables):
            for _ in range(n):
                table.append(pool.take())
        return True

    def advance(self, seq: Sequence, new_length: int, hashes: Seq[int] | None = None) -> None:
        """After a step stored keys up to `new_length`: make the pages that are now full
        shareable (when their chain hashes are given; mercury/engine.py:232-241) and give
        back the pages that every later query's window has passed."""
        seq.num_computed = new_length
        full = new_length // self.page_size
        for group, pool in enumerate(self.pools):
            table = seq.tables[group]
            if hashes is not None:
                for index in range(seq.committed[group], min(full, len(hashes))):
                    if table[index] >= 0:
                        pool.commit(table[index], hashes[index])
                seq.committed[group] = max(seq.committed[group], min(full, len(hashes)))
            first = self._first_needed(group, new_length)
            for index in range(min(first, len(table)) - 1, -1, -1):
                if table[index] < 0:
                    break
                pool.release(table[index])
                table[index] = -1

    # ------------------------------------------------------------------ debugging

    def keep_journal(self) -> None:
        """From now on note every page that gets a first holder or goes back unhashed."""
        for pool in self.pools:
            if pool.journal is None:
                pool.journal = []

    def drain_journal(self) -> list[list[int]]:
        """Per group, the pages noted since the last call (each once)."""
        out = []
        for pool in self.pools:
            noted, pool.journal = pool.journal or [], ([] if pool.journal is not None else None)
            out.append(sorted({page for _what, page in noted}))
        return out

    # ------------------------------------------------------------------ checks

    def num_available(self) -> list[int]:
        return [pool.num_available() for pool in self.pools]

    def leaked_pages(self) -> int:
        """Pages held although no sequence is live."""
        return 0 if self.live else sum(pool.num_held() for pool in self.pools)

    def check_invariants(self) -> None:
        """No page lost, held twice without a hash, or freed twice; every live sequence's
        pages are held; slots are unique."""
        for pool in self.pools:
            pool.check_invariants()
        for group, pool in enumerate(self.pools):
            holders: dict[int, int] = {}
            for seq in self.live.values():
                seen = set()
                for page in seq.tables[group]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise AssertionError(f"{seq.seq_id}: page {page} twice in one table")
                    seen.add(page)
                    holders[page] = holders.get(page, 0) + 1
            for page in range(pool.num_pages):
                if pool.ref[page] != holders.get(page, 0):
                    raise AssertionError(
                        f"group {group} page {page}: {pool.ref[page]} holds recorded, "
                        f"{holders.get(page, 0)} tables list it"
                    )
                if holders.get(page, 0) > 1 and pool.hash_of[page] is None:
                    raise AssertionError(f"group {group} page {page} is shared without a hash")
        slots = [seq.slot for seq in self.live.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot has two owners")
        if len(slots) + len(self._free_slots) != self.num_slots:
            raise AssertionError("a state slot was lost")
