"""Continuous batching with prompts cut into portions.

One pass per engine step (mercury/scheduler.py:122-179), extended by a per-step token
budget: first every running request gets room for what it runs next (one decoded token, or
the next portion of its prompt), then waiting requests are admitted in policy order while
sequences, tokens and pages allow.

What happens when pages run out is decided here: the request admitted last is preempted by
recompute (its pages go back, it waits again as a longer prompt and usually finds its own
pages still cached), as in mercury/scheduler.py:91-101, :127-135. A request that cannot
be admitted for lack of pages blocks the queue under `fcfs`, is skipped under `lpm`, and
under `lpm_aging` is skipped until it starves (mercury/scheduler.py:155-159).
"""

from __future__ import annotations

import bisect
import time
from dataclasses import dataclass, field

from ..cache.hashing import page_hashes
from ..cache.manager import CacheManager
from .request import Request, RequestState


@dataclass
class PlannedEntry:
    request: Request
    start: int          # position of the first token this step runs
    count: int          # how many tokens it runs
    samples: bool       # whether the step reaches the request's last known token


@dataclass
class Plan:
    entries: list[PlannedEntry] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    sched_seconds: float = 0.0

    def __bool__(self) -> bool:
        return bool(self.entries)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)

    @property
    def num_decode(self) -> int:
        return sum(1 for e in self.entries if e.count == 1 and e.samples)


class Scheduler:
    def __init__(self, cache: CacheManager, policy: str = "fcfs", max_running: int = 64,
                 prefill_budget: int = 8192, max_batched_tokens: int = 8192,
                 prefill_chunk: int = 2048, aging_tokens_per_s: float = 2000.0,
                 max_wait_s: float = 5.0, scan_limit: int = 128, prefix_caching: bool = True,
                 cryptographic_hashes: bool = False):
        self.cache = cache
        self.policy = policy
        self.max_running = max_running
        self.prefill_budget = prefill_budget
        self.max_batched_tokens = max_batched_tokens
        self.prefill_chunk = prefill_chunk
        self.aging = aging_tokens_per_s
        self.max_wait_s = max_wait_s
        self.scan_limit = scan_limit
        self.prefix_caching = prefix_caching
        self.cryptographic = cryptographic_hashes
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self.stats = {"steps": 0, "sched_seconds": 0.0, "preemptions": 0, "admissions": 0,
                      "max_waiting": 0, "scan_limit_exceeded": 0, "scored_requests": 0}

    # ------------------------------------------------------------------ queue operations

    def add(self, r: Request) -> None:
        r.state = RequestState.WAITING
        bisect.insort(self.waiting, r, key=lambda x: x.arrival)

    def _release(self, r: Request) -> None:
        if r.seq is not None:
            self.cache.close(r.seq)
            r.seq = None

    def abort(self, rid: str) -> Request | None:
        for queue in (self.waiting, self.running):
            for r in queue:
                if r.rid == rid:
                    queue.remove(r)
                    self._release(r)
                    r.end(RequestState.ABORTED, "abort")
                    return r
        return None

    def drop(self, r: Request) -> None:
        """Finished normally: give the pages back; the hashed ones stay cached."""
        if r in self.running:
            self.running.remove(r)
        elif r in self.waiting:
            self.waiting.remove(r)
        self._release(r)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def hashes_of(self, tokens) -> list[int]:
        if not self.prefix_caching:
            return []
        return page_hashes(tokens, self.cache.page_size, cryptographic=self.cryptographic)

    def _preempt(self, r: Request) -> None:
        self.running.remove(r)
        self._release(r)
        r.back_to_waiting()
        r.hashes = self.hashes_of(r.tokens)
        self.stats["preemptions"] += 1
        bisect.insort(self.waiting, r, key=lambda x: x.arrival)

    def _score(self, r: Request, now: float) -> float:
        """Admission priority, high first (mercury/scheduler.py:103-120)."""
        if self.policy == "fcfs":
            return -r.arrival
        cached = self.cache.cached_prefix_tokens(r.hashes)
        if self.policy == "lpm":
            return float(cached)
        waited = now - r.arrival
        if waited >= self.max_wait_s:
            return float("inf")
        return cached + self.aging * waited

    # ------------------------------------------------------------------ one pass

    def schedule(self, now: float) -> Plan:
        t0 = time.perf_counter()
        preempted: list[Request] = []
        planned: dict[str, PlannedEntry] = {}
        budget = self.max_batched_tokens

        def give(r: Request, count: int) -> bool:
            """Pages for `count` more tokens of r, preempting from the back of the running
            list while there are none. False if r itself had to go."""
            nonlocal budget
            while not self.cache.ensure(r.seq, r.num_computed + count):
                victim = self.running[-1]
                if victim.rid in planned:
                    budget += planned.pop(victim.rid).count
                self._preempt(victim)
                preempted.append(victim)
                if victim is r:
                    return False
            return True

        # 1. decode tokens first, then the next portions of prompts still being prefilled
        for decode_pass in (True, False):
            for r in list(self.running):
                if r.state is not RequestState.RUNNING or r.rid in planned:
                    continue
                remaining = r.seq_len - r.num_computed
                if (remaining == 1) != decode_pass:
                    continue
                count = min(remaining, self.prefill_chunk, budget)
                if count <= 0:
                    continue
                if give(r, count):
                    planned[r.rid] = PlannedEntry(r, r.num_computed, count, count == remaining)
                    budget -= count

        # 2. admissions in policy order
        head = self.waiting[: self.scan_limit]
        tail = self.waiting[self.scan_limit:]
        if tail:
            self.stats["scan_limit_exceeded"] += 1
        self.stats["scored_requests"] += len(head)
        order = sorted(head, key=lambda r: (-self._score(r, now), r.arrival)) + tail
        admitted: list[Request] = []
        prefill_left = self.prefill_budget
        for r in order:
            if r in preempted:
                continue      # it just lost its pages; let it wait one step
            if len(self.running) + len(admitted) >= self.max_running or budget <= 0:
                break
            if not self.cache.has_slot():
                break
            hit_pages = self.cache.match_prefix(r.hashes, r.seq_len) if r.hashes else 0
            new_tokens = r.seq_len - hit_pages * self.cache.page_size
            if admitted and new_tokens > prefill_left:
                break
            seq = self.cache.open(r.rid)
            if not self.cache.admit(seq, r.hashes, r.seq_len):
                self.cache.close(seq)
                starving = self.policy == "lpm_aging" and self._score(r, now) == float("inf")
                if self.policy == "fcfs" or starving:
                    break
                continue
            r.start_running(seq, now)
            prefill_left -= new_tokens
            count = min(new_tokens, self.prefill_chunk, budget)
            planned[r.rid] = PlannedEntry(r, r.num_computed, count, count == new_tokens)
            budget -= count
            admitted.append(r)

        if admitted:
            ids = {id(r) for r in admitted}
            self.waiting = [r for r in self.waiting if id(r) not in ids]
            self.running.extend(admitted)
            self.stats["admissions"] += len(admitted)

        elapsed = time.perf_counter() - t0
        self.stats["steps"] += 1
        self.stats["sched_seconds"] += elapsed
        self.stats["max_waiting"] = max(self.stats["max_waiting"], len(self.waiting))
        entries = [planned[r.rid] for r in self.running if r.rid in planned]
        return Plan(entries=entries, preempted=preempted, sched_seconds=elapsed)

    def snapshot(self) -> dict:
        steps = self.stats["steps"] or 1
        return {"policy": self.policy, "waiting": len(self.waiting), "running": len(self.running),
                "mean_sched_seconds": self.stats["sched_seconds"] / steps, **self.stats}
