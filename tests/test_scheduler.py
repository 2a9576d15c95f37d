"""The scheduler's decisions, without a model: a tiny driver books each planned entry as
computed and hands back deterministic tokens (the idea of the reference's
DeterministicRunner, mercury/testing.py:20-64)."""

from __future__ import annotations

import zlib

import pytest

from mercury_b200.cache import CacheManager, extend_hashes
from mercury_b200.engine.request import Request, RequestState
from mercury_b200.engine.scheduler import Scheduler

PAGE = 16


class Driver:
    def __init__(self, num_pages=64, **options):
        self.cache = CacheManager([0], num_pages, PAGE, options.get("max_running", 64))
        self.sched = Scheduler(self.cache, **options)
        self.now = 1000.0
        self.plans = []
        self.finished: list[Request] = []

    def add(self, rid, prompt, max_tokens=4, arrival=None):
        r = Request(rid=rid, prompt=list(prompt), max_tokens=max_tokens,
                    arrival=self.now if arrival is None else arrival,
                    hashes=self.sched.hashes_of(prompt))
        self.sched.add(r)
        return r

    def step(self):
        plan = self.sched.schedule(self.now)
        self.plans.append(plan)
        for e in plan.entries:
            r = e.request
            covered = len(r.seq.tables[0]) * PAGE
            assert covered >= e.start + e.count, "planned tokens have no pages"
            assert e.start == r.num_computed
            extend_hashes(r.hashes, r.tokens, PAGE)
            self.cache.advance(r.seq, e.start + e.count, r.hashes)
            if e.samples:
                r.out.append((zlib.crc32(r.rid.encode()) + 7919 * len(r.out)) % 1000)
                if len(r.out) >= r.max_tokens:
                    r.state = RequestState.FINISHED
                    self.sched.drop(r)
                    self.finished.append(r)
        self.cache.check_invariants()
        return plan

    def run(self, limit=10_000):
        steps = 0
        while self.sched.has_work():
            self.step()
            steps += 1
            assert steps < limit, "the scheduler does not finish"
        return steps


def prompt(n, base=0):
    return [(base + i) % 997 for i in range(n)]


def test_fcfs_admits_in_arrival_order():
    d = Driver(max_running=2)
    for i in range(4):
        d.add(f"r{i}", prompt(20, i * 100), arrival=float(i))
    plan = d.step()
    assert [e.request.rid for e in plan.entries] == ["r0", "r1"]


def test_prompts_are_cut_into_portions_under_the_token_budget():
    d = Driver(max_batched_tokens=48, prefill_chunk=32, max_running=4)
    r = d.add("long", prompt(100), max_tokens=3)
    counts = []
    while not r.out:
        plan = d.step()
        assert plan.num_tokens <= 48
        counts.append([e.count for e in plan.entries if e.request is r][0])
    assert counts == [32, 32, 32, 4]
    plan = d.step()
    assert [(e.count, e.samples) for e in plan.entries] == [(1, True)]


def test_decode_tokens_come_before_prompt_portions_and_share_the_budget():
    d = Driver(max_batched_tokens=40, prefill_chunk=64, max_running=8)
    a = d.add("a", prompt(10), max_tokens=50, arrival=0.0)
    d.step()
    assert len(a.out) == 1
    b = d.add("b", prompt(100, 300), max_tokens=2, arrival=1.0)
    plan = d.step()
    by_rid = {e.request.rid: e for e in plan.entries}
    assert by_rid["a"].count == 1 and by_rid["a"].samples
    assert by_rid["b"].count == 39 and not by_rid["b"].samples      # 40 - 1 decode token
    plan = d.step()
    by_rid = {e.request.rid: e for e in plan.entries}
    assert by_rid["b"].start == 39 and by_rid["b"].count == 39
    assert plan.entries[0].request is a


def test_lpm_prefers_the_cached_prefix_and_fcfs_does_not():
    for policy, first in (("lpm", "warm"), ("fcfs", "cold")):
        d = Driver(policy=policy, max_running=1)
        d.add("seed", prompt(48), max_tokens=1)
        d.run()
        d.add("cold", prompt(48, 500), arrival=2000.0)
        d.add("warm", prompt(48) + [5, 6], arrival=2001.0)
        plan = d.step()
        assert plan.entries[0].request.rid == first
        if policy == "lpm":
            assert plan.entries[0].request.num_cached == 48
            assert plan.entries[0].start == 48 and plan.entries[0].count == 2


def test_when_the_front_does_not_fit_fcfs_blocks_and_lpm_skips():
    for policy, expect in (("fcfs", ["hold"]), ("lpm", ["hold", "small"])):
        d = Driver(num_pages=8, policy=policy, max_running=4)
        d.add("hold", prompt(64), max_tokens=30, arrival=0.0)
        d.step()
        d.add("big", prompt(100, 300), arrival=1.0)        # 7 pages, only 4 left
        d.add("small", prompt(20, 600), arrival=2.0)
        plan = d.step()
        assert [e.request.rid for e in plan.entries] == expect


def test_aging_lets_a_waiting_request_overtake_and_starvation_blocks():
    d = Driver(policy="lpm_aging", max_running=1, aging_tokens_per_s=10.0, max_wait_s=5.0)
    d.add("seed", prompt(64), max_tokens=1)
    d.run()
    d.add("old", prompt(32, 500), arrival=d.now - 4.0)       # 4 s * 10 = 40 < 64 cached
    d.add("warm", prompt(64) + [1], arrival=d.now)
    assert d.step().entries[0].request.rid == "warm"
    d2 = Driver(policy="lpm_aging", max_running=1, aging_tokens_per_s=10.0, max_wait_s=5.0)
    d2.add("seed", prompt(64), max_tokens=1)
    d2.run()
    d2.add("old", prompt(32, 500), arrival=d2.now - 6.0)     # waited past max_wait_s
    d2.add("warm", prompt(64) + [1], arrival=d2.now)
    assert d2.step().entries[0].request.rid == "old"


def test_scan_limit_bounds_the_scored_head():
    d = Driver(policy="lpm", scan_limit=2, max_running=1)
    d.add("seed", prompt(48), max_tokens=1)
    d.run()
    d.add("a", prompt(20, 100), arrival=3000.0)
    d.add("b", prompt(20, 200), arrival=3001.0)
    d.add("warm", prompt(48) + [9], arrival=3002.0)           # outside the scanned head
    assert d.step().entries[0].request.rid == "a"
    assert d.sched.stats["scan_limit_exceeded"] == 1


def test_when_pages_run_out_the_newest_is_preempted_and_resumes():
    d = Driver(num_pages=6, max_running=4)
    a = d.add("a", prompt(40), max_tokens=40, arrival=0.0)     # 3 pages, grows to 5
    b = d.add("b", prompt(40, 300), max_tokens=40, arrival=1.0)
    d.step()
    assert a.state is RequestState.RUNNING and b.state is RequestState.RUNNING
    preempted = []
    while not preempted:
        preempted = d.step().preempted
    assert preempted == [b] and b.state is RequestState.WAITING and b.seq is None
    assert b.preemptions == 1 and a.state is RequestState.RUNNING
    kept = list(b.out)
    d.run()
    assert len(a.out) == 40 and len(b.out) == 40 and b.out[:len(kept)] == kept
    assert d.cache.leaked_pages() == 0


def test_two_hundred_requests_give_every_page_back():
    d = Driver(num_pages=40, max_running=8, max_batched_tokens=96, prefill_chunk=40, policy="lpm")
    for i in range(200):
        shared = prompt(32, (i % 5) * 50)
        d.add(f"r{i}", shared + prompt(1 + (i * 7) % 60, 400 + i), max_tokens=1 + i % 9,
              arrival=float(i))
    d.run()
    assert len(d.finished) == 200
    assert all(len(r.out) == r.max_tokens for r in d.finished)
    assert d.cache.leaked_pages() == 0 and d.cache.num_available() == [40]
    assert d.cache.stats["hit_tokens"] > 0
    assert max(p.num_tokens for p in d.plans) <= 96


def test_abort_gives_pages_back_mid_prompt():
    d = Driver(max_batched_tokens=32, prefill_chunk=16, max_running=2)
    d.add("x", prompt(100), max_tokens=5)
    d.step()
    assert d.cache.num_available()[0] < 64
    assert d.sched.abort("x").state is RequestState.ABORTED
    assert d.cache.num_available() == [64] and not d.sched.has_work()
    assert d.sched.abort("nobody") is None
