"""The engine loop: drain commands, schedule, run one step, sample, route tokens.

`Engine.submit` / `step` / `abort` keep the reference's meaning (mercury/engine.py:104-113,
:144, :154); `generate` is the offline entry point the reference's tests spell out by hand
(tests/test_runner.py:65-77 of the reference): submit every prompt, step until nothing is
left, return the tokens by request. The loop runs on the caller's thread; there is no
server around it.

A step is launched and read back in two halves, and `step()` puts the launch of the next
step between them whenever the next plan cannot depend on what the tokens turn out to be:
the requests that go on get a stand-in for the token that is still on the device, the
scheduler plans with it, the next step takes the real ids from the device, and only then
does the host wait for the tokens of the step in front. The GPU so never waits for the
host's bookkeeping. A request that ends on a token read this way (end of sequence) has
one surplus token computed, which is dropped.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable

from ..cache.hashing import extend_hashes
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, request_seed
from .batch import StepEntry
from .metrics import EngineMetrics, StepRecord, request_record
from .request import Request, RequestState
from .runner import ModelRunner
from .scheduler import Plan, Scheduler


@dataclass(slots=True)
class StreamEvent:
    """What a request's sink receives (mercury/engine.py:17-25): kind is "token", "done",
    "error" or "preempted"."""

    rid: str
    kind: str
    token: int | None = None
    index: int = 0
    finish_reason: str | None = None
    message: str | None = None
    t: float = 0.0


Sink = Callable[[StreamEvent], None]

STAND_IN = -1     # in a request's output: a token sampled on the device and not read back yet


@dataclass
class _Flight:
    """A step that has been launched: its plan, whose row of sampled tokens is whose, and
    the sampler's handle to read them back with."""

    plan: Plan
    sampling: list[Request] = field(default_factory=list)
    handle: tuple[int, int] | None = None
    t_start: float = 0.0
    prepare_s: float = 0.0
    kernel_ms: dict | None = None


class Engine:
    def __init__(self, cfg: EngineConfig, runner: ModelRunner | None = None,
                 clock: Callable[[], float] = time.perf_counter, ops=None):
        self.cfg = cfg
        self.clock = clock
        if runner is None:
            runner = ModelRunner(
                cfg.model, dtype=cfg.torch_dtype, device=cfg.device, page_size=cfg.block_size,
                num_pages=cfg.num_blocks, max_seqs=cfg.max_running,
                max_step_tokens=cfg.max_batched_tokens, max_model_len=cfg.max_model_len, ops=ops,
                cuda_graphs=cfg.cuda_graphs, poison_pages=cfg.debug_poison_pages)
        self.runner = runner
        if cfg.time_kernels:
            runner.time_kernels = True
        cfg.validate_against(runner.spec.max_positions)
        self.cache = runner.cache
        # a request skips the tokens of a cached prefix in every layer or in none, so one
        # mixer that has to see every token (state of its own) rules the skip out
        prefix_caching = cfg.prefix_caching and runner.model.skips_cached_prefix
        self.sched = Scheduler(
            self.cache, policy=cfg.policy, max_running=cfg.max_running,
            prefill_budget=cfg.prefill_budget, max_batched_tokens=cfg.max_batched_tokens,
            prefill_chunk=cfg.prefill_chunk, aging_tokens_per_s=cfg.aging_tokens_per_s,
            max_wait_s=cfg.max_wait_s, scan_limit=cfg.scan_limit, prefix_caching=prefix_caching,
            cryptographic_hashes=cfg.cryptographic_hashes)
        self.sampler = Sampler(runner.ops, runner.device, cfg.max_running)
        self.metrics = EngineMetrics(cfg.max_step_records)
        self.eos_ids = set(runner.spec.eos_token_ids or ())
        self._commands: list[tuple[str, object]] = []
        self._sinks: dict[str, Sink] = {}
        self._submitted = 0
        self._flight: _Flight | None = None
        self.lookahead = cfg.lookahead
        # debugging aid: called as tap(requests, logits) with the float32 logits rows a step
        # samples from (row i belongs to requests[i], whose next output index is len(out))
        self.tap: Callable | None = None

    # ------------------------------------------------------------------ client side

    def submit(self, rid: str, prompt_ids: list[int], max_tokens: int, sink: Sink,
               params: SamplingParams | None = None, arrival: float | None = None) -> None:
        params = params or SamplingParams()
        arrival = self.clock() if arrival is None else arrival
        ceiling = min(self.runner.max_model_len, self.cfg.kv_capacity_tokens)
        if rid in self._sinks:
            return self._reject(rid, sink, f"a request named {rid!r} is still under way")
        if not prompt_ids:
            return self._reject(rid, sink, "prompt must contain at least one token")
        if max_tokens < 1:
            return self._reject(rid, sink, "max_tokens must be at least 1")
        if len(prompt_ids) + max_tokens > ceiling:
            return self._reject(
                rid, sink, f"prompt ({len(prompt_ids)}) + max_tokens ({max_tokens}) exceeds the "
                           f"{ceiling}-token ceiling of this engine")
        vocab = self.runner.vocab_size
        if any(not 0 <= int(t) < vocab for t in prompt_ids):
            return self._reject(rid, sink, f"a prompt token lies outside the vocabulary of {vocab}")
        r = Request(rid=rid, prompt=[int(t) for t in prompt_ids], max_tokens=max_tokens,
                    arrival=arrival, hashes=self.sched.hashes_of(prompt_ids), params=params,
                    seed=request_seed(params, self.cfg.seed, rid))
        self._sinks[rid] = sink
        self._submitted += 1
        self._commands.append(("add", r))

    def abort(self, rid: str) -> None:
        self._commands.append(("abort", rid))

    def _reject(self, rid: str, sink: Sink, message: str) -> None:
        self.metrics.counters["rejected_requests"] += 1
        sink(StreamEvent(rid=rid, kind="error", message=message, t=self.clock()))

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams]
                 | None = None, max_tokens: int = 16) -> list[list[int]]:
        """Generate for every prompt (token ids in, token ids out), batching them as the
        scheduler sees fit. Raises if a prompt is refused."""
        outs: dict[str, list[int]] = {}
        errors: list[str] = []

        def sink_for(rid):
            def sink(event: StreamEvent) -> None:
                if event.kind == "token":
                    outs[rid].append(event.token)
                elif event.kind == "error":
                    errors.append(f"{rid}: {event.message}")
            return sink

        base = self._submitted
        for i, prompt in enumerate(prompts):
            rid = f"gen-{base + i}"
            outs[rid] = []
            p = params[i] if isinstance(params, list) else params
            self.submit(rid, prompt, max_tokens, sink_for(rid), p, arrival=float(base + i))
        if errors:
            # nothing of a refused call stays queued
            mine = set(outs)
            self._commands = [c for c in self._commands
                              if not (c[0] == "add" and c[1].rid in mine)]
            for rid in mine:
                self._sinks.pop(rid, None)
            raise ValueError("; ".join(errors))
        self.run_until_idle()
        return [outs[f"gen-{base + i}"] for i in range(len(prompts))]

    def run_until_idle(self) -> None:
        self._drain_commands()
        while self.sched.has_work() or self._commands or self._flight is not None:
            if self.step() is None and not self._commands and self.sched.has_work():
                raise RuntimeError("the scheduler has work but planned nothing: the pool is too "
                                   "small for the waiting request")

    # ------------------------------------------------------------------ the loop

    def step(self) -> StepRecord | None:
        """Read back one step (launching it first if none is under way) and, where that is
        safe, launch the step after it before waiting for the tokens."""
        t_start = time.perf_counter()
        self._drain_commands()
        flight = self._flight
        self._flight = None
        if flight is None:
            flight = self._launch(None, t_start)
            if flight is None:
                self.metrics.counters["idle_steps"] += 1
                return None
        ahead = None
        if self.lookahead and self._can_look_ahead(flight):
            for r in flight.sampling:
                # it goes on unless this token ends it; a request that has already ended
                # (end of sequence found one step late, or aborted) gets no stand-in
                if not r.done and len(r.out) + 1 < r.max_tokens:
                    r.out.append(STAND_IN)
                    r.unread = 1
            ahead = self._launch(flight, time.perf_counter())
            if ahead is not None:
                self.metrics.counters["steps_launched_ahead"] += 1
        record = self._complete(flight)
        self._flight = ahead
        return record

    def _can_look_ahead(self, flight: _Flight) -> bool:
        """Whether the plan of the next step is the same whatever the tokens of this one
        are: nobody new could be admitted, nobody has to be preempted for pages, and no
        command is waiting. (A request that ends on its token is found out one step late;
        that costs one surplus token, not a different plan for the others.)"""
        if self._commands:
            return False
        sched = self.sched
        ending = any(len(r.out) + 1 >= r.max_tokens for r in flight.sampling)
        if sched.waiting and (ending or (len(sched.running) < sched.max_running
                                         and self.cache.has_slot())):
            return False
        short = [0] * len(self.cache.pools)
        sampled = {id(r) for r in flight.sampling}
        for r in sched.running:
            if r.seq is None:
                continue
            length = r.seq_len + (1 if id(r) in sampled else 0)
            target = min(length, r.num_computed + sched.prefill_chunk)
            for group, pages in enumerate(self.cache.pages_short(r.seq, target)):
                short[group] += pages
        return all(n <= free for n, free in zip(short, self.cache.num_available()))

    def _launch(self, before: _Flight | None, t_start: float) -> _Flight | None:
        """Plan a step and put it on the device. `before` is the step in front if its tokens
        have not been read yet: stand-ins among this step's inputs are taken from there."""
        plan: Plan = self.sched.schedule(self.clock())
        for r in plan.preempted:
            self._emit(r, StreamEvent(rid=r.rid, kind="preempted", t=self.clock()))
        if not plan:
            return None
        row_of = {id(r): row for row, r in enumerate(before.sampling)} if before else {}
        entries, sampling = [], []
        page = self.cache.page_size
        for e in plan.entries:
            r = e.request
            hashes = None
            if self.sched.prefix_caching:
                # pages are hashed (and shared) only once all their tokens are known
                if r.known_len // page > len(r.hashes):
                    extend_hashes(r.hashes, r.tokens[:r.known_len], page,
                                  self.cfg.cryptographic_hashes)
                hashes = r.hashes
            late = None
            if r.unread and e.start + e.count == r.seq_len:
                late = (e.count - 1, row_of[id(r)])
            entries.append(StepEntry(r.seq, r.token_slice(e.start, e.count),
                                     [e.count - 1] if e.samples else [], hashes, late))
            if e.samples:
                sampling.append(r)
        sampled = self.sampler.on_device(before.handle) if before and before.handle else None
        logits = self.runner.step(entries, sampled)
        handle = None
        if sampling and self.tap is not None:
            self.tap(sampling, logits)
        if sampling:
            handle = self.sampler.begin(logits, [(r.params, r.seed, len(r.out)) for r in sampling])
        kernel_ms = dict(self.runner.last_kernel_ms) if getattr(self.runner, "time_kernels", False) else None
        return _Flight(plan, sampling, handle, t_start, getattr(self.runner, "last_prepare_s", 0.0),
                       kernel_ms)

    def _complete(self, flight: _Flight) -> StepRecord:
        """Wait for the step's tokens and route them."""
        tokens = self.sampler.finish(flight.handle) if flight.handle is not None else []
        now = self.clock()
        for r, token in zip(flight.sampling, tokens):
            if r.done:
                r.unread = 0
                self.metrics.counters["surplus_tokens"] += 1
                continue       # ended or aborted while this step ran: a surplus token
            self._accept(r, token, now)
        if self.cfg.debug_invariants:
            self.cache.check_invariants()
        plan = flight.plan
        record = StepRecord(
            t=now, num_entries=len(plan.entries), num_decode=plan.num_decode,
            num_tokens=plan.num_tokens, sched_s=plan.sched_seconds,
            step_s=time.perf_counter() - flight.t_start, waiting=len(self.sched.waiting),
            running=len(self.sched.running), free_pages=min(self.cache.num_available()),
            preempted=len(plan.preempted), prepare_s=flight.prepare_s, kernel_ms=flight.kernel_ms)
        self.metrics.add_step(record)
        return record

    def _drain_commands(self) -> None:
        commands, self._commands = self._commands, []
        for kind, payload in commands:
            if kind == "add":
                self.sched.add(payload)
            elif kind == "abort":
                r = self.sched.abort(payload)
                if r is not None and r.unread:
                    r.out.pop()            # the stand-in of a token that will not be read
                    r.unread = 0
                if r is not None:
                    self.metrics.counters["aborted_requests"] += 1
                    r.life.end = self.clock()
                    self.metrics.finished.append(request_record(r))
                    self._emit(r, StreamEvent(rid=r.rid, kind="done", finish_reason="abort",
                                              t=r.life.end), close=True)
                else:
                    self._sinks.pop(payload, None)

    def _accept(self, r: Request, token: int, now: float) -> None:
        if r.unread:
            index = len(r.out) - 1          # the stand-in becomes the token
            r.out[index] = int(token)
            r.unread = 0
        else:
            index = len(r.out)
            r.out.append(int(token))
        if r.life.first_token is None:
            r.life.first_token = now
        self._emit(r, StreamEvent(rid=r.rid, kind="token", token=int(token), index=index, t=now))
        if r.done:
            return   # the sink raised and the request was aborted
        if len(r.out) >= r.max_tokens:
            self._finish(r, "length", now)
        elif not r.params.ignore_eos and int(token) in self.eos_ids:
            self._finish(r, "stop", now)

    def _finish(self, r: Request, reason: str, now: float) -> None:
        r.end(RequestState.FINISHED, reason, now)
        self.sched.drop(r)
        self.metrics.counters["finished_requests"] += 1
        self.metrics.finished.append(request_record(r))
        self._emit(r, StreamEvent(rid=r.rid, kind="done", finish_reason=reason, t=now), close=True)

    def _emit(self, r: Request, event: StreamEvent, close: bool = False) -> None:
        sink = self._sinks.pop(r.rid, None) if close else self._sinks.get(r.rid)
        if sink is None:
            return
        try:
            sink(event)
        except Exception:
            # a sink that raises loses its request, not the loop (mercury/engine.py:259-262)
            self.abort(r.rid)

    # ------------------------------------------------------------------ reporting

    def leaked_pages(self) -> int:
        return self.cache.leaked_pages()

    def snapshot(self) -> dict:
        return {"config": self.cfg.to_dict(), "scheduler": self.sched.snapshot(),
                "cache": {**self.cache.stats, "available": self.cache.num_available(),
                          "evictions": [p.evictions for p in self.cache.pools]},
                "engine": self.metrics.summary(), "submitted": self._submitted}
