"""Logits of every schedule that the benchmark times, against the plain implementation, at
the layer widths of Qwen2.5-0.5B (two layers): a 2048-token prompt in one step and in four
portions of 512 (eager, captured and replayed); decode-only steps of 8 to 64 live sequences
through the captured batch-size buckets at contexts of 600 to 2048 tokens, every bucket
replayed with other lengths; and a captured prompt shape replayed with its tokens split
differently between the sequences and at another context length. The runner is driven
directly, since trace replay stops at four live requests."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from mercury_b200.engine.batch import StepEntry
from wide import WIDTHS, model, oracle_rows, relative_error, tokens_for

pytestmark = pytest.mark.gpu

NAME = "0.5B"
# float32: kernels and oracle differ only in the order of float32 sums. bfloat16 at these
# widths: the plain PyTorch twin of the kernels (float32 arithmetic, bfloat16 storage
# between kernels) is itself off from the float64 oracle by 1.3e-2 of the largest logit.
TOLERANCE = {torch.float32: 3e-5, torch.bfloat16: 2.3e-2}
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


class Driver:
    """Sequences by name over one `ModelRunner`; tokens come from `tokens_for(NAME, ...)`."""

    def __init__(self, dtype, max_seqs, num_tokens, max_step_tokens=2048, cuda_graphs=True):
        from mercury_b200.engine.runner import ModelRunner

        _raw, config, tensors = model(NAME)
        self.dtype = dtype
        self.runner = ModelRunner(config=config, tensors=tensors, dtype=dtype, device="cuda",
                                  page_size=16, num_pages=num_tokens // 16 + max_seqs,
                                  max_seqs=max_seqs, max_step_tokens=max_step_tokens,
                                  max_model_len=4096, cuda_graphs=cuda_graphs)
        self.live: dict = {}          # rid -> (Sequence, length, seed)

    def open(self, rid, length, seed):
        self.live[rid] = (self.runner.open(rid), length, seed)

    def close(self, rid):
        self.runner.close(self.live.pop(rid)[0])

    def step(self, parts):
        """`parts`: [(rid, count, wanted places)]: each request's next `count` tokens.
        Returns the worst relative error over the wanted rows (0.0 if none is wanted)."""
        entries, expect = [], []
        for rid, count, want in parts:
            seq, length, seed = self.live[rid]
            at = seq.num_computed
            entries.append(StepEntry(seq, tokens_for(NAME, length, seed)[at:at + count], list(want)))
            expect.append((length, seed, tuple(at + w for w in want)))
        logits = self.runner.step(entries)
        if logits is None:
            return 0.0
        got = logits.float().cpu().numpy()
        assert np.isfinite(got).all()
        worst, row = 0.0, 0
        for (rid, _count, _want), (length, seed, rows) in zip(parts, expect):
            if not rows:
                continue
            want = oracle_rows(NAME, length, seed, rows)
            err = relative_error(got[row:row + len(rows)], want)
            assert err <= TOLERANCE[self.dtype], (
                f"request {rid} positions {rows[0]}..{rows[-1]}: relative error {err:.3e}")
            worst = max(worst, err)
            row += len(rows)
        return worst

    def finish(self):
        assert not self.runner.cache.live
        self.runner.cache.check_invariants()
        assert self.runner.cache.leaked_pages() == 0


def chosen_rows(length: int, count: int, seed: int) -> list[int]:
    """Exactly `count` places among `length` tokens: the edges of pages and tiles first,
    random ones for the rest (the count is fixed so that a step's shape comes back)."""
    edges = [0, 1, 15, 16, 17, 63, 64, 65, 127, 128, 255, 256, length - 2, length - 1,
             511, 512, 513, 1023, 1024, 1535, 1536, 1537]
    gen = torch.Generator().manual_seed(seed)
    picked: list[int] = []
    for p in edges + torch.randint(0, length, (4 * count,), generator=gen).tolist():
        if 0 <= p < length and p not in picked and len(picked) < count:
            picked.append(p)
    return sorted(picked)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("cut", [2048, 512], ids=["one-step", "4x512"])
def test_prompt_of_2048_tokens(dtype, cut):
    """The prompt step of the benchmark: three prompts in a row, so that the first runs
    eagerly, the second is captured as a graph and replayed, and the third replays it."""
    driver = Driver(dtype, max_seqs=2, num_tokens=2048)
    for turn, seed in enumerate((31, 32, 33)):
        rid = f"p{turn}"
        driver.open(rid, 2048, seed)
        for start in range(0, 2048, cut):
            driver.step([(rid, cut, chosen_rows(cut, 64 if cut == 2048 else 20, seed + start))])
        driver.close(rid)
    assert driver.runner.graph_replays >= 2, "the captured prompt step was never replayed"
    driver.finish()


def _fill(driver, group):
    """Prefill the sequences of `group` = [(rid, length, seed)] up to three tokens before
    their end, several prompts to a step."""
    waiting = list(group)
    while waiting:
        batch, room = [], driver.runner.max_step_tokens
        while waiting and len(batch) < 4 and waiting[0][1] - 3 <= room:
            rid, length, seed = waiting.pop(0)
            driver.open(rid, length, seed)
            batch.append((rid, length - 3, []))
            room -= length - 3
        assert batch
        driver.step(batch)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("live", [8, 16, 17, 33, 64])
def test_decode_steps_through_the_buckets(dtype, live):
    """Decode-only steps of `live` sequences (buckets 8, 16, 32, 64, 64): three steps on one
    set of sequences, then, on the same captured graph, three steps on another set with
    other lengths. With 8 live sequences the first set holds the benchmark's 2048-token
    contexts."""
    if live == 8:
        first = [(f"a{i}", 2040 + 3 * i, 500 + i) for i in range(live)]
    else:
        first = [(f"a{i}", 600 + (53 * i) % 400, 500 + i) for i in range(live)]
    second = [(f"b{i}", 640 + (97 * i + 11) % 700, 700 + i) for i in range(live)]
    most = max(sum(length for _r, length, _s in group) for group in (first, second))
    driver = Driver(dtype, max_seqs=64, num_tokens=most + 64 * 16, max_step_tokens=4096)
    for group in (first, second):
        _fill(driver, group)
        for _ in range(3):
            before = driver.runner.graph_replays
            driver.step([(rid, 1, [0]) for rid, _length, _seed in group])
            assert driver.runner.graph_replays == before + 1
        for rid, _length, _seed in group:
            driver.close(rid)
    assert len(driver.runner._graphs) == 1, "both sets must run on one captured bucket"
    driver.finish()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("long_first", [False, True], ids=["short-then-long", "long-then-short"])
def test_captured_prompt_shape_with_another_split(dtype, long_first):
    """A prompt step's graph is kept per (tokens, sequences, longest portion, wanted rows).
    The same shape comes back with the tokens split the other way round between the two
    sequences, and at a context on the other side of every length-dependent choice made at
    capture (key tiles per row tile, CTAs per row tile)."""
    driver = Driver(dtype, max_seqs=2, num_tokens=2 * 1100, max_step_tokens=2048)
    driver.open("x", 1100, 41)
    driver.open("y", 1100, 42)

    def shape_steps():
        driver.step([("x", 40, [39]), ("y", 24, [0, 23])])     # first sight: eager
        driver.step([("x", 24, [5]), ("y", 40, [38, 39])])     # second: captured and replayed
        driver.step([("x", 40, [0]), ("y", 24, [10, 23])])     # replayed, split as at first

    def grow(count):
        driver.step([("x", count, [count - 1]), ("y", count, [count - 1])])

    if long_first:
        grow(800)
        shape_steps()
    else:
        shape_steps()
        grow(800)
    before = driver.runner.graph_replays
    driver.step([("x", 24, [23]), ("y", 40, [0, 39])])          # the captured shape, far from capture
    driver.step([("x", 40, [39]), ("y", 24, [1, 23])])
    assert driver.runner.graph_replays == before + 2
    driver.close("x")
    driver.close("y")
    driver.finish()
