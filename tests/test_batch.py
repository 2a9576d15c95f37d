"""The step's host buffer: rows of block tables that are kept from one step to the next
must read exactly as if every step had written them from nothing."""

import random

import pytest
import torch

from mercury_b200.cache.manager import CacheManager
from mercury_b200.engine.batch import BatchBuffers, StepEntry

PAGE = 4


def fields(batch):
    return {
        "token_ids": batch.token_ids.tolist(), "positions": batch.positions.tolist(),
        "seq_of_token": batch.seq_of_token.tolist(), "q_start": batch.q_start.tolist(),
        "kv_len": batch.kv_len.tolist(), "slots": batch.slots.tolist(),
        "logit_rows": batch.logit_rows.tolist(), "tables": [t.tolist() for t in batch.tables],
        "shape": (batch.num_tokens, batch.num_seqs, batch.max_q_len, batch.max_kv_len,
                  batch.num_logit_rows, batch.decode_only),
    }


@pytest.mark.parametrize("windows", [(0,), (0, 6), (6,)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_kept_rows_equal_rows_written_anew(windows, seed):
    rng = random.Random(seed)
    cache = CacheManager(windows, 400, PAGE, 4)
    append_only = [w == 0 for w in windows]
    kept = BatchBuffers("cpu", 64, 4, 32, len(windows), pin=False, append_only=append_only)
    live, serial = [], 0
    for _step in range(300):
        if live and rng.random() < 0.08:
            cache.close(live.pop(rng.randrange(len(live))))
        while len(live) < 4 and rng.random() < 0.5:
            live.append(cache.open(f"s{serial}"))
            serial += 1
        if not live:
            continue
        chosen = [s for s in live if rng.random() < 0.8] or live[:1]
        if rng.random() < 0.3:
            rng.shuffle(chosen)
        decode = rng.random() < 0.7
        entries = []
        for seq in chosen:
            n = 1 if decode and seq.num_computed else rng.randint(1, 9)
            if seq.num_computed + n > 32 * PAGE:
                continue
            assert cache.ensure(seq, seq.num_computed + n)
            entries.append(StepEntry(seq, [rng.randrange(100) for _ in range(n)],
                                     [n - 1] if rng.random() < 0.7 else []))
        if not entries:
            continue
        fixed = rng.random() < 0.7       # a captured step's layout, or the exact one
        capacities = dict(token_capacity=4, seq_capacity=4, page_capacity=32, row_capacity=4) \
            if fixed and all(len(e.tokens) == 1 for e in entries) else {}
        anew = BatchBuffers("cpu", 64, 4, 32, len(windows), pin=False)
        assert fields(kept.build(entries, PAGE, **capacities)) == \
            fields(anew.build(entries, PAGE, **capacities))
        for e in entries:
            cache.advance(e.seq, e.seq.num_computed + len(e.tokens))
        if any(s.num_computed >= 30 * PAGE for s in live):
            for s in [s for s in live if s.num_computed >= 30 * PAGE]:
                live.remove(s)
                cache.close(s)


def test_entries_that_do_not_fit_are_refused():
    cache = CacheManager((0,), 16, PAGE, 2)
    buffers = BatchBuffers("cpu", 8, 2, 4, 1, pin=False)
    seq = cache.open("a")
    cache.ensure(seq, 3)
    with pytest.raises(ValueError):
        buffers.build([StepEntry(seq, [1, 2, 3], [3])], PAGE)
    with pytest.raises(ValueError):
        buffers.build([StepEntry(seq, list(range(9)), [])], PAGE)
    with pytest.raises(ValueError):
        buffers.build([StepEntry(seq, [1, 2, 3], [0])], PAGE, token_capacity=2)
