"""Traces for the replay tests: the same requests cut in different ways.

Each builder returns `(steps, rows)`: `steps` is the list of JSON-able step objects that
`trace_run` reads, and `rows[step number]` lists, in output order, the (request id,
position) whose logits that step writes. The oracle computes every request whole, so any
row of any cutting can be checked against it.
"""

from __future__ import annotations

import random

ROUND = 64


def _rounded(n: int) -> int:
    return -(-n // ROUND) * ROUND


def whole(requests: dict[str, list[int]]):
    """Each request alone, all its tokens in one step, logits everywhere."""
    steps, rows = [], {}
    for number, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": number, "end": [rid],
                      "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}]})
        rows[number] = [(rid, p) for p in range(len(tokens))]
    return steps, rows


def decode_tail(requests: dict[str, list[int]], tail: int = 32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps, rows = [], {}
    number = 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": number, "end": [],
                      "entries": [{"id": rid, "tokens": tokens[:head], "want": [head - 1]}]})
        rows[number] = [(rid, head - 1)]
        number += 1
        for p in range(head, len(tokens)):
            steps.append({"step": number, "end": [rid] if p == len(tokens) - 1 else [],
                          "entries": [{"id": rid, "tokens": [tokens[p]], "want": [0]}]})
            rows[number] = [(rid, p)]
            number += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps, rows


def portions(requests: dict[str, list[int]], sizes=(2, 7, 16, 3, 33, 2, 64, 5, 17, 2, 31)):
    """Portions of changing size, down to two tokens, not aligned to pages."""
    steps, rows = [], {}
    number = 0
    turn = 0
    for rid, tokens in requests.items():
        at = 0
        while at < len(tokens):
            n = min(sizes[turn % len(sizes)], len(tokens) - at)
            turn += 1
            done = at + n == len(tokens)
            steps.append({"step": number, "end": [rid] if done else [],
                          "entries": [{"id": rid, "tokens": tokens[at:at + n],
                                       "want": list(range(n))}]})
            rows[number] = [(rid, at + i) for i in range(n)]
            at += n
            number += 1
    return steps, rows


def mixed(requests: dict[str, list[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
          tail: int = 32, first_portion: int | None = None):
    """Up to `max_live` requests alive, portions of some beside single decoded tokens of
    others, some left out of a step; a new request starts only when the rounded token
    counts of the live ones leave room in `max_tokens`, so pages get used again. With
    `first_portion` a request's first entry brings that many tokens and wants the last one
    only, so that a replay with prefix caching may start it on cached pages."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}
    steps, rows = [], {}
    number = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting[0]
            held = sum(_rounded(len(requests[r])) for r in live)
            if held + _rounded(len(tokens)) > max_tokens:
                break
            waiting.pop(0)
            live[rid] = 0
        if not live:
            raise ValueError("a request does not fit the pool at all")
        entries, out_rows, ended = [], [], []
        chosen = [r for r in live if rng.random() < 0.8] or [next(iter(live))]
        for rid in chosen:
            tokens = requests[rid]
            at = live[rid]
            prompt_end = max(1, len(tokens) - tail)
            if at == 0 and first_portion:
                n = min(first_portion, prompt_end)
                want = [n - 1]
            elif at < prompt_end:
                n = min(rng.choice((2, 3, 5, 8, 13, 16, 21, 40)), prompt_end - at)
                want = list(range(n)) if rng.random() < 0.5 else [n - 1]
            else:
                n, want = 1, [0]
            entries.append({"id": rid, "tokens": tokens[at:at + n], "want": want})
            out_rows += [(rid, at + w) for w in want]
            live[rid] = at + n
            if live[rid] == len(tokens):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        steps.append({"step": number, "entries": entries, "end": ended})
        rows[number] = out_rows
        number += 1
    return steps, rows
