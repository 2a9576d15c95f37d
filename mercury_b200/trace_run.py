"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come from standard input, one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Each entry brings a request's next tokens and the places among them whose logits are
wanted; all entries of a step run as ONE batch through the engine's own step function
(`ModelRunner.step`), from the cache that earlier steps left. `end` lists the requests that
are finished after the step; their pages and state slot go back to the pool. For a step
that wants something, `OUT/<step>.f32` receives the logits as little-endian float32
`[wanted, vocab]`, in the order of the entries and of each `want`. After every step a line
`done <step>` is printed and flushed. Nothing is sampled.

The page pool is sized for `--max-tokens` tokens, so pages of finished requests are used
again by later ones. The reference has no such program; its nearest piece is
`ModelRunner.forward_prompt` (mercury/runner.py:182-206).

Two switches for testing the cache. `--prefix-caching`: the full pages of every request
are hashed as its tokens arrive (chain hashes over the tokens fed so far) and stay in the
pool after the request ends; a new request whose first entry begins with pages that are
still there starts on them and runs only the rest of that entry (never skipping a place
whose logits are wanted, and always leaving one token to run). The logits written are
the same either way, beyond rounding. `--poison-pages`: pages are filled with NaN whenever
they change hands (see `ModelRunner`).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from .cache.hashing import extend_hashes, page_hashes
from .config.engine_config import engine_dtype
from .engine.batch import StepEntry
from .engine.runner import ModelRunner

MAX_LIVE = 4          # requests alive at a time
ROUND_TO = 64         # a request's token count is rounded up to this before it is summed


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    p.add_argument("--out", required=True, help="folder that receives <step>.f32")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--device", default="cuda")
    p.add_argument("--prefix-caching", action="store_true",
                   help="a new request starts on cached pages of an equal prefix")
    p.add_argument("--poison-pages", action="store_true",
                   help="debugging: fill pages with NaN whenever they change hands")
    return p


def make_runner(args, ops=None) -> ModelRunner:
    page = args.block_size
    if ROUND_TO % page and page % ROUND_TO:
        raise SystemExit(f"--block-size {page} neither divides nor is a multiple of {ROUND_TO}")
    tokens = -(-args.max_tokens // max(page, ROUND_TO)) * max(page, ROUND_TO)
    return ModelRunner(
        args.model,
        dtype=engine_dtype(args.dtype),
        device=args.device,
        page_size=page,
        num_pages=max(1, tokens // page),
        max_seqs=MAX_LIVE,
        max_step_tokens=max(tokens, 1),
        max_model_len=None,
        ops=ops,
        poison_pages=getattr(args, "poison_pages", False),
    )


class _Live:
    """A request under replay: its sequence and, with prefix caching, the tokens fed so far
    and the chain hashes of their full pages."""

    def __init__(self, seq):
        self.seq = seq
        self.tokens: list[int] = []
        self.hashes: list[int] = []


def _start_on_cached_pages(runner: ModelRunner, held: _Live, tokens: list[int], want: list[int]):
    """A new request's first entry: take what the pool still holds of its leading pages.
    Returns the entry's tokens and wanted places with the covered tokens cut off."""
    page = runner.page_size
    usable = min(want) if want else len(tokens) - 1     # no wanted place may be skipped
    hashes = page_hashes(tokens, page)[:max(0, usable) // page]
    if not hashes or not runner.cache.admit(held.seq, hashes, len(tokens)):
        return tokens, want
    skipped = held.seq.num_computed
    return tokens[skipped:], [w - skipped for w in want]


def replay(runner: ModelRunner, lines, out_dir: Path, report=print,
           prefix_caching: bool = False) -> int:
    out_dir.mkdir(parents=True, exist_ok=True)
    live: dict[str, _Live] = {}
    page = runner.page_size
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for item in step.get("entries", []):
            rid = str(item["id"])
            tokens = [int(t) for t in item["tokens"]]
            want = [int(w) for w in item.get("want", [])]
            held = live.get(rid)
            hashes = None
            if held is None:
                held = live[rid] = _Live(runner.open(rid))
                if prefix_caching:
                    held.tokens += tokens
                    tokens, want = _start_on_cached_pages(runner, held, tokens, want)
            elif prefix_caching:
                held.tokens += tokens
            if prefix_caching:
                extend_hashes(held.hashes, held.tokens, page)
                hashes = held.hashes
            entries.append(StepEntry(held.seq, tokens, want, hashes))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                data = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                data.astype("<f4", copy=False).tofile(out_dir / f"{step['step']}.f32")
        for rid in step.get("end", []):
            held = live.pop(str(rid), None)
            if held is not None:
                runner.close(held.seq)
        report(f"done {step['step']}")
    return 0


def main(argv=None, ops=None) -> int:
    args = build_parser().parse_args(argv)
    runner = make_runner(args, ops)

    def report(text: str) -> None:
        sys.stdout.write(text + "\n")
        sys.stdout.flush()

    return replay(runner, sys.stdin, Path(args.out), report, prefix_caching=args.prefix_caching)


if __name__ == "__main__":
    raise SystemExit(main())
