"""Command line: generate tokens from a model folder.

    python -m mercury_b200.generate --model DIR --prompt-ids 1,2,3 --max-tokens 16

The engine options carry the reference server's names and meanings
(mercury/server.py:249-284: --model --device --dtype --policy --block-size --num-blocks
--max-running --prefill-budget --max-model-len --aging-tokens-per-s --max-wait-s
--scan-limit --cryptographic-hashes --debug-invariants --seed); the reference has no
offline command, so the prompt and sampling options are this program's own. Token ids go
in and token ids come out; one JSON line per prompt.

`--random-weights CONFIG.json` first writes a model folder with seeded random weights
into --model (which must not hold a model yet) and then generates from it.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .config import EngineConfig, autosize_blocks, config_from_dict
from .engine import Engine
from .sampling import SamplingParams


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("mercury_b200.generate")
    p.add_argument("--model", required=True, help="folder with config.json and safetensors")
    p.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                   help="write seeded random weights for this config.json into --model first")
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="comma-separated token ids; repeat for several prompts")
    p.add_argument("--prompt-file", default=None, help="one prompt per line, ids separated by spaces or commas")
    p.add_argument("--max-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--device", default="cuda")
    p.add_argument("--dtype", default="bfloat16", help="bfloat16 or float32")
    p.add_argument("--policy", default="fcfs", choices=("fcfs", "lpm", "lpm_aging"))
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--num-blocks", type=int, default=4096, help="-1 sizes to free memory")
    p.add_argument("--max-running", type=int, default=64)
    p.add_argument("--prefill-budget", type=int, default=8192)
    p.add_argument("--max-batched-tokens", type=int, default=8192)
    p.add_argument("--prefill-chunk", type=int, default=2048)
    p.add_argument("--max-model-len", type=int, default=8192)
    p.add_argument("--aging-tokens-per-s", type=float, default=2000.0)
    p.add_argument("--max-wait-s", type=float, default=5.0)
    p.add_argument("--scan-limit", type=int, default=128)
    p.add_argument("--no-prefix-caching", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--no-lookahead", action="store_true",
                   help="read every step's tokens before the next step is launched")
    p.add_argument("--cryptographic-hashes", action="store_true")
    p.add_argument("--debug-invariants", action="store_true")
    p.add_argument("--debug-poison-pages", action="store_true",
                   help="fill cache pages with NaN whenever they change hands")
    p.add_argument("--time-kernels", action="store_true",
                   help="time every class of kernel call with CUDA events (steps run eagerly) "
                        "and print the sums to stderr")
    p.add_argument("--seed", type=int, default=0)
    return p


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    folder = Path(args.model)
    if args.random_weights:
        from .weights import write_random_model

        if (folder / "config.json").exists():
            raise SystemExit(f"{folder} already holds a model; --random-weights will not overwrite it")
        _entry, config = config_from_dict(json.loads(Path(args.random_weights).read_text()))
        write_random_model(folder, config, args.seed)
    prompts = [_parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        prompts += [_parse_ids(line) for line in Path(args.prompt_file).read_text().splitlines()
                    if line.strip()]
    if not prompts:
        raise SystemExit("no prompt: give --prompt-ids or --prompt-file")

    cfg = EngineConfig(
        model=str(folder), device=args.device, dtype=args.dtype, block_size=args.block_size,
        num_blocks=args.num_blocks if args.num_blocks > 0 else 1, max_running=args.max_running,
        prefill_budget=args.prefill_budget, max_batched_tokens=args.max_batched_tokens,
        prefill_chunk=args.prefill_chunk, max_model_len=args.max_model_len, policy=args.policy,
        aging_tokens_per_s=args.aging_tokens_per_s, max_wait_s=args.max_wait_s,
        scan_limit=args.scan_limit, prefix_caching=not args.no_prefix_caching,
        cuda_graphs=not args.no_cuda_graphs, lookahead=not args.no_lookahead, cryptographic_hashes=args.cryptographic_hashes,
        debug_invariants=args.debug_invariants, debug_poison_pages=args.debug_poison_pages,
        time_kernels=args.time_kernels, seed=args.seed)
    if args.num_blocks < 0:
        from .engine.runner import kv_bytes_per_token_of

        weights = sum(f.stat().st_size for f in folder.glob("*.safetensors"))
        cfg.num_blocks = autosize_blocks(kv_bytes_per_token_of(folder, cfg.torch_dtype), cfg,
                                         reserve_bytes=weights)
        print(f"[mercury_b200] autosized to {cfg.num_blocks} pages", file=sys.stderr, flush=True)
    longest = max(len(p) for p in prompts) + args.max_tokens
    cfg.max_model_len = min(cfg.max_model_len, max(longest, cfg.block_size))
    if cfg.kv_capacity_tokens < cfg.max_model_len:
        raise SystemExit(f"--num-blocks {cfg.num_blocks} x --block-size {cfg.block_size} holds fewer "
                         f"tokens than one request needs ({cfg.max_model_len})")
    engine = Engine(cfg)
    # no per-request seed: each request then draws from a stream of its own, derived from
    # the engine's seed (--seed) and the request's name
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p,
                            ignore_eos=args.ignore_eos, seed=None)
    outs = engine.generate(prompts, params, args.max_tokens)
    for prompt, out in zip(prompts, outs):
        print(json.dumps({"prompt_tokens": len(prompt), "output_ids": out}), flush=True)
    if args.time_kernels:
        print(json.dumps({"kernel_ms": engine.metrics.summary().get("kernel_ms", {})}),
              file=sys.stderr, flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
