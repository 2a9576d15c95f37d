"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl mercury_b200|reference]

The default run has the layer sizes of Qwen2.5-0.5B (24 layers, hidden 896, 14 query heads,
2 KV heads of 64, feed-forward 4864, vocabulary 151936, tied head) with seeded random
weights in bfloat16, pages of 16 tokens, a model length of 4096, and decodes a batch of 8
requests whose contexts hold 2048 tokens. One "step" is one decode step of the whole batch.

It prints ONE JSON line:
  value      decoded tokens per second, timed on the device with CUDA events over K steps
             issued back to back (after W warm-up steps); the block of K steps is timed five
             times and the median block gives `value` and `ms_per_step` (`repeats` holds the
             minimum, median and maximum);
  e2e        the same through `Engine.step()`: every step copies its inputs from pinned host
             memory, samples on the device and reads the tokens back to the host;
  prefill    one 2048-token prompt in one step: tokens/s, ms, and flops / time / peak;
             `prefill_512x4` is the same prompt in four portions of 512;
  roofline   for the decode step: bytes it has to read (every weight once, the cache of
             the live requests) / time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64, `point_rooflines` their fractions;
  kernels    per class of kernel call, for the decode step and for the prompt step: the
             milliseconds it takes (CUDA events around every call of a step launched eagerly
             behind a device-side delay, so that the launches queue up), what the model needs
             of it (bytes to read, or flops) and that over time over the measured peak.
Weights (about 1 GB) are far larger than the 126 MB L2, so every step streams them from
HBM again; no extra L2 flush is needed ("l2" in config says so).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 24, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 32768,
}
SIZES = {
    "0.5b": QWEN25_05B,
    "1.5b": {**QWEN25_05B, "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12,
             "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960},
    "7b": {**QWEN25_05B, "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28,
           "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
           "vocab_size": 152064, "tie_word_embeddings": False},
}
BATCH = 8
CONTEXT = 2048        # tokens each request holds when decoding starts
MODEL_LEN = 4096      # benchmark context length: the most a request may reach
PREFILL_TOKENS = 2048
BLOCK = 16
SEED = 0
REPEATS = 5           # how often the block of K decode steps is timed
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
METRIC = "decode tok/s at batch 8 (Qwen2.5-0.5B sizes, 2048-token contexts)"


def bench_config(peak_kind: str) -> dict:
    """The `config` of the JSON line: every size of the run, flat; the same for both arms."""
    c = QWEN25_05B
    return {"model": "Qwen2.5-0.5B sizes", "layers": c["num_hidden_layers"],
            "layers_of_model": c["num_hidden_layers"], "hidden": c["hidden_size"],
            "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
            "head_dim": c["head_dim"], "intermediate": c["intermediate_size"],
            "vocab": c["vocab_size"], "tied": c["tie_word_embeddings"], "global_batch": BATCH,
            "seq_len": CONTEXT, "max_model_len": MODEL_LEN, "kv_block": BLOCK,
            "parallelism": "single GPU", "l2": "inputs>L2 (1 GB of weights streamed per step)",
            "peaks": peak_kind}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        raw = json.loads(path.read_text())
        out = dict(FALLBACK_PEAKS)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if isinstance(raw.get(key), (int, float)):
                out[key] = float(raw[key])
        return out, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while a timed region runs."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None

    def stop(self, window: tuple[float, float] | None = None) -> dict:
        """Median SM clock and the throttle reasons seen; with `window` (start, end in
        time.time() seconds) only the samples taken inside it count."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        self.proc.wait()
        import datetime

        clocks, top, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7 or not parts[1].isdigit():
                continue
            if window is not None:
                try:
                    stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    continue
                if not window[0] <= stamp <= window[1]:
                    continue
            clocks.append(int(parts[1]))
            top = int(parts[2]) if parts[2].isdigit() else top
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": top,
                "reasons": sorted(reasons), "samples": len(clocks)}


def class_costs(cfg: dict, batch: int, context: int, tokens: int) -> dict:
    """What each class of kernel call has to move or compute: for a decode step of `batch`
    requests at `context` tokens ("decode": bytes read) and for a prompt step of `tokens`
    tokens ("prefill": flops, or bytes for the classes that only move data)."""
    h, i, v, layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (n_q + 2 * n_kv) * d
    kv_layer = 2 * n_kv * d * 2                   # bytes of keys and values per token and layer
    decode = {
        "q/k/v product": ("hbm", layers * 2 * (qkv * h + qkv)),
        "q/k/v + rotary + store": ("hbm", layers * 2 * (qkv * h + qkv)),
        "attention": ("hbm", layers * batch * context * kv_layer),
        "residual product": ("hbm", layers * 2 * (n_q * d * h + h * i)),
        "gated product": ("hbm", layers * 2 * 2 * i * h),
        "product": ("hbm", 2 * v * h),
        "norm": ("hbm", 2 * batch * h * 6),
        "embedding": ("hbm", batch * h * 6),
        "sampling": ("hbm", batch * v * 4),
    }
    t = tokens
    prefill = {
        "q/k/v product": ("tensor", layers * 2 * t * qkv * h),
        "q/k/v + rotary + store": ("tensor", layers * 2 * t * qkv * h),
        "rotary + store": ("hbm", layers * t * (2 * qkv * 2 + 2 * n_kv * d * 2)),
        "attention": ("tensor", 2 * t * t * n_q * d * layers),
        "residual product": ("tensor", layers * 2 * t * (n_q * d * h + h * i)),
        "gated product": ("tensor", layers * 2 * t * 2 * i * h),
        "gate": ("hbm", layers * t * 3 * i * 2),
        "product": ("hbm", 2 * v * h),
        # every norm reads the float32 stream and a bfloat16 delta, writes both back
        "norm": ("hbm", (2 * layers + 1) * t * h * (4 + 2 + 4 + 2)),
        "embedding": ("hbm", t * h * 6),
    }
    return {"decode": decode, "prefill": prefill}


def model_numbers(cfg: dict) -> dict:
    """Bytes a decode step must read and flops a prefill must do, from the sizes alone."""
    h, i, v, layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (n_q + 2 * n_kv) * d
    per_layer = qkv * h + qkv + n_q * d * h + 2 * i * h + h * i + 2 * h
    head = v * h
    params_read = layers * per_layer + head + h   # tied table read once by the head
    if not cfg["tie_word_embeddings"]:
        pass  # the embedding table is only gathered from, not streamed
    kv_per_token = 2 * layers * n_kv * d * 2
    gemm_flops_per_token = 2 * layers * (qkv * h + n_q * d * h + 3 * i * h)
    return {"weight_bytes": 2 * params_read, "kv_bytes_per_token": kv_per_token,
            "gemm_flops_per_token": gemm_flops_per_token,
            "attn_flops": lambda t: 2 * t * t * n_q * d * layers, "head_flops_per_row": 2 * head}


def make_runner(torch, config, tensors, batch, page_tokens, graphs=True, gemm=None):
    from mercury_b200.engine.runner import ModelRunner
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda", gemm=gemm) if gemm else None
    return ModelRunner(config=config, tensors=tensors, dtype=torch.bfloat16, device="cuda",
                       page_size=BLOCK, num_pages=page_tokens // BLOCK, max_seqs=batch,
                       max_step_tokens=max(PREFILL_TOKENS, batch), max_model_len=MODEL_LEN,
                       cuda_graphs=graphs, ops=ops)


def timed(torch, fn, reps: int) -> float:
    """Milliseconds per call of fn over `reps` calls, by CUDA events."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def fill_contexts(torch, runner, batch, context, vocab):
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 1)
    seqs = []
    for b in range(batch):
        seq = runner.open(f"bench-{b}")
        tokens = torch.randint(0, vocab, (context,), generator=gen).tolist()
        for at in range(0, context, PREFILL_TOKENS):
            runner.step([StepEntry(seq, tokens[at:at + PREFILL_TOKENS], [])])
        seqs.append(seq)
    torch.cuda.synchronize()
    return seqs


def decode_rate(torch, runner, batch, context, vocab, steps, warmup, load_window=None, repeats=1):
    """(tokens/s, ms per step, launches per step, [ms per step of every repeat]) of `steps`
    decode steps of `batch`, timed `repeats` times in a row (the median repeat counts). With
    `load_window` (a list) the same steps keep running, untimed, until a second has passed
    since the timed region began, and [start, end] of that stretch is appended: the clock
    sampler needs more than the few dozen milliseconds the timed steps take."""
    from mercury_b200.engine.batch import StepEntry

    seqs = fill_contexts(torch, runner, batch, context, vocab)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    gen = torch.Generator().manual_seed(SEED + 2)
    feed = torch.randint(0, vocab, (steps * repeats + warmup + 1, batch), generator=gen).tolist()
    turn = [0]

    def one():
        tokens = feed[turn[0]]
        turn[0] += 1
        logits = runner.step([StepEntry(s, [tokens[i]], [0]) for i, s in enumerate(seqs)])
        runner.ops.argmax(logits, out)

    if load_window is not None:
        feed += feed * (int(1.2 / 0.0005) // len(feed) + 1)
    for _ in range(warmup):
        one()
    before = runner.launch_count()
    began = time.time()
    samples = [timed(torch, one, steps) for _ in range(repeats)]
    ms = statistics.median(samples)
    launches = (runner.launch_count() - before) / (steps * repeats)
    if load_window is not None:
        while time.time() - began < 1.0 and turn[0] < len(feed) - 1 and \
                seqs[0].num_computed + 2 < runner.max_model_len:
            one()
        torch.cuda.synchronize()
        load_window.extend([began, time.time()])
    for s in seqs:
        runner.close(s)
    return batch * 1e3 / ms, ms, launches, samples


def kernel_classes(torch, runner, batch, context, vocab, cfg, peak) -> dict:
    """Milliseconds per class of kernel call of one decode step of `batch` requests and of
    one prompt step, each launched eagerly with CUDA events around every call; a delay on
    the device lets the launches queue up first, so that the events see kernels back to
    back and not the host's launch loop. Beside each: what the model needs of the class
    (bytes or flops), and that over time over the measured peak."""
    from mercury_b200.engine.batch import StepEntry

    costs = class_costs(cfg, batch, context, PREFILL_TOKENS)
    out = {}
    seqs = fill_contexts(torch, runner, batch, context, vocab)
    gen = torch.Generator().manual_seed(SEED + 6)
    tokens = torch.randint(0, vocab, (8, batch), generator=gen).tolist()
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    sampled = torch.empty(batch, dtype=torch.int32, device="cuda")
    runner.time_kernels = True
    try:
        rows = []
        for turn in range(4):                      # the first two are warm-up
            torch.cuda._sleep(20_000_000)          # about 10 ms: the step's launches queue up behind it
            logits = runner.step([StepEntry(s, [tokens[turn][i]], [0]) for i, s in enumerate(seqs)])
            rows.append(dict(runner.last_kernel_ms))
        decode = {k: statistics.median(r.get(k, 0.0) for r in rows[2:]) for k in rows[-1]}
        torch.cuda._sleep(20_000_000)
        runner.ops.begin_timing()
        runner.ops.argmax(logits, sampled)
        decode["sampling"] = runner.ops.end_timing().get("sampling", 0.0)
        for s in seqs:
            runner.close(s)
        rows = []
        for turn in range(3):
            seq = runner.open(f"classes-{turn}")
            torch.cuda._sleep(40_000_000)
            runner.step([StepEntry(seq, prompt, [PREFILL_TOKENS - 1])])
            rows.append(dict(runner.last_kernel_ms))
            runner.close(seq)
        prefill = {k: statistics.median(r.get(k, 0.0) for r in rows[1:]) for k in rows[-1]}
    finally:
        runner.time_kernels = False
    for name, measured in (("decode", decode), ("prefill", prefill)):
        block = {}
        for kind, ms in sorted(measured.items()):
            bound, amount = costs[name].get(kind, ("hbm", 0))
            top = peak["hbm_gbs"] * 1e9 if bound == "hbm" else peak["bf16_tflops"] * 1e12
            block[kind] = {"ms": round(ms, 4), "bound": bound,
                           "frac": round(amount / (ms * 1e-3) / top, 4) if ms > 0 and amount else None}
        block["sum_ms"] = round(sum(measured.values()), 4)
        out[name] = block
    return out


def prefill_rate(torch, runner, vocab, reps=5):
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 3)
    tokens = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for rep in range(reps + 2):
        seq = runner.open(f"prefill-{rep}")
        ms = timed(torch, lambda: runner.step([StepEntry(seq, tokens, [PREFILL_TOKENS - 1])]), 1)
        runner.close(seq)
        if rep >= 2:
            times.append(ms)
    return statistics.median(times)


def prefill_portions_rate(torch, runner, vocab, portion=512, reps=5):
    """The 2048-token prompt as portions of `portion` tokens, one step each; ms for all."""
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 3)
    tokens = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []

    def run(seq):
        for at in range(0, PREFILL_TOKENS, portion):
            last = at + portion >= PREFILL_TOKENS
            runner.step([StepEntry(seq, tokens[at:at + portion], [portion - 1] if last else [])])

    for rep in range(reps + 2):
        seq = runner.open(f"portions-{rep}")
        ms = timed(torch, lambda: run(seq), 1)
        runner.close(seq)
        if rep >= 2:
            times.append(ms)
    return statistics.median(times)


def e2e_rate(torch, config, tensors, batch, context, vocab, steps, warmup):
    """Decode tokens/s through Engine.step(): host tokens in, host tokens out."""
    from mercury_b200 import Engine, EngineConfig, SamplingParams
    runner = make_runner(torch, config, tensors, batch, batch * (context + 256))
    cfg = EngineConfig(model="(in memory)", dtype="bfloat16", block_size=BLOCK,
                       num_blocks=runner.cache.pools[0].num_pages, max_running=batch,
                       max_batched_tokens=max(PREFILL_TOKENS, batch), prefill_chunk=PREFILL_TOKENS,
                       max_model_len=MODEL_LEN, prefix_caching=False, seed=SEED)
    engine = Engine(cfg, runner=runner)
    gen = torch.Generator().manual_seed(SEED + 4)
    produced = []
    started = set()

    def sink(event):
        produced.append(event.kind)
        started.add(event.rid)

    for b in range(batch):
        prompt = torch.randint(0, vocab, (context,), generator=gen).tolist()
        engine.submit(f"e2e-{b}", prompt, steps + warmup + batch + 8, sink,
                      SamplingParams(ignore_eos=True))
    while len(started) < batch:          # prompts first: until every request decodes
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    size_before = len(produced)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    tokens = sum(1 for kind in produced[size_before:] if kind == "token")
    assert tokens == batch * steps, (tokens, batch, steps)
    lay = runner.buffers._layout(batch, batch, -(-(context + steps + warmup + batch + 8) // BLOCK), batch)
    return tokens / seconds, lay["size"] * 4, batch * 4


def other_sizes(torch, args) -> dict:
    """The side workloads of the benchmark description, one flat block: decode at batch 8 and
    the 2048-token prompt at Qwen2.5-1.5B and 7B sizes (all their layers, random weights), and
    the mixed serving workload at 1.5B sizes. A size that fails says so and does not take the
    line with it."""
    from types import SimpleNamespace

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    out = {}
    for name in ("1.5b", "7b"):
        try:
            raw = SIZES[name]
            _entry, config = config_from_dict(raw)
            tensors = random_tensors(config, SEED, torch.bfloat16)
            runner = make_runner(torch, config, tensors, BATCH, BATCH * (CONTEXT + 256))
            steps = min(args.steps, 32)
            rate, ms, _l, _s = decode_rate(torch, runner, BATCH, CONTEXT, raw["vocab_size"], steps,
                                           max(3, min(args.warmup, 8)))
            out[f"{name}_decode_b8"] = round(rate, 1)
            out[f"{name}_decode_ms"] = round(ms, 4)
            out[f"{name}_prefill_ms"] = round(prefill_rate(torch, runner, raw["vocab_size"], reps=3), 3)
            out[f"{name}_layers"] = raw["num_hidden_layers"]
            del runner
            torch.cuda.empty_cache()
            if name == "1.5b":
                mixed = run_mixed(SimpleNamespace(size=name, policy="lpm"), prepared=(config, tensors))
                out["1.5b_mixed_output_tokens_per_s"] = mixed["output_tokens_per_s"]
                out["1.5b_mixed_prefix_hit_tokens"] = mixed["prefix_hit_tokens"]
                out["1.5b_mixed_requests"] = 32
            del tensors
            torch.cuda.empty_cache()
        except Exception as exc:      # a side workload must not cost the headline its line
            out[f"{name}_error"] = f"{type(exc).__name__}: {exc}"[:200]
    return out


def run_ours(args) -> dict:
    import torch

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    peak, peak_kind = peaks()
    _entry, config = config_from_dict(QWEN25_05B)
    tensors = random_tensors(config, SEED, torch.bfloat16)
    vocab = QWEN25_05B["vocab_size"]
    numbers = model_numbers(QWEN25_05B)

    sampler = ClockSampler()
    sampler.start()
    runner = make_runner(torch, config, tensors, 64, 64 * (CONTEXT + 256))
    window: list[float] = []
    value, ms, launches, samples = decode_rate(torch, runner, BATCH, CONTEXT, vocab, args.steps,
                                               args.warmup, load_window=window, repeats=REPEATS)
    clocks = sampler.stop(tuple(window))
    b1, ms1, _, _ = decode_rate(torch, runner, 1, CONTEXT, vocab, args.steps, args.warmup, repeats=3)
    b64, ms64, _, _ = decode_rate(torch, runner, 64, CONTEXT, vocab, args.steps, args.warmup, repeats=3)
    prefill_ms = prefill_rate(torch, runner, vocab)
    portions_ms = prefill_portions_rate(torch, runner, vocab)
    kernels = kernel_classes(torch, runner, BATCH, CONTEXT, vocab, QWEN25_05B, peak)
    del runner
    torch.cuda.empty_cache()
    e2e, h2d, d2h = e2e_rate(torch, config, tensors, BATCH, CONTEXT, vocab, args.steps, args.warmup)
    del tensors
    torch.cuda.empty_cache()
    sizes = {} if args.no_sizes else other_sizes(torch, args)

    def step_bytes(batch, steps_before):
        return numbers["weight_bytes"] + batch * (CONTEXT + steps_before) * numbers["kv_bytes_per_token"]

    def fraction(batch, step_ms, steps_before):
        return round(step_bytes(batch, steps_before) / (step_ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)

    middle = args.warmup + REPEATS * args.steps // 2
    achieved = step_bytes(BATCH, middle) / (ms * 1e-3) / 1e9
    flops = (PREFILL_TOKENS * numbers["gemm_flops_per_token"] + numbers["attn_flops"](PREFILL_TOKENS)
             + numbers["head_flops_per_row"])
    return {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random N(0,0.02) weights",
        "config": bench_config(peak_kind),
        "repeats": {"n": REPEATS, "ms_min": round(min(samples), 4),
                    "ms_median": round(statistics.median(samples), 4), "ms_max": round(max(samples), 4)},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "prefill_512x4": {"value": round(PREFILL_TOKENS * 1e3 / portions_ms, 1),
                          "tokens": PREFILL_TOKENS, "ms": round(portions_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)},
        "point_rooflines": {"decode_b1": {"ms": round(ms1, 4), "frac": fraction(1, ms1, args.warmup + 3 * args.steps // 2)},
                            "decode_b64": {"ms": round(ms64, 4), "frac": fraction(64, ms64, args.warmup + 3 * args.steps // 2)}},
        "kernels": kernels,
        "sizes": sizes,
        "clocks": clocks,
    }


def run_part(args) -> dict:
    """`--only decode|prefill|products`: one small workload for profilers, with the same
    model, weights and shapes as the full run. Prints what it measured, not the bench line."""
    import torch

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    if args.only == "mixed":
        return run_mixed(args)
    raw = SIZES[args.size]
    _entry, config = config_from_dict(raw)
    vocab = raw["vocab_size"]
    if args.only == "products":
        from types import SimpleNamespace

        from mercury_b200.kernels.ops import CudaOps

        def replayed(fn, calls=10):
            """Microseconds per call of fn, `calls` of them replayed from a CUDA graph: the
            device's time without the host's share (a product of a few microseconds is
            launched more slowly than it runs)."""
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(calls):
                    fn()
            graph.replay()
            return timed(torch, graph.replay, max(args.steps, 3)) / calls * 1e3

        out = {}
        for name, (m, n, k) in {"qkv": (2048, 1152, 896), "o": (2048, 896, 896),
                                "gate_up": (2048, 9728, 896), "down": (2048, 896, 4864),
                                "qkv_7b": (2048, 4608, 3584), "down_7b": (2048, 3584, 18944)}.items():
            x = torch.randn(m, k).bfloat16().cuda()
            w = torch.randn(n, k).bfloat16().cuda()
            y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            for gemm in ("library", "tcgen05"):
                ops = CudaOps("cuda", gemm=gemm)
                us = replayed(lambda: ops.linear(x, w, None, y))
                ops.check_errors()
                out[f"{name}_{gemm}_us"] = round(us, 1)
                out[f"{name}_{gemm}_tflops"] = round(2 * m * n * k / us / 1e6, 1)
            ops = CudaOps("cuda")
            error = torch.zeros(1, dtype=torch.int32, device="cuda")
            stream = torch.cuda.current_stream

            def pairs():
                assert ops.lib.mb_gemm_pair(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 0, m, n, k,
                                            None, 0, 0.0, 0, None, None, None, None, error.data_ptr(),
                                            stream().cuda_stream) == 0
            us = replayed(pairs)
            assert int(error.item()) == 0
            out[f"{name}_pairs_us"] = round(us, 1)
            out[f"{name}_pairs_tflops"] = round(2 * m * n * k / us / 1e6, 1)
        # the gated product: gate/up with the SiLU gate in the epilogue, one CTA per tile against
        # pairs of CTAs, and the library's product followed by the gate kernel
        for name, (m, width, k) in {"gated_0.5b": (2048, 4864, 896), "gated_1.5b": (2048, 8960, 1536),
                                    "gated_7b": (2048, 18944, 3584)}.items():
            x = torch.randn(m, k).bfloat16().cuda()
            w = (torch.randn(2 * width, k) * 0.05).bfloat16().cuda()
            y = torch.empty(m, width, dtype=torch.bfloat16, device="cuda")
            both = torch.empty(m, 2 * width, dtype=torch.bfloat16, device="cuda")
            ctx = SimpleNamespace(buffer=lambda *_a, **_k: both)
            for label, gemm, min_k in (("one_cta", "auto", 1 << 30), ("pairs", "auto", 0),
                                       ("library_and_gate", "library", 0)):
                ops = CudaOps("cuda", gemm=gemm)
                ops.pair_min_k = min_k
                ops.gated_max_elements = 1 << 40
                us = replayed(lambda: ops.linear_swiglu(x, w, y, ctx))
                ops.check_errors()
                out[f"{name}_{label}_us"] = round(us, 1)
                out[f"{name}_{label}_tflops"] = round(4 * m * width * k / us / 1e6, 1)
        return out
    tensors = random_tensors(config, SEED, torch.bfloat16)
    batch = args.batch
    runner = make_runner(torch, config, tensors, max(batch, 2), max(batch, 2) * (CONTEXT + 256),
                         graphs=not args.no_graphs, gemm=args.gemm)
    if args.only == "prefill":
        return {"prefill_ms": round(prefill_rate(torch, runner, vocab, reps=args.steps), 3)}
    if args.only == "kernels":
        return kernel_classes(torch, runner, batch, CONTEXT, vocab, raw, peaks()[0])
    rate, ms, launches, _samples = decode_rate(torch, runner, batch, CONTEXT, vocab, args.steps,
                                               args.warmup)
    return {"decode_tokens_per_s": round(rate, 1), "ms_per_step": round(ms, 4), "batch": batch,
            "launches_per_step": launches, "graphs": not args.no_graphs}


def run_mixed(args, prepared=None) -> dict:
    """`--only mixed`: 32 requests through Engine.generate, prompt lengths uniform in
    [64, 2048], half of them sharing one 512-token prefix, 128 greedy tokens each (the
    benchmark description's serving workload, by default at Qwen2.5-1.5B sizes)."""
    import torch

    from mercury_b200 import Engine, EngineConfig, SamplingParams
    from mercury_b200.config import config_from_dict
    from mercury_b200.engine.runner import ModelRunner
    from mercury_b200.weights import random_tensors

    raw = SIZES[args.size]
    if prepared is None:
        _entry, config = config_from_dict(raw)
        tensors = random_tensors(config, SEED, torch.bfloat16)
    else:
        config, tensors = prepared
    gen = torch.Generator().manual_seed(SEED + 5)
    shared = torch.randint(0, raw["vocab_size"], (512,), generator=gen).tolist()
    prompts = []
    for i in range(32):
        n = int(torch.randint(64, 2049, (1,), generator=gen))
        body = torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist()
        prompts.append((shared + body[512:]) if (i % 2 == 0 and n > 512) else body)
    pool_tokens = 32 * (2048 + 128 + BLOCK)
    runner = ModelRunner(config=config, tensors=tensors, dtype=torch.bfloat16, device="cuda",
                         page_size=BLOCK, num_pages=pool_tokens // BLOCK, max_seqs=32,
                         max_step_tokens=4096, max_model_len=MODEL_LEN)
    cfg = EngineConfig(model="(in memory)", dtype="bfloat16", block_size=BLOCK,
                       num_blocks=pool_tokens // BLOCK, max_running=32, max_batched_tokens=4096,
                       prefill_chunk=2048, max_model_len=MODEL_LEN, policy=args.policy, seed=SEED)
    engine = Engine(cfg, runner=runner)
    engine.generate([prompts[0][:64]], SamplingParams(ignore_eos=True), 4)      # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, SamplingParams(ignore_eos=True), 128)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    produced = sum(len(o) for o in outs)
    snap = engine.snapshot()
    return {"workload": "mixed: 32 requests, prompts 64..2048, 16 share a 512-token prefix, 128 tokens each",
            "size": args.size, "policy": args.policy, "output_tokens": produced,
            "prompt_tokens": sum(len(p) for p in prompts), "seconds": round(seconds, 3),
            "output_tokens_per_s": round(produced / seconds, 1),
            "prefix_hit_tokens": snap["cache"]["hit_tokens"], "steps": snap["engine"]["steps"],
            "preemptions": snap["scheduler"]["preemptions"], "leaked_pages": engine.leaked_pages()}


def run_reference(args) -> dict:
    """The unmodified reference (installed under baseline/_ref) on the same model folder,
    batch and context, through its own Engine.submit/step."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "mercury").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}
    try:
        import torch

        from mercury_b200.config import config_from_dict
        from mercury_b200.weights import write_random_model

        sys.path.insert(0, str(ref))
        from mercury.config import EngineConfig as RefConfig
        from mercury.engine import Engine as RefEngine
        from mercury.request import SamplingParams as RefParams
    except Exception as err:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import failed: {type(err).__name__}: {err}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device on this box"}
    try:
        return _time_reference(args, torch, config_from_dict, write_random_model, RefConfig,
                               RefEngine, RefParams)
    except Exception as err:  # noqa: BLE001
        return {"impl": "reference",
                "unavailable": " ".join(f"the reference failed while running: "
                                        f"{type(err).__name__}: {err}".split())[:300]}


def _time_reference(args, torch, config_from_dict, write_random_model, RefConfig, RefEngine,
                    RefParams) -> dict:
    _entry, config = config_from_dict(QWEN25_05B)
    vocab = QWEN25_05B["vocab_size"]
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(Path(tmp) / "model", config, SEED)
        cfg = RefConfig(model=str(folder), device="cuda", dtype="bfloat16", block_size=BLOCK,
                        num_blocks=BATCH * (CONTEXT + 256) // BLOCK, max_running=BATCH,
                        max_model_len=MODEL_LEN, prefill_budget=BATCH * CONTEXT, seed=SEED)
        engine = RefEngine(cfg)
        gen = torch.Generator().manual_seed(SEED + 4)
        produced = []
        for b in range(BATCH):
            prompt = torch.randint(0, vocab, (CONTEXT,), generator=gen).tolist()
            engine.submit(f"ref-{b}", prompt, args.steps + args.warmup + 8,
                          lambda ev: produced.append(ev.kind), RefParams(ignore_eos=True))
        engine.step()                       # admits and prefills every prompt
        for _ in range(args.warmup):
            engine.step()
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        before = len(produced)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        clocks = sampler.stop()
        tokens = sum(1 for kind in produced[before:] if kind == "token")
    rate = round(tokens / seconds, 1)
    return {"impl": "reference", "metric": METRIC,
            "value": rate, "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(1e3 * seconds / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random N(0,0.02) weights",
            "config": bench_config(peaks()[1]),
            # the reference has no device-timed number: its only clock is the wall clock around
            # its own Engine.step, host tokens in and out, which is an end-to-end number by
            # nature; the bytes it copies per step are its own business and not counted here
            "timing": "wall clock around Engine.step, host tokens in and out",
            "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": None,
                    "d2h_bytes_per_step": None},
            "clocks": clocks}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="mercury_b200", choices=("mercury_b200", "reference"))
    p.add_argument("--only", default="all",
                   choices=("all", "decode", "prefill", "products", "mixed", "kernels"),
                   help="run one part only (for profilers and side workloads); prints its own JSON")
    p.add_argument("--size", default=None, choices=tuple(SIZES),
                   help="layer sizes of --only decode/prefill/mixed (default 0.5b; mixed: 1.5b)")
    p.add_argument("--policy", default="lpm", choices=("fcfs", "lpm", "lpm_aging"))
    p.add_argument("--batch", type=int, default=BATCH, help="decode batch of --only decode")
    p.add_argument("--no-graphs", action="store_true", help="launch kernels one by one")
    p.add_argument("--no-sizes", action="store_true",
                   help="leave the 1.5B and 7B side workloads out of the full run (about a minute)")
    p.add_argument("--gemm", default=None, choices=("library", "tcgen05", "auto"),
                   help="many-token product of --only prefill/decode (default: the engine's)")
    args = p.parse_args()
    if args.gpus != 1:
        print("bench.py measures a single-GPU engine; --gpus must be 1", flush=True)
        return 2
    if args.size is None:
        args.size = "1.5b" if args.only == "mixed" else "0.5b"
    if args.only != "all":
        print(json.dumps(run_part(args)), flush=True)
        return 0
    args.warmup = max(3, args.warmup)
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
