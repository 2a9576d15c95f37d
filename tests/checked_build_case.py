"""Run by tests/test_aux_gpu.py in a process of its own with MERCURY_B200_BOUNDS_CHECK=1, so
that the checked variant of the kernel library is the one that loads. Prints one JSON line.

First a mixed replay of tiny model A in both precisions (every kernel of a step runs with
its checks and nothing may be reported), then single kernels fed one bad index each: a page
number beyond the pool, a block-table column beyond the table, a position beyond the
rotation tables, a token id outside the vocabulary. The tensors behind the pool and the
tables are larger than the limits say, so even an unchecked access would stay inside
allocated memory."""

from __future__ import annotations

import json
import sys
from pathlib import Path
from types import SimpleNamespace

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import replay_cases  # noqa: E402
from replay_check import requests_for, run_and_check, sharpened_model  # noqa: E402
from mercury_b200.engine.runner import ModelRunner  # noqa: E402
from mercury_b200.kernels.library import KernelError  # noqa: E402
from mercury_b200.kernels.ops import CudaOps  # noqa: E402
from mercury_b200.parts.base import LayerCache  # noqa: E402


def main() -> None:
    out = {}
    ops = CudaOps("cuda")
    out["checked"] = ops.checked
    lengths = (37, 70, 129, 45)
    requests = requests_for("A", lengths)
    steps, rows = replay_cases.mixed(requests, 320, seed=2)
    for dtype in (torch.float32, torch.bfloat16):
        _raw, config, tensors = sharpened_model("A")
        runner = ModelRunner(config=config, tensors=tensors, dtype=dtype, device="cuda", page_size=16,
                             num_pages=20, max_seqs=4, max_step_tokens=320, max_model_len=320)
        assert not runner.use_graphs
        out[f"replay_{str(dtype).split('.')[-1]}"] = run_and_check(runner, "A", lengths, steps, rows, dtype)

    # ---- one bad index at a time
    n_q, n_kv, d, page, pool, big = 4, 2, 64, 16, 8, 16
    k_all = torch.zeros((big, n_kv, page, d), dtype=torch.bfloat16, device="cuda")
    v_all = torch.zeros_like(k_all)
    angles = torch.rand((128, d // 2)) * 6
    cos_all, sin_all = angles.cos().cuda(), angles.sin().cuda()
    tables = (cos_all[:64], sin_all[:64])           # the rotation tables "have" 64 rows

    def batch(position, table_row, width=4):
        dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        table = dev([table_row + [-1] * (width - len(table_row))])
        return SimpleNamespace(positions=dev([position]), seq_of_token=dev([0]), q_start=dev([0, 1]),
                               kv_len=dev([position + 1]), num_seqs=1, max_q_len=1,
                               max_kv_len=position + 1, attention_splits=None), table

    def attempt(what, position, table_row, tables=tables, width=4):
        b, table = batch(position, table_row, width)
        cache = LayerCache(k_all[:pool], v_all[:pool], page, table, True)
        qkv = torch.randn((1, (n_q + 2 * n_kv) * d), device="cuda").bfloat16()
        attended = torch.zeros((1, n_q * d), dtype=torch.bfloat16, device="cuda")
        ops.rope_cache_write(qkv, n_q, n_kv, d, tables, b, cache)
        ops.paged_attention(qkv, n_q, n_kv, d, b, cache, 0.125, 0, attended)
        try:
            ops.check_errors()
            out[what] = "not reported"
        except KernelError as err:
            out[what] = str(err)
        torch.cuda.synchronize()

    attempt("good", 20, [3, 5])
    attempt("page", 20, [3, pool + 2])               # page 10 of a pool of 8
    # position 70 needs column 4 of a table of 4 (the rotation tables here have 128 rows)
    attempt("column", 70, [3, 5, 1, 2], tables=(cos_all, sin_all))
    # row 64 of rotation tables of 64 rows (the block table is wide enough)
    attempt("position", 64, [3, 5, 1, 2, 0], width=8)
    ids = torch.tensor([5, 1000], dtype=torch.int32, device="cuda")
    table = torch.randn((300, 32), device="cuda").bfloat16()
    h = torch.zeros((2, 32), dtype=torch.float32, device="cuda")
    ops.embed(ids, table, h)
    try:
        ops.check_errors()
        out["token"] = "not reported"
    except KernelError as err:
        out["token"] = str(err)
    attempt("good_again", 20, [3, 5])
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
