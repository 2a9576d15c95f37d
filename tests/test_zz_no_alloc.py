"""The attention entry point for callers that cannot allocate device memory.

Some users of the kernel library live inside a host program that owns all device memory
(or may not block on the allocator), so they cannot give the split-key attention kernel
the scratch buffer it needs. `mb_paged_attention_static` keeps that scratch in an array
inside the library. This test calls it through its exported C symbol, exactly as such a
caller would, twice in a row (the array is shared and keeps the first call's contents),
and compares each result with the ordinary entry point's. It also checks that a problem
larger than the built-in array is refused instead of run.

The file is named so that pytest collects it last.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_ARGS = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
               c_int, c_void_p]


def _case(seed, dtype, n_q=6, n_kv=2, d=64, page=16, kv_lens=(300, 77, 130), q_lens=(1, 1, 3)):
    gen = torch.Generator().manual_seed(seed)
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 3
    perm = torch.randperm(num_pages, generator=gen).tolist()
    max_pages = max(-(-kv // page) for kv in kv_lens)
    table = torch.full((len(kv_lens), max_pages), -1, dtype=torch.int32)
    seq_of, q_start = [], [0]
    for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
        for i in range(-(-kv // page)):
            table[s, i] = perm.pop()
        seq_of += [s] * q
        q_start.append(q_start[-1] + q)
    tokens = len(seq_of)
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    k = torch.randn((num_pages, n_kv, page, d), generator=gen).to(dtype).cuda()
    v = torch.randn((num_pages, n_kv, page, d), generator=gen).to(dtype).cuda()
    qkv = torch.randn((tokens, (n_q + 2 * n_kv) * d), generator=gen).to(dtype).cuda()
    return dict(qkv=qkv, k=k, v=v, table=table.cuda(), q_start=dev(q_start), kv_len=dev(list(kv_lens)),
                seq_of=dev(seq_of), tokens=tokens, seqs=len(kv_lens), max_q=max(q_lens), n_q=n_q,
                n_kv=n_kv, d=d, page=page)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from mercury_b200.kernels import library

    lib = library.load()
    static = lib.mb_paged_attention_static
    static.argtypes = STATIC_ARGS
    static.restype = c_int
    flag = 0 if dtype == torch.float32 else 1
    stream = torch.cuda.current_stream().cuda_stream
    splits = 4
    for call, seed in enumerate((11, 12)):          # two calls in a row share the array
        c = _case(seed, dtype)
        floats = lib.mb_attention_scratch_floats(c["tokens"], c["n_q"], c["d"], splits)
        scratch = torch.empty(floats, dtype=torch.float32, device="cuda")
        want = torch.zeros((c["tokens"], c["n_q"] * c["d"]), dtype=dtype, device="cuda")
        got = torch.zeros_like(want)
        common = (c["qkv"].data_ptr(), c["qkv"].shape[1], c["k"].data_ptr(), c["v"].data_ptr(),
                  c["table"].data_ptr(), c["table"].shape[1], c["q_start"].data_ptr(),
                  c["kv_len"].data_ptr(), c["seq_of"].data_ptr())
        sizes = (c["tokens"], c["seqs"], c["max_q"], c["n_q"], c["n_kv"], c["d"], c["page"],
                 c["d"] ** -0.5, 0, splits, flag, stream)
        rc = lib.mb_paged_attention_simt(*common, want.data_ptr(), scratch.data_ptr(), floats, *sizes)
        assert rc == 0
        rc = static(*common, got.data_ptr(), *sizes)
        assert rc == 0, f"call {call}: the static entry point returned {rc}"
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        tol = 2e-6 if dtype == torch.float32 else 5e-3
        err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert err <= tol, f"call {call}: differs from the ordinary entry point by {err:.2e}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from mercury_b200.kernels import library

    lib = library.load()
    static = lib.mb_paged_attention_static
    static.argtypes = STATIC_ARGS
    static.restype = c_int
    c = _case(13, torch.bfloat16)
    out = torch.zeros((c["tokens"], c["n_q"] * c["d"]), dtype=torch.bfloat16, device="cuda")
    # 4096 tokens x 64 heads x 64 splits x 66 floats is far beyond the 4 Mi floats built in
    rc = static(c["qkv"].data_ptr(), c["qkv"].shape[1], c["k"].data_ptr(), c["v"].data_ptr(),
                c["table"].data_ptr(), c["table"].shape[1], c["q_start"].data_ptr(),
                c["kv_len"].data_ptr(), c["seq_of"].data_ptr(), out.data_ptr(), 4096, c["seqs"],
                c["max_q"], 64, 2, 64, c["page"], 0.125, 0, 64, 1,
                torch.cuda.current_stream().cuda_stream)
    assert rc == 5, "a problem beyond the built-in scratch must be refused (MB_ERR_SCRATCH)"
    torch.cuda.synchronize()
