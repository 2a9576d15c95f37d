"""Each CUDA kernel alone against its plain PyTorch twin, at sizes other than the engine's:
widths and vocabularies that are no power of two, head sizes in steps of 16, odd numbers
of heads and groups, every page size, padding rows, pages given back."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from kernel_twins import TorchOps
from mercury_b200.parts.base import LayerCache

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def ops():
    from mercury_b200.kernels.ops import CudaOps

    return CudaOps("cuda")


@pytest.fixture(scope="module")
def twin():
    return TorchOps(exact=True)


def rand(shape, dtype, seed, scale=1.0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=gen) * scale).to(dtype).cuda()


def close(got, want, dtype, what="", terms=1):
    """float32: the same sum of `terms` products in another order, whose rounding grows
    like sqrt(terms) * 2^-24; bfloat16: one rounding of the result."""
    tol = max(2e-6, 2 * terms ** 0.5 * 2.0 ** -24) if dtype == torch.float32 else 5e-3
    scale = max(float(want.abs().max()), 1e-6)
    err = float((got.double() - want.double()).abs().max()) / scale
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.0e}"


# ------------------------------------------------------------------------------ embedding

@pytest.mark.parametrize("table_dtype", DTYPES, ids=IDS)
def test_embed(ops, twin, table_dtype):
    table = rand((1000, 200), table_dtype, 0)
    ids = torch.randint(0, 1000, (37,), dtype=torch.int32).cuda()
    got = torch.empty((37, 200), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    ops.embed(ids, table, got)
    twin.embed(ids, table, want)
    assert torch.equal(got, want)


# ------------------------------------------------------------------------------ norm

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("rows,cols", [(1, 896), (7, 1536), (64, 100), (1000, 896), (3, 4100),
                                       (259, 1536), (300, 2048), (257, 100), (2048, 3584)])
@pytest.mark.parametrize("with_delta", [True, False])
def test_add_rmsnorm(ops, twin, dtype, rows, cols, with_delta):
    h = rand((rows, cols), torch.float32, 1)
    delta = rand((rows, cols), dtype, 2) if with_delta else None
    weight = rand((cols,), dtype, 3) + 1
    h_want = h.clone()
    got = torch.empty((rows, cols), dtype=dtype, device="cuda")
    want = torch.empty_like(got)
    ops.add_rmsnorm(h, delta, weight, 1e-5, got)
    twin.add_rmsnorm(h_want, delta, weight, 1e-5, want)
    close(got, want, dtype, "normed")
    close(h, h_want, torch.float32, "residual")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_add_rmsnorm_selected_rows_and_wide_weight(ops, twin, dtype):
    h = rand((50, 330), torch.float32, 4)
    delta = rand((50, 330), dtype, 5)
    weight = rand((330,), torch.float32, 6) + 1     # a weight stored in 32-bit stays 32-bit
    rows = torch.tensor([49, 0, 17, 17, 3], dtype=torch.int32).cuda()
    before = h.clone()
    got = torch.empty((5, 330), dtype=dtype, device="cuda")
    want = torch.empty_like(got)
    ops.add_rmsnorm(h, delta, weight, 1e-6, got, rows)
    twin.add_rmsnorm(before.clone(), delta, weight, 1e-6, want, rows)
    close(got, want, dtype)
    assert torch.equal(h, before), "selected-row mode must leave the residual alone"


def test_add_rmsnorm_zero_row(ops):
    h = torch.zeros((2, 96), dtype=torch.float32, device="cuda")
    out = torch.empty((2, 96), dtype=torch.bfloat16, device="cuda")
    ops.add_rmsnorm(h, None, torch.ones(96, dtype=torch.bfloat16, device="cuda"), 1e-6, out)
    assert torch.count_nonzero(out) == 0


# ------------------------------------------------------------------------------ products

@pytest.mark.parametrize("m,n,k", [(1, 151, 70), (5, 130, 896), (77, 1152, 96), (130, 64, 4864),
                                   (64, 64, 16), (3, 1000, 1),
                                   # few tokens, K % 32 == 0, N % 16 == 0: the skinny kernels
                                   (1, 1152, 896), (8, 896, 4864), (16, 9728, 896), (33, 9728, 896),
                                   (9, 4112, 320), (13, 48, 96), (2, 151936, 64), (3, 896, 64)])
@pytest.mark.parametrize("x_dtype,w_dtype,o_dtype", [
    (torch.float32, torch.float32, torch.float32),
    (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.float32),
    (torch.bfloat16, torch.float32, torch.bfloat16),
], ids=["f32", "bf16", "bf16-f32out", "bf16-f32weight"])
def test_linear(ops, twin, m, n, k, x_dtype, w_dtype, o_dtype):
    x = rand((m, k), x_dtype, 7)
    w = rand((n, k), w_dtype, 8, 0.1)
    bias = rand((n,), w_dtype, 9) if n % 2 else None
    got = torch.empty((m, n), dtype=o_dtype, device="cuda")
    want = torch.empty_like(got)
    ops.linear(x, w, bias, got)
    twin.linear(x, w, bias, want)
    close(got, want, o_dtype, terms=k)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (2048, 1152, 896), (130, 200, 72), (300, 9728, 896),
                                   (17, 151936, 64), (1000, 896, 4864), (129, 257, 8)])
@pytest.mark.parametrize("tile", [1, 2], ids=["128x128", "128x256"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32], ids=["bf16out", "f32out"])
def test_tcgen05_product(twin, m, n, k, tile, out_dtype):
    """The TMA + tensor-memory kernel called directly, both tile shapes, edges in M, N and K."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 51)
    w = rand((n, k), torch.bfloat16, 52, 0.1)
    bias = rand((n,), torch.bfloat16, 53) if n % 2 else None
    got = torch.zeros((m, n), dtype=out_dtype, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mb_gemm_tcgen05(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                             got.data_ptr(), int(out_dtype == torch.float32), m, n, k,
                             error.data_ptr(), tile, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert int(error.item()) == 0, "a bounded wait in the kernel ran out"
    want = torch.empty_like(got)
    twin.linear(x, w, bias, want)
    close(got, want, out_dtype, terms=k)


@pytest.mark.parametrize("m", [256, 300, 2048, 2049])
@pytest.mark.parametrize("k", [896, 1536, 3584])
@pytest.mark.parametrize("width", [4864, 200], ids=["w4864", "w200"])
def test_tcgen05_persistent_gated_product(twin, m, k, width):
    """The persistent kernel with the SiLU gate in its epilogue, called directly at the
    prompt-step sizes that select it: full and ragged row tiles, one row beyond a tile,
    widths that are no multiple of its 128-column tiles, three lengths of the sum."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 71)
    w = rand((2 * width, k), torch.bfloat16, 72, 0.05)
    got = torch.zeros((m, width), dtype=torch.bfloat16, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mb_gemm_tcgen05_persistent(x.data_ptr(), w.data_ptr(), None, got.data_ptr(), 2, m, width,
                                        k, error.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert int(error.item()) == 0, "a bounded wait in the kernel ran out"
    gate = x.double() @ w[:width].double().T
    up = x.double() @ w[width:].double().T
    want = gate * torch.sigmoid(gate) * up
    # as the separate kernels do, gate and up are rounded to bfloat16 before the gate and the
    # result once more: three roundings of 2^-9 each at worst
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert err <= 3 * 2.0 ** -8, err
    # and every element relative to its own size (a swapped half or a stale accumulator
    # would pass neither)
    loose = (got.double() - want).abs() <= 2.0 ** -6 * want.abs() + 2e-3 * want.abs().max()
    assert bool(loose.all())


@pytest.mark.parametrize("mode,out_dtype", [(0, torch.bfloat16), (1, torch.float32)], ids=["bf16out", "f32out"])
@pytest.mark.parametrize("m,n,k", [(256, 1152, 896), (300, 896, 4864), (2049, 200, 1536)])
def test_tcgen05_persistent_plain_product(twin, m, n, k, mode, out_dtype):
    """The persistent kernel's plain modes (bias, bfloat16 or float32 out)."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 73)
    w = rand((n, k), torch.bfloat16, 74, 0.1)
    bias = rand((n,), torch.bfloat16, 75)
    got = torch.zeros((m, n), dtype=out_dtype, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mb_gemm_tcgen05_persistent(x.data_ptr(), w.data_ptr(), bias.data_ptr(), got.data_ptr(), mode,
                                        m, n, k, error.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and int(error.item()) == 0
    want = torch.empty_like(got)
    twin.linear(x, w, bias, want)
    close(got, want, out_dtype, terms=k)


@pytest.mark.parametrize("m", [256, 300, 2048, 2049])
@pytest.mark.parametrize("k", [896, 1536, 3584])
@pytest.mark.parametrize("width", [4864, 200], ids=["w4864", "w200"])
@pytest.mark.parametrize("scaled", [False, True], ids=["plain", "row-scaled"])
def test_pair_gated_product(m, k, width, scaled):
    """The product on pairs of SMs (one 256-row MMA per two CTAs) with the SiLU gate in its
    epilogue, called directly: full and ragged row tiles (the odd CTA of the last pair may own
    no row at all), widths that are no multiple of the tile, three lengths of the sum, and
    with the rows scaled by 1/rms from sums of squares that come in pieces."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 71)
    w = rand((2 * width, k), torch.bfloat16, 72, 0.05)
    got = torch.zeros((m, width), dtype=torch.bfloat16, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    pieces = torch.rand((m, 5), generator=torch.Generator().manual_seed(3)).cuda() * 300 + 20 if scaled else None
    rc = lib.mb_gemm_pair(x.data_ptr(), w.data_ptr(), None, got.data_ptr(), 2, m, width, k,
                          pieces.data_ptr() if scaled else None, 5 if scaled else 0, 1e-5, 640,
                          None, None, None, None, error.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert int(error.item()) == 0, "a bounded wait in the kernel ran out"
    scale = torch.rsqrt(pieces.double().sum(1) / 640 + 1e-5)[:, None] if scaled else 1.0
    gate = (x.double() @ w[:width].double().T) * scale
    up = (x.double() @ w[width:].double().T) * scale
    want = gate * torch.sigmoid(gate) * up
    err = float((got.double() - want).abs().max() / want.abs().max())
    assert err <= 3 * 2.0 ** -8, err
    loose = (got.double() - want).abs() <= 2.0 ** -6 * want.abs() + 2e-3 * want.abs().max()
    assert bool(loose.all())


@pytest.mark.parametrize("m,n,k", [(256, 1152, 896), (300, 896, 4864), (2049, 200, 1536), (2048, 4608, 320),
                                   (129, 264, 64), (4096, 896, 896)])
def test_pair_plain_product(twin, m, n, k):
    """The same kernel's plain mode (bias, bfloat16 out): tiles of 128 and of 256 columns."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 73)
    w = rand((n, k), torch.bfloat16, 74, 0.1)
    bias = rand((n,), torch.bfloat16, 75)
    got = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mb_gemm_pair(x.data_ptr(), w.data_ptr(), bias.data_ptr(), got.data_ptr(), 0, m, n, k,
                          None, 0, 0.0, 0, None, None, None, None, error.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and int(error.item()) == 0
    want = torch.empty_like(got)
    twin.linear(x, w, bias, want)
    close(got, want, torch.bfloat16, terms=k)


@pytest.mark.parametrize("m,n,k", [(256, 896, 896), (300, 896, 4864), (2049, 200, 1536), (2048, 4608, 320),
                                   (129, 264, 64)])
@pytest.mark.parametrize("next_norm", [False, True], ids=["add", "add+next-norm"])
def test_pair_residual_product(m, n, k, next_norm):
    """The same kernel adding into the float32 stream, and leaving what the product after the
    next norm takes: the stream times that norm's weight in bfloat16, and the rows' sums of
    squares in pieces that add up."""
    from mercury_b200.kernels import library

    lib = library.load()
    x = rand((m, k), torch.bfloat16, 76)
    w = rand((n, k), torch.bfloat16, 77, 0.1)
    h = rand((m, n), torch.float32, 78)
    h0 = h.clone()
    norm_w = rand((n,), torch.bfloat16, 79) if next_norm else None
    pieces = lib.mb_gemm_pair_tiles(m, n)
    next_x = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    next_ss = torch.full((m, pieces), float("nan"), device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.mb_gemm_pair(x.data_ptr(), w.data_ptr(), None, None, 3, m, n, k, None, 0, 0.0, 0,
                          h.data_ptr(), norm_w.data_ptr() if next_norm else None,
                          next_x.data_ptr() if next_norm else None,
                          next_ss.data_ptr() if next_norm else None, error.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and int(error.item()) == 0
    want = h0.double() + x.double() @ w.double().T
    assert float((h.double() - want).abs().max() / want.abs().max()) <= 2 * k ** 0.5 * 2.0 ** -24
    if next_norm:
        scaled = want * norm_w.double()
        assert float((next_x.double() - scaled).abs().max() / scaled.abs().max()) <= 2.0 ** -8
        sums = (want * want).sum(1)
        assert float((next_ss.double().sum(1) - sums).abs().max() / sums.max()) <= 1e-5


def test_tcgen05_refuses_an_odd_k():
    from mercury_b200.kernels import library

    assert library.load().mb_gemm_tcgen05_supports(128, 128, 100) == 0


@pytest.mark.parametrize("m,width,k", [(1, 4864, 896), (8, 128, 64), (12, 336, 96), (16, 4864, 896),
                                       (70, 320, 96), (5, 200, 80), (3, 48, 4864)])
def test_linear_swiglu(ops, twin, m, width, k):
    """Few tokens take the fused kernel, the others the product followed by the gate."""
    x = rand((m, k), torch.bfloat16, 21)
    w = rand((2 * width, k), torch.bfloat16, 22, 0.1)
    got = torch.empty((m, width), dtype=torch.bfloat16, device="cuda")
    want = torch.empty_like(got)
    ctx = SimpleNamespace(buffer=lambda name, rows, cols, dtype=None: torch.empty(
        (rows, cols), dtype=torch.bfloat16, device="cuda"))
    ops.linear_swiglu(x, w, got, ctx)
    twin.linear_swiglu(x, w, want)
    # gate and up are rounded to bfloat16 before the gate, then the result once more
    err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
    assert err <= 3 * 2.0 ** -8, err
    # with the matrix of the product behind named (the few-token kernel asks L2 for it while it
    # finishes; sizes that are no multiple of a line, and one too large to be asked for): the
    # same result, and the matrix untouched
    for rows in (7, 896, 5000):
        ahead = rand((rows, width + 3), torch.bfloat16, 23)
        kept = ahead.clone()
        again = torch.zeros_like(got)
        ops.look_ahead_min_tokens = 1
        ops.look_ahead_max_bytes = 4 * 1024 * 1024
        ops.linear_swiglu(x, w, again, ctx, ahead=ahead)
        torch.cuda.synchronize()
        assert torch.equal(again, got) and torch.equal(ahead, kept)


def fake_ctx(ops):
    def buffer(name, rows, cols, dtype=None):
        kind = torch.float32 if dtype == "float32" else (dtype or torch.bfloat16)
        return torch.empty((rows, cols), dtype=kind, device="cuda")

    return SimpleNamespace(ops=ops, dtype=torch.bfloat16, buffer=buffer)


@pytest.mark.parametrize("m,n,k", [(1, 896, 896), (8, 896, 4864), (16, 1536, 320), (40, 896, 896),
                                   (5, 100, 70)])
def test_linear_residual(ops, twin, m, n, k):
    """Few tokens: the product is added into the float32 stream by the kernel itself; other
    shapes hand the product back for the next norm to add."""
    x = rand((m, k), torch.bfloat16, 31)
    w = rand((n, k), torch.bfloat16, 32, 0.1)
    bias = rand((n,), torch.bfloat16, 33) if m % 2 else None
    h = rand((m, n), torch.float32, 34)
    want = h.double() + x.double() @ w.double().T + (bias.double() if bias is not None else 0)
    got = ops.linear_residual(x, w, bias, h, fake_ctx(ops), "tmp")
    result = h.double() if got is None else h.double() + got.double()
    assert (got is None) == (m <= 16 and n % 16 == 0 and k % 32 == 0)
    tol = 2 * k ** 0.5 * 2.0 ** -24 + (0 if got is None else 2.0 ** -8)
    assert float((result - want).abs().max() / want.abs().max()) <= tol


@pytest.mark.parametrize("m,n,k", [(1, 896, 896), (8, 896, 4864), (16, 1536, 320), (3, 64, 128)])
def test_linear_residual_leaves_the_next_norm(ops, twin, m, n, k):
    """The product that updates the stream also leaves the stream times the next norm's
    weight and the rows' sums of squares; the products after it scale their rows by 1/rms.
    Checked through all three consumers against the norm's output computed separately."""
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda")
    ops.fuse_next_norm = True
    norm = SimpleNamespace(weight=rand((n,), torch.bfloat16, 61, 0.1) + 1, eps=1e-6, size=n)
    x = rand((m, k), torch.bfloat16, 35)
    w = rand((n, k), torch.bfloat16, 45, 0.1)
    h = rand((m, n), torch.float32, 55)
    h_want = (h.double() + x.double() @ w.double().T).float()
    ctx = fake_ctx(ops)
    ctx.prenormed = None
    assert ops.linear_residual(x, w, None, h, ctx, "tmp", then_norm=norm) is None
    assert ctx.prenormed is not None and ctx.prenormed[0] is norm
    pending = ctx.prenormed[1]
    assert float((h.double() - h_want.double()).abs().max() / h_want.abs().max()) <= 2 * k ** 0.5 * 2.0 ** -24
    normed = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    twin.add_rmsnorm(h_want.clone(), None, norm.weight, norm.eps, normed)
    # materialised: the plain norm of the updated stream
    got = pending.materialize()
    assert float((got.double() - normed.double()).abs().max() / normed.double().abs().max()) <= 2.0 ** -7
    # a plain product, the gated product and the q/k/v product fed with the pending input
    w1 = rand((256, n), torch.bfloat16, 62, 0.1)
    out, want = (torch.empty((m, 256), dtype=torch.float32, device="cuda") for _ in range(2))
    ops.linear(pending, w1, None, out)
    twin.linear(normed, w1, None, want)
    assert float((out - want).abs().max() / want.abs().max()) <= 2.0 ** -6
    w2 = rand((2 * 96, n), torch.bfloat16, 63, 0.1)
    out, want = (torch.empty((m, 96), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    ops.linear_swiglu(pending, w2, out, ctx)
    twin.linear_swiglu(normed, w2, want)
    assert float((out.double() - want.double()).abs().max() / want.double().abs().max()) <= 2.0 ** -5
    n_q, n_kv, d, page = 3, 1, 64, 16
    kv_lens = tuple(range(20, 20 + m))
    batch, table = make_batch((1,) * m, kv_lens, page, 64, seed=7)
    kc, vc = fill_cache(batch, table, kv_lens, (1,) * m, n_kv, d, page, 64, torch.bfloat16, 8, False)
    kc2, vc2 = kc.clone(), vc.clone()
    w3 = rand(((n_q + 2 * n_kv) * d, n), torch.bfloat16, 64, 0.1)
    b3 = rand(((n_q + 2 * n_kv) * d,), torch.bfloat16, 65)
    angles = torch.rand((64, d // 2), generator=torch.Generator().manual_seed(9)) * 6
    tables = (angles.cos().cuda(), angles.sin().cuda())
    qkv = torch.zeros((m, (n_q + 2 * n_kv) * d), dtype=torch.bfloat16, device="cuda")
    qkv2 = qkv.clone()
    ops.qkv_rope_store(pending, w3, b3, qkv, n_q, n_kv, d, tables, batch, LayerCache(kc, vc, page, table, True))
    twin.qkv_rope_store(normed, w3, b3, qkv2, n_q, n_kv, d, tables, batch, LayerCache(kc2, vc2, page, table, True))
    for got, want in ((qkv[:, :n_q * d], qkv2[:, :n_q * d]), (kc, kc2), (vc, vc2)):
        assert float((got.double() - want.double()).abs().max() / want.double().abs().max()) <= 2.0 ** -5


@pytest.mark.parametrize("m,hidden", [(1, 896), (8, 896), (13, 1536), (16, 320)])
def test_products_that_normalise_their_own_input(ops, twin, m, hidden):
    """linear, linear_swiglu and qkv_rope_store given a PendingNorm against the same ops given
    the norm's output."""
    from mercury_b200.kernels.ops import CudaOps
    from mercury_b200.parts.norm import PendingNorm

    ops = CudaOps("cuda")
    ops.fuse_norm = True
    h = rand((m + 3, hidden), torch.float32, 41)
    norm_w = rand((hidden,), torch.bfloat16, 42, 0.1) + 1
    ctx = fake_ctx(ops)
    rows = torch.tensor(list(range(m + 2, 2, -1)), dtype=torch.int32).cuda()   # m rows, reversed
    for use_rows in (False, True):
        pending = PendingNorm(h[:m] if not use_rows else h, norm_w, 1e-6, rows if use_rows else None,
                              ctx, hidden)
        normed = torch.empty((m, hidden), dtype=torch.bfloat16, device="cuda")
        twin.add_rmsnorm((h[:m] if not use_rows else h).clone(), None, norm_w, 1e-6, normed,
                         rows if use_rows else None)
        w = rand((1024, hidden), torch.bfloat16, 43, 0.1)
        got = torch.empty((m, 1024), dtype=torch.float32, device="cuda")
        want = torch.empty_like(got)
        ops.linear(pending, w, None, got)
        twin.linear(normed, w, None, want)
        # the norm's output is rounded to bfloat16 either way; its last bit may differ
        assert float((got - want).abs().max() / want.abs().max()) <= 2.0 ** -7
    pending = PendingNorm(h[:m], norm_w, 1e-6, None, ctx, hidden)
    twin.add_rmsnorm(h[:m].clone(), None, norm_w, 1e-6, normed)
    w2 = rand((2 * 336, hidden), torch.bfloat16, 44, 0.1)
    got = torch.empty((m, 336), dtype=torch.bfloat16, device="cuda")
    want = torch.empty_like(got)
    ops.linear_swiglu(pending, w2, got, ctx)
    twin.linear_swiglu(normed, w2, want)
    assert float((got.double() - want.double()).abs().max() / want.double().abs().max()) <= 4 * 2.0 ** -8
    n_q, n_kv, d, page = 3, 1, 64, 16
    kv_lens = tuple(range(20, 20 + m))
    batch, table = make_batch((1,) * m, kv_lens, page, 64, seed=7)
    k, v = fill_cache(batch, table, kv_lens, (1,) * m, n_kv, d, page, 64, torch.bfloat16, 8, False)
    k2, v2 = k.clone(), v.clone()
    w3 = rand(((n_q + 2 * n_kv) * d, hidden), torch.bfloat16, 45, 0.1)
    b3 = rand(((n_q + 2 * n_kv) * d,), torch.bfloat16, 46)
    angles = torch.rand((64, d // 2), generator=torch.Generator().manual_seed(9)) * 6
    tables = (angles.cos().cuda(), angles.sin().cuda())
    qkv = torch.zeros((m, (n_q + 2 * n_kv) * d), dtype=torch.bfloat16, device="cuda")
    qkv2 = qkv.clone()
    ops.qkv_rope_store(pending, w3, b3, qkv, n_q, n_kv, d, tables, batch, LayerCache(k, v, page, table, True))
    twin.qkv_rope_store(normed, w3, b3, qkv2, n_q, n_kv, d, tables, batch, LayerCache(k2, v2, page, table, True))
    for got, want in ((qkv[:, :n_q * d], qkv2[:, :n_q * d]), (k, k2), (v, v2)):
        assert float((got.double() - want.double()).abs().max() / want.double().abs().max()) <= 4 * 2.0 ** -8


def test_products_fed_by_tma(ops, twin):
    """Large matrices take the few-token kernel whose weights come by TMA into per-warp rings
    (by itself from 12 Mi elements on, the gated product from 64 Mi): forced here on small shapes too, every epilogue."""
    lib = ops.lib
    assert lib.mb_gemm_skinny_set_fed_min(1) == 0
    try:
        for m, n, k in ((1, 1152, 896), (8, 896, 4864), (16, 9728, 896), (13, 48, 64), (3, 896, 64),
                        (2, 151936, 64), (9, 4112, 320)):
            test_linear(ops, twin, m, n, k, torch.bfloat16, torch.bfloat16, torch.bfloat16)
            test_linear(ops, twin, m, n, k, torch.bfloat16, torch.bfloat16, torch.float32)
        for m, n, k in ((1, 896, 896), (8, 896, 4864), (16, 1536, 320)):
            test_linear_residual(ops, twin, m, n, k)
            test_linear_residual_leaves_the_next_norm(ops, twin, m, n, k)
        for m, width, k in ((1, 4864, 896), (8, 128, 64), (12, 336, 128), (16, 4864, 896), (3, 48, 4864)):
            test_linear_swiglu(ops, twin, m, width, k)
        ops.check_errors()
    finally:
        assert lib.mb_gemm_skinny_set_fed_min(12 * 1024 * 1024) == 0


QKV_ATTENTION_CASES = [
    # n_q, n_kv, d, page, hidden, q_lens, kv_lens, window, rotate
    (14, 2, 64, 16, 896, (1, 1, 1), (2048, 300, 1), 0, True),
    (14, 2, 64, 16, 896, (1,) * 8, (64, 65, 63, 128, 129, 640, 700, 17), 0, True),
    (4, 2, 64, 16, 128, (2, 1, 3, 8), (700, 300, 3, 72), 128, True),       # several new tokens
    (8, 8, 128, 32, 256, (1, 9, 16), (45, 60, 130), 16, True),
    (12, 2, 128, 16, 1536, (1, 2), (500, 129), 0, True),
    (7, 1, 64, 64, 64, (2, 1), (333, 64), 0, False),                         # no rotation
    (8, 1, 64, 8, 96, (1, 1, 1), (64, 65, 1000), 0, True),
]


@pytest.mark.parametrize("splits", [1, 2, 8])
@pytest.mark.parametrize("case", range(len(QKV_ATTENTION_CASES)), ids=lambda i: f"case{i}")
def test_projection_rotation_store_and_attention_in_one_op(twin, case, splits):
    """`qkv_attention` on decode-like batches: the plain product leaves bare q/k/v, the cluster
    attention kernel rotates the queries, rotates and stores the new keys and values, and
    attends. Pages, poisoned outside the sequences' keys, and output against the twin."""
    from mercury_b200.kernels.ops import CudaOps

    n_q, n_kv, d, page, hidden, q_lens, kv_lens, window, rotate = QKV_ATTENTION_CASES[case]
    ops = CudaOps("cuda", decode_splits=splits)
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 4
    drop = [max(0, kv - q - window + 1) for q, kv in zip(q_lens, kv_lens)] if window else None
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=2, seed=3, drop_before=drop)
    k, v = fill_cache(batch, table, kv_lens, q_lens, n_kv, d, page, num_pages, torch.bfloat16, 4, True)
    tokens = batch.num_tokens
    x = rand((tokens, hidden), torch.bfloat16, 23)
    w = rand(((n_q + 2 * n_kv) * d, hidden), torch.bfloat16, 24, 0.1)
    bias = rand(((n_q + 2 * n_kv) * d,), torch.bfloat16, 25)
    angles = torch.rand((max(kv_lens) + 1, d // 2), generator=torch.Generator().manual_seed(5)) * 6
    tables = (angles.cos().cuda(), angles.sin().cuda()) if rotate else None
    qkv = torch.zeros((tokens, (n_q + 2 * n_kv) * d), dtype=torch.bfloat16, device="cuda")
    qkv_twin = qkv.clone()
    k_twin, v_twin = k.clone(), v.clone()
    got = torch.zeros((tokens, n_q * d), dtype=torch.bfloat16, device="cuda")
    want = torch.zeros_like(got)
    calls = lambda: ops.launches + ops.library_calls       # (more than 16 tokens: the library's product)
    before = calls()
    ops.qkv_attention(x, w, bias, qkv, n_q, n_kv, d, tables, batch, LayerCache(k, v, page, table, True),
                      d ** -0.5, window, got)
    assert calls() - before == 2, "the product, then attention"
    twin.qkv_attention(x, w, bias, qkv_twin, n_q, n_kv, d, tables, batch,
                       LayerCache(k_twin, v_twin, page, table, True), d ** -0.5, window, want)
    assert torch.equal(torch.isnan(k), torch.isnan(k_twin)), "keys stored in the wrong slots"
    assert torch.equal(torch.isnan(v), torch.isnan(v_twin)), "values stored in the wrong slots"
    for mine, theirs in ((k, k_twin), (v, v_twin)):
        a, b = torch.nan_to_num(mine).double(), torch.nan_to_num(theirs).double()
        assert float((a - b).abs().max() / b.abs().max()) <= 4 * 2.0 ** -8
    live = batch.seq_of_token >= 0
    assert torch.isfinite(got[live]).all(), "attention read a poisoned slot"
    attention_close(got[live], want[live], torch.bfloat16, "clusters")
    # a call that only reads another layer's cache must not take the one-op path
    launches = ops.launches
    ops.qkv_attention(x, w, bias, qkv, n_q, n_kv, d, tables, batch, LayerCache(k, v, page, table, False),
                      d ** -0.5, window, got)
    assert ops.launches - launches == 2          # the fused q/k/v kernel, then attention (both this package's)
    attention_close(got[live], want[live], torch.bfloat16, "clusters")


@pytest.mark.parametrize("slices", [2, 4])
def test_products_with_k_shared_between_the_blocks_of_a_cluster(ops, twin, slices):
    """The few-token products may cut K over the blocks of a thread-block cluster (they do
    so by themselves only for long K and few row tiles): forced here on every shape."""
    lib = ops.lib
    assert lib.mb_gemm_skinny_set_slices(slices, slices) == 0
    try:
        for m, n, k in ((1, 1152, 896), (8, 896, 4864), (16, 9728, 896), (13, 48, 96), (3, 896, 64)):
            test_linear(ops, twin, m, n, k, torch.bfloat16, torch.bfloat16, torch.bfloat16)
            test_linear(ops, twin, m, n, k, torch.bfloat16, torch.bfloat16, torch.float32)
        for m, n, k in ((1, 896, 896), (8, 896, 4864), (16, 1536, 320)):
            test_linear_residual(ops, twin, m, n, k)
            test_linear_residual_leaves_the_next_norm(ops, twin, m, n, k)
        for shape in ((14, 2, 64, 16, 896), (12, 2, 128, 16, 1536), (3, 1, 64, 8, 96)):
            test_qkv_rope_store_fused(ops, twin, *shape, (1, 1, 1), (40, 17, 300))
            test_qkv_rope_store_fused(ops, twin, *shape, (1,) * 9, tuple(range(5, 50, 5)))
    finally:
        assert lib.mb_gemm_skinny_set_slices(0, 0) == 0
    assert lib.mb_gemm_skinny_set_slices(3, 1) != 0


@pytest.mark.parametrize("n_q,n_kv,d,page,hidden", [(14, 2, 64, 16, 896), (12, 2, 128, 16, 1536),
                                                    (3, 1, 64, 8, 96), (4, 4, 128, 32, 64)])
@pytest.mark.parametrize("q_lens,kv_lens", [((1, 1, 1), (40, 17, 300)), ((1,) * 9, tuple(range(5, 50, 5))),
                                            ((20, 1, 2), (20, 64, 33))])
def test_qkv_rope_store_fused(ops, twin, n_q, n_kv, d, page, hidden, q_lens, kv_lens):
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 4
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=2, seed=3)
    k, v = fill_cache(batch, table, kv_lens, q_lens, n_kv, d, page, num_pages, torch.bfloat16, 4, True)
    tokens = batch.num_tokens
    x = rand((tokens, hidden), torch.bfloat16, 23)
    w = rand(((n_q + 2 * n_kv) * d, hidden), torch.bfloat16, 24, 0.1)
    bias = rand(((n_q + 2 * n_kv) * d,), torch.bfloat16, 25)
    angles = torch.rand((max(kv_lens) + 1, d // 2), generator=torch.Generator().manual_seed(5)) * 6
    tables = (angles.cos().cuda(), angles.sin().cuda())
    qkv = torch.zeros((tokens, (n_q + 2 * n_kv) * d), dtype=torch.bfloat16, device="cuda")
    qkv_twin = qkv.clone()
    k_twin, v_twin = k.clone(), v.clone()
    ops.qkv_rope_store(x, w, bias, qkv, n_q, n_kv, d, tables, batch, LayerCache(k, v, page, table, True))
    twin.qkv_rope_store(x, w, bias, qkv_twin, n_q, n_kv, d, tables, batch,
                        LayerCache(k_twin, v_twin, page, table, True))
    live = batch.seq_of_token >= 0
    q_got, q_want = qkv[live][:, :n_q * d], qkv_twin[live][:, :n_q * d]
    # the projection is rounded to bfloat16, rotated, and rounded again
    tol = 3 * 2.0 ** -8
    assert float((q_got.double() - q_want.double()).abs().max() / q_want.double().abs().max()) <= tol
    assert torch.equal(torch.isnan(k), torch.isnan(k_twin)), "keys stored in the wrong slots"
    assert torch.equal(torch.isnan(v), torch.isnan(v_twin))
    for got, want in ((k, k_twin), (v, v_twin)):
        got, want = torch.nan_to_num(got).double(), torch.nan_to_num(want).double()
        assert float((got - want).abs().max() / want.abs().max()) <= tol


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_swiglu(ops, twin, dtype):
    gate_up = rand((33, 2 * 517), dtype, 10, 3.0)
    got = torch.empty((33, 517), dtype=dtype, device="cuda")
    want = torch.empty_like(got)
    ops.swiglu(gate_up, got)
    twin.swiglu(gate_up, want)
    close(got, want, dtype)


# ------------------------------------------------------------------------------ attention

def make_batch(q_lens, kv_lens, page_size, num_pages, pad_tokens=0, seed=0, drop_before=None):
    """A ragged batch with scattered pages. `drop_before[s]` marks the pages of sequence s
    that lie wholly below that position as given back (-1)."""
    gen = torch.Generator().manual_seed(seed)
    num_seqs = len(q_lens)
    max_pages = max(-(-kv // page_size) for kv in kv_lens) + 1
    perm = torch.randperm(num_pages, generator=gen).tolist()
    table = torch.full((num_seqs, max_pages), -1, dtype=torch.int32)
    positions, seq_of, q_start = [], [], [0]
    for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
        for i in range(-(-kv // page_size)):
            table[s, i] = perm.pop()
        if drop_before is not None:
            for i in range(drop_before[s] // page_size):
                table[s, i] = -1
        positions += list(range(kv - q, kv))
        seq_of += [s] * q
        q_start.append(q_start[-1] + q)
    positions += [0] * pad_tokens
    seq_of += [-1] * pad_tokens
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return SimpleNamespace(
        num_tokens=len(positions), num_seqs=num_seqs, max_q_len=max(q_lens),
        max_kv_len=max(kv_lens), positions=as_dev(positions), seq_of_token=as_dev(seq_of),
        q_start=as_dev(q_start), kv_len=as_dev(list(kv_lens))), table.cuda()


def fill_cache(batch, table, kv_lens, q_lens, n_kv, d, page_size, num_pages, dtype, seed, poison):
    """Pages holding random keys for the positions computed before this step, and poison
    (NaN) everywhere else, so that any read outside a sequence's keys shows."""
    fill = float("nan") if poison else 0.0
    k = torch.full((num_pages, n_kv, page_size, d), fill, dtype=dtype, device="cuda")
    v = torch.full((num_pages, n_kv, page_size, d), fill, dtype=dtype, device="cuda")
    gen = torch.Generator().manual_seed(seed)
    for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
        for pos in range(kv - q):
            page = int(table[s, pos // page_size])
            if page < 0:
                continue
            k[page, :, pos % page_size] = torch.randn((n_kv, d), generator=gen).to(dtype).cuda()
            v[page, :, pos % page_size] = torch.randn((n_kv, d), generator=gen).to(dtype).cuda()
    return k, v


ATTENTION_CASES = [
    # n_q, n_kv, d, page, q_lens, kv_lens, window
    (4, 2, 16, 16, (5, 1, 33), (5, 40, 33), 0),
    (3, 1, 32, 8, (1, 1, 1, 1), (1, 9, 24, 40), 0),
    (14, 2, 64, 16, (1, 17, 1), (300, 17, 64), 0),
    (6, 2, 48, 16, (40, 1, 2), (100, 77, 50), 24),
    (7, 1, 64, 32, (64, 1), (64, 129), 0),
    (12, 2, 128, 16, (3, 1), (130, 257), 0),
    (20, 1, 80, 64, (2, 1), (70, 200), 0),
    (8, 8, 256, 16, (1, 9), (45, 60), 16),
    (5, 5, 112, 8, (31, 1), (31, 32), 0),


    (14, 2, 64, 16, (130, 1, 9), (130, 515, 300), 0),
    (6, 3, 128, 32, (70, 2), (200, 66), 50),
    (8, 1, 64, 8, (1, 1, 1), (64, 65, 1000), 0),
    (14, 2, 64, 64, (200, 3), (500, 131), 0),
    (7, 7, 64, 128, (150,), (400,), 0),
    (4, 2, 64, 16, (300, 1, 70), (600, 200, 70), 100),
    (14, 2, 64, 16, (1, 1, 1, 1), (2048, 300, 64, 1), 0),
    (16, 8, 128, 16, (2, 1), (500, 129), 0),
    (4, 2, 64, 16, (1, 2), (700, 300), 128),
    (7, 1, 64, 64, (2,), (333,), 0),
    # one block walks more keys than the 256 block-table entries it keeps in shared memory
    (14, 2, 64, 16, (1, 1), (5000, 4101), 0),
    (4, 2, 128, 8, (1, 2), (2500, 40), 0),
]


def attention_close(got, want, dtype, kernel):
    """The tensor-core kernels round the probabilities to bfloat16 before P.V and the result
    once more: two roundings of 2^-8, against one for the CUDA-core kernel."""
    if kernel in ("mma", "tcgen05", "clusters", "clusters-tma"):
        err = float((got.double() - want.double()).abs().max()) / float(want.abs().max())
        assert err <= 2 * 2.0 ** -8, f"attention (mma): relative error {err:.3e}"
    else:
        close(got, want, dtype, "attention")


@pytest.mark.parametrize("kernel,dtype", [("simt", torch.float32), ("simt", torch.bfloat16),
                                          ("mma", torch.bfloat16), ("tcgen05", torch.bfloat16),
                                          ("clusters", torch.bfloat16), ("clusters-tma", torch.bfloat16)],
                         ids=["f32", "bf16", "bf16-mma", "bf16-tcgen05", "bf16-clusters", "bf16-clusters-tma"])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("case", range(len(ATTENTION_CASES)), ids=lambda i: f"case{i}")
def test_rope_store_and_attention(twin, dtype, kernel, splits, case):
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda", decode_splits=splits)
    n_q, n_kv, d, page, q_lens, kv_lens, window = ATTENTION_CASES[case]
    if kernel == "mma" and not ops.lib.mb_attention_mma_supports(d):
        pytest.skip("head size left to the CUDA-core kernel")
    if kernel == "tcgen05" and not ops.lib.mb_attention_tcgen05_supports(
            d, page, n_q, n_kv, (n_q + 2 * n_kv) * d):
        pytest.skip("left to the other attention kernels")
    if kernel in ("clusters", "clusters-tma") and not (ops.lib.mb_attention_mma_supports(d)
                                                       and max(q_lens) * (n_q // n_kv) <= 16):
        pytest.skip("the cluster kernel is for decode-like batches of head size 64 or 128")
    if kernel == "clusters-tma":
        if not 8 <= page <= 64:
            pytest.skip("the TMA-fed form is for pages of 8 to 64 tokens")
        ops.decode_long_ranges = True      # the form that large batches take
    # for the tensor-memory kernel the split is the number of CTAs that share a row tile, for
    # the decode clusters the number of blocks of a (sequence, KV head)
    clusters = (None,)
    if kernel == "tcgen05":
        clusters = (1,) if splits == 1 else (2, 4)
    elif kernel in ("clusters", "clusters-tma"):
        clusters = (1,) if splits == 1 else (2, 4, 8)
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 5
    drop = [max(0, kv - q - window + 1) for q, kv in zip(q_lens, kv_lens)] if window else None
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=3, seed=1,
                              drop_before=drop)
    k, v = fill_cache(batch, table, kv_lens, q_lens, n_kv, d, page, num_pages, dtype, 2, True)
    tokens = batch.num_tokens
    qkv = rand((tokens, (n_q + 2 * n_kv) * d), dtype, 3)
    angles = torch.rand((max(kv_lens) + 1, d // 2), generator=torch.Generator().manual_seed(4)) * 6
    tables = (angles.cos().cuda(), angles.sin().cuda())

    qkv_twin, k_twin, v_twin = qkv.clone(), k.clone(), v.clone()
    cache = LayerCache(k, v, page, table, True)
    cache_twin = LayerCache(k_twin, v_twin, page, table, True)
    ops.rope_cache_write(qkv, n_q, n_kv, d, tables, batch, cache)
    twin.rope_cache_write(qkv_twin, n_q, n_kv, d, tables, batch, cache_twin)
    live = batch.seq_of_token >= 0
    close(qkv[live], qkv_twin[live], dtype, "rotated q/k")
    assert torch.equal(torch.isnan(k), torch.isnan(k_twin)), "keys stored in the wrong slots"
    close(torch.nan_to_num(k), torch.nan_to_num(k_twin), dtype, "stored keys")
    close(torch.nan_to_num(v), torch.nan_to_num(v_twin), dtype, "stored values")

    want = torch.zeros((tokens, n_q * d), dtype=dtype, device="cuda")
    twin.paged_attention(qkv_twin, n_q, n_kv, d, batch, cache_twin, d ** -0.5, window, want)
    for cluster in clusters:
        ops.prompt_cluster = cluster
        if kernel in ("clusters", "clusters-tma"):
            ops.decode_splits = cluster
        got = torch.zeros_like(want)
        ops.paged_attention(qkv, n_q, n_kv, d, batch, cache, d ** -0.5, window, got,
                            kernel=None if kernel in ("clusters", "clusters-tma") else kernel)
        ops.check_errors()
        assert torch.isfinite(got[live]).all(), "attention read a poisoned slot"
        attention_close(got[live], want[live], dtype, kernel)


@pytest.mark.parametrize("kernel,dtype", [("simt", torch.float32), ("simt", torch.bfloat16),
                                          ("mma", torch.bfloat16), (None, torch.bfloat16)],
                         ids=["f32", "bf16", "bf16-mma", "bf16-clusters"])
@pytest.mark.parametrize("splits", [1, 5])
def test_attention_finds_one_far_key(twin, dtype, kernel, splits):
    """Among 700 keys one far key matches the query strongly; the output must be that
    key's value. Its place is moved over page edges and tile edges."""
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda", decode_splits=splits)
    n_q, n_kv, d, page, kv = 4, 2, 64, 16, 700
    for far in (0, 15, 16, 31, 32, 333, 698):
        batch, table = make_batch((1,), (kv,), page, 60, seed=far)
        k, v = fill_cache(batch, table, (kv,), (1,), n_kv, d, page, 60, dtype, 5, False)
        k *= 0.05
        qkv = torch.zeros((1, (n_q + 2 * n_kv) * d), dtype=dtype, device="cuda")
        direction = torch.nn.functional.normalize(rand((d,), torch.float32, 6), dim=0)
        qkv[0, :n_q * d] = (direction * 12).repeat(n_q).to(dtype)
        slot = int(table[0, far // page])
        k[slot, :, far % page] = (direction * 12).to(dtype)
        cache = LayerCache(k, v, page, table, False)
        ops.rope_cache_write(qkv, n_q, n_kv, d, None, batch, cache)
        got = torch.zeros((1, n_q * d), dtype=dtype, device="cuda")
        ops.paged_attention(qkv, n_q, n_kv, d, batch, cache, d ** -0.5, 0, got, kernel=kernel)
        want = v[slot, :, far % page].float().repeat_interleave(n_q // n_kv, dim=0).reshape(-1)
        err = float((got[0].float() - want).abs().max())
        assert err < 0.05, f"far key at {far}: output is off by {err}"


def test_attention_refuses_what_it_cannot_do(ops):
    batch, table = make_batch((1,), (4,), 16, 4)
    k = torch.zeros((4, 1, 16, 272), dtype=torch.bfloat16, device="cuda")
    cache = LayerCache(k, k.clone(), 16, table, True)
    qkv = torch.zeros((1, 3 * 272), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((1, 272), dtype=torch.bfloat16, device="cuda")
    from mercury_b200.kernels.library import KernelError

    with pytest.raises(KernelError):
        ops.paged_attention(qkv, 1, 1, 272, batch, cache, 1.0, 0, out)


# ------------------------------------------------------------------------------ sampling

@pytest.mark.parametrize("vocab", [1517, 151936])
def test_argmax_lowest_index_wins(ops, vocab):
    logits = rand((9, vocab), torch.float32, 11)
    logits[3, 700] = logits[3, 20] = 50.0
    logits[5, vocab - 1] = 60.0
    out = torch.empty(9, dtype=torch.int32, device="cuda")
    ops.argmax(logits, out)
    assert out.tolist() == torch.argmax(logits, dim=-1).tolist()
    assert out[3] == 20


@pytest.mark.parametrize("vocab", [331, 4097, 151936])
def test_sample_lands_in_the_right_interval(ops, vocab):
    """The drawn token's cumulative-probability interval contains u (within float32
    rounding of the sums); greedy rows are the argmax; top-p keeps the right set."""
    rows = 12
    logits = rand((rows, vocab), torch.float32, 12, 2.0)
    temperature = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.7, 0.2, 1.0, 0.0, 5.0, 0.7, 1.0, 0.05]).cuda()
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.9, 0.5, 0.1, 0.3, 0.95, 0.0, 0.999, 1.0]).cuda()
    u = torch.tensor([0.5, 0.0, 0.999999, 0.25, 0.5, 0.75, 0.3, 0.1, 0.6, 0.9, 0.42, 0.8]).cuda()
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample(logits, temperature, top_p, u, out)
    for r in range(rows):
        t, p = float(temperature[r]), float(top_p[r])
        tok = int(out[r])
        if t <= 0:
            assert tok == int(torch.argmax(logits[r]))
            continue
        probs = torch.softmax(logits[r].double().cpu() / max(t, 1e-5), dim=-1)
        if p < 1.0:
            ordered, index = probs.sort(descending=True)
            before = ordered.cumsum(-1) - ordered
            kept = torch.zeros_like(probs).scatter_(0, index, ordered.masked_fill(before > p, 0.0))
            # the crossing token may fall either way when float32 sums touch the threshold
            edge = (before - p).abs() < 1e-5
            assert kept[tok] > 0 or bool(edge[index == tok]), f"row {r}: dropped token drawn"
            probs = kept
        cdf = probs.cumsum(-1) / probs.sum()
        low = float(cdf[tok - 1]) if tok > 0 else 0.0
        assert low - 1e-4 <= float(u[r]) <= float(cdf[tok]) + 1e-4, (r, tok, low, float(cdf[tok]))
