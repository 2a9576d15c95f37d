"""The kernel set of the engine: thin Python wrappers that hand tensors' addresses, sizes
and the current stream to the compiled sm_100a kernels.

This is the only kernel set the product has. It needs a CUDA device of compute capability
10.x and the compiled library, and raises when either is missing.
"""

from __future__ import annotations

import contextlib
import functools

import torch

from . import library
from .library import KernelError, check

_F32, _BF16 = 0, 1


def _flag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _timed(kind: str):
    """Marks a kernel-set method as one class of the step's time. While `begin_timing()` is
    in force the outermost such call is bracketed by CUDA events and booked under `kind`;
    otherwise the method runs as it is."""
    def wrap(method):
        @functools.wraps(method)
        def run(self, *args, **kwargs):
            if self._timing is None or self._timing_depth:
                return method(self, *args, **kwargs)
            label = self._timing_label or kind
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._timing_depth += 1
            start.record()
            try:
                return method(self, *args, **kwargs)
            finally:
                stop.record()
                self._timing_depth -= 1
                self._timing.append((label, start, stop))
        return run
    return wrap


class CudaOps:
    def __init__(self, device="cuda", decode_splits: int | None = None, gemm: str = "auto",
                 dependent_launch: bool = False):
        """`gemm` picks the bfloat16 product on many tokens: "tcgen05" (this package's
        TMA + tensor-memory kernel wherever it takes the shape), "library" (cuBLAS through
        torch.mm, where the reference calls F.linear), "auto" (the default: the gated gate/up
        product with its SiLU epilogue on the persistent tcgen05 kernel, where fusing beats
        library product plus gate kernel, and the plain products on the library, which is
        still ahead there) or "simt" (the CUDA-core kernel). Few tokens always take the weight-streaming
        kernels. The float32 engine always runs the CUDA-core kernel: a library product
        would need its reduced-precision mode switched off process-wide to be a true 32-bit
        product."""
        if gemm not in ("library", "simt", "tcgen05", "auto"):
            raise KernelError(f"unknown gemm choice {gemm!r}")
        self.gemm = gemm
        self.skinny = True     # few-token products go to the weight-streaming kernels
        # ... up to this many weight elements: a larger matrix (the LM head) is bound by HBM
        # alone, and there the library's kernel streams faster (measured on B200 with 8
        # tokens, weights cold: 151936 x 896 in 52 us against 76 us, 5.3 against 3.6 TB/s)
        self.skinny_max_elements = 96 * 1024 * 1024
        # ... and from this many on, weights come by TMA (gemm_skinny.cu: skinny_fed_kernel);
        # only those launches have a wait that can give up and so an error word to look at
        self.fed_min_elements = 12 * 1024 * 1024
        # The gated product of a prompt step runs on pairs of SMs (gemm_pair.cu) from this K
        # on; below it the one-CTA persistent kernel is level or ahead (measured on B200 at
        # 2048 tokens: K 896, 34 us one CTA against 35 us pairs; K 1536, 91 against 86; at 4096
        # tokens, K 3584 and 2 x 18944 rows, 1515 against 1028)
        self.pair_min_k = 1024
        # The gated few-token product asks L2 for the down-proj's matrix while it finishes, up
        # to this many bytes (a matrix that L2 cannot hold beside everything else gains nothing)
        self.look_ahead_max_bytes = 32 * 1024 * 1024
        # ... and from this many tokens on (measured on B200 inside the captured decode step,
        # 0.5B sizes: 16 sequences 0.950 -> 0.907 ms; 8 sequences 0.598 -> 0.605, one sequence
        # 0.566 -> 0.578: with few tokens the kernel is too short for the lines to arrive)
        self.look_ahead_min_tokens = 9
        # ... and beyond this many weight elements the library's product followed by the gate
        # kernel is ahead of both (measured on B200 at 2048 tokens, replayed from a graph:
        # 2 x 4864 x 896, 35 us fused against 43; 2 x 8960 x 1536, 87 against 101;
        # 2 x 18944 x 3584, 503 against 424: there the library's 1.5 PFLOP/s outweigh the
        # gate kernel's extra pass)
        self.gated_max_elements = 64 * 1024 * 1024
        # ... and so it is for small portions, below this many multiply-adds (replayed from a
        # graph: 512 tokens at 0.5B widths 17.5 us fused against 14.9; 1024 tokens 23.5 against
        # 25.2; 256 tokens at 1.5B widths 16.2 against 16.5; 512 tokens 25.4 against 28.5)
        self.gated_min_products = 8 * 10 ** 9
        # "auto": the tensor-memory (tcgen05) kernel for prompt portions of head sizes 64 and
        # 128, the mma.sync kernels for everything else; "mma": the mma.sync kernels only
        self.attention = "auto"
        self.prompt_cluster: int | None = None  # override of the CTAs per row tile (1, 2, 4)
        # decode-like batches: the key ranges of a (sequence, KV head) as one cluster of up to
        # 8 blocks, merged through distributed shared memory, while fewer than 32 ranges are
        # wanted; beyond that (very long contexts in a small batch) the ranges go through
        # global memory as before
        self.decode_clusters = True
        self.prompt_splits: int | None = None   # override of the key split of prompt portions
        # Normalising inside the consuming product saves a launch but makes every block
        # redo the row statistics; measured on B200 the separate norm kernel is faster for
        # the Qwen2 shapes, so the fusion is off unless asked for.
        self.fuse_norm = False
        # The product that adds into the stream also leaves the stream times the next norm's
        # weight and the rows' sums of squares; the product after that norm multiplies its
        # result rows by 1/rms. The norm's own launch disappears.
        self.fuse_next_norm = True
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: the engine's kernels are CUDA only and there is "
                              "no CPU path")
        self.device = torch.device(device)
        major, _minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}x")
        self.lib = library.load()
        # the checked variant of the library (MERCURY_B200_BOUNDS_CHECK=1): indices are
        # compared with their limits inside the kernels; see csrc/common.cuh
        self.checked = bool(self.lib.mb_check_enabled())
        self.lib.mb_gemm_skinny_set_fed_min(self.fed_min_elements)
        # let each kernel be scheduled while its predecessor drains (see csrc/common.cuh)
        self.dependent_launch = bool(dependent_launch)     # True: on every launch, not only in graphs
        self.lib.mb_set_dependent_launch(int(dependent_launch))
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_splits = decode_splits
        # Key ranges per (sequence, KV head) of a captured decode step, whose grid is fixed at
        # capture. Measured on B200 at 2048-token contexts: about `graph_blocks_per_sm_small`
        # blocks per SM while the batch brings at most `graph_small_rows` (sequence, KV head)
        # pairs, at most `graph_max_ranges_small` ranges each (a range then still holds three
        # or more 64-key tiles); about `graph_blocks_per_sm_large` per SM beyond that.
        self.graph_small_rows = 16
        self.decode_long_ranges: bool | None = None   # override of the choice of `_long_ranges`
        self.graph_max_ranges_small = 12
        self.graph_blocks_per_sm_small = 1
        self.graph_blocks_per_sm_large = 2
        self._scratch: torch.Tensor | None = None
        # scratch and counters that a larger request replaced: graphs captured earlier still
        # write to them, so they are never given back to the allocator
        self._retired: list[torch.Tensor] = []
        self._counters: torch.Tensor | None = None   # zeroed tickets of the in-kernel split merge
        self._tc_error: torch.Tensor | None = None   # error word of the tcgen05 kernels
        self._tc_pending = False
        self._argmax_scratch: torch.Tensor | None = None
        self._timing: list | None = None      # (kind, start event, stop event) while timing
        self._timing_depth = 0
        self._event_overhead_ms: float | None = None
        self._timing_label: str | None = None  # overrides the class of the calls inside `_as`
        self._pinned_stream: int | None = None
        self.launches = 0
        self.library_calls = 0
        # Which launch (by count) last wrote a float32 residual stream. A residual product
        # reads the stream before it waits for the kernel in front (see mb_gemm_skinny) unless
        # that kernel is this writer. Only this library's kernels let their successor start
        # early, and each of them that writes a stream is noted here.
        self._last_stream_write = -1
        # split-K partial sums stay float32
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # ------------------------------------------------------------------ helpers

    def _stream(self) -> int:
        if self._pinned_stream is not None:
            return self._pinned_stream
        return torch.cuda.current_stream(self.device).cuda_stream

    def set_dependent_launch(self, enabled: bool) -> None:
        """Launch the kernels that follow with (or without) the programmatic-serialization
        attribute; see csrc/common.cuh."""
        self.lib.mb_set_dependent_launch(int(bool(enabled) or self.dependent_launch))

    def pin_stream(self) -> None:
        """Look the current stream up once for the many launches of a step."""
        self._pinned_stream = torch.cuda.current_stream(self.device).cuda_stream

    def unpin_stream(self) -> None:
        self._pinned_stream = None

    @contextlib.contextmanager
    def _as(self, label: str):
        """Calls made inside are booked under `label` instead of their own class."""
        before, self._timing_label = self._timing_label, label
        try:
            yield
        finally:
            self._timing_label = before

    def begin_timing(self) -> None:
        """From now on bracket every kernel-set call with CUDA events (eager steps only: a
        replayed graph makes no calls)."""
        self._timing = []

    def end_timing(self) -> dict[str, float]:
        """Milliseconds per class of call since `begin_timing()`; waits for the device. What
        a pair of events measures with nothing between them (a few microseconds) is taken
        off every call."""
        events, self._timing = self._timing or [], None
        if events and self._event_overhead_ms is None:
            empty = []
            for _ in range(20):
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                stop.record()
                empty.append((start, stop))
            torch.cuda.synchronize(self.device)
            gaps = sorted(a.elapsed_time(b) for a, b in empty)
            self._event_overhead_ms = gaps[len(gaps) // 2]
        torch.cuda.synchronize(self.device)
        out: dict[str, float] = {}
        for kind, start, stop in events:
            out[kind] = out.get(kind, 0.0) + max(0.0, start.elapsed_time(stop) - self._event_overhead_ms)
        return out

    def _scratch_for(self, floats: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < floats:
            if self._scratch is not None:
                # a captured graph may hold the old buffer's address: keep it allocated
                self._retired.append(self._scratch)
            self._scratch = torch.empty(max(floats, 1 << 20), dtype=torch.float32,
                                        device=self.device)
        return self._scratch

    def _counters_for(self, count: int) -> torch.Tensor:
        """Zeroed tickets of the in-kernel split merge (the last block resets its own)."""
        if self._counters is None or self._counters.numel() < count:
            if self._counters is not None:
                self._retired.append(self._counters)
            self._counters = torch.zeros(max(count, 4096), dtype=torch.int32, device=self.device)
        return self._counters

    @staticmethod
    def _rows(t: torch.Tensor) -> torch.Tensor:
        if not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")
        return t

    # ------------------------------------------------------------------ kernels

    @_timed("embedding")
    def embed(self, token_ids, table, out):
        self._rows(out)
        check(self.lib.mb_embed(_ptr(token_ids), _ptr(table), _flag(table.dtype), _ptr(out),
                                out.shape[0], out.shape[1], table.shape[0], self._stream()),
              "embed")
        self.launches += 1
        self._note_stream_write()

    def _note_stream_write(self) -> None:
        self._last_stream_write = self.launches + self.library_calls

    def patch_tokens(self, token_ids, token_from, sampled):
        """token_ids[t] = sampled[token_from[t]] wherever token_from[t] >= 0: ids that the
        step before has sampled on the device and the host has not read yet."""
        check(self.lib.mb_patch_tokens(_ptr(token_ids), _ptr(token_from), _ptr(sampled),
                                       token_ids.shape[0], self._stream()), "patch_tokens")
        self.launches += 1

    @_timed("norm")
    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None):
        count = h.shape[0] if rows is None else rows.shape[0]
        if delta is not None and delta.dtype != out.dtype:
            raise KernelError("add_rmsnorm: delta and out must share the activation dtype")
        check(self.lib.mb_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), _flag(weight.dtype),
                                      _ptr(out), _ptr(rows), count, h.shape[1], float(eps),
                                      _flag(out.dtype), self._stream()), "add_rmsnorm")
        self.launches += 1
        if rows is None:
            self._note_stream_write()

    def _error_word(self) -> torch.Tensor:
        if self._tc_error is None:
            self._tc_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._tc_error

    def _check_limits(self, cache, tables=None) -> None:
        """Checked build: tell the kernels that follow how many pages the pool of `cache`
        has and how many rows the rotation tables have."""
        if self.checked and cache is not None:
            rows = tables[0].shape[0] if tables is not None else 0
            check(self.lib.mb_check_set_limits(cache.k.shape[0], rows, self._stream()),
                  "check limits")

    def check_errors(self) -> None:
        """Raise if a bounded wait inside a tcgen05 kernel ran out since the last check
        (reads one word from the device, so it synchronises). In the checked build also
        raise if a kernel met an index beyond its limit."""
        if self.checked:
            import ctypes

            word = (ctypes.c_int * 4)()
            check(self.lib.mb_check_read(word, self._stream()), "check read")
            if word[0]:
                kind = {1: "a page number beyond the pool", 2: "a block-table column beyond the table",
                        3: "a position beyond the rotation tables", 4: "a token id outside the vocabulary",
                        5: "a sequence number beyond the batch"}.get(word[0], f"kind {word[0]}")
                raise KernelError(f"bounds check: {kind}: {word[1]} (limit {word[2]}), "
                                  f"{word[3]} bad indices in all; the accesses were skipped")
        if not self._tc_pending or self._tc_error is None:
            self._tc_pending = False
            return
        self._tc_pending = False
        code = int(self._tc_error.item())
        if code:
            self._tc_error.zero_()
            role = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue or the softmax",
                    4: "the producer's drain or the wait for the output", 5: "the MMA issuer (P)",
                    6: "the meeting of a row's two softmax threads",
                    7: "a weight ring of a few-token product",
                    8: "the key tiles of the decode attention"}.get(code, f"code {code}")
            raise KernelError(f"a kernel gave up waiting in {role}; its output is invalid")

    # -- inputs that may still be an unevaluated norm (parts/norm.py: PendingNorm)

    def can_fuse_norm(self, rows: int, hidden: int, weight) -> bool:
        """Whether a few-token product can normalise its own input for this shape."""
        return (self.fuse_norm and self.skinny and rows <= 16 and hidden % 32 == 0
                and weight.dtype == torch.bfloat16)

    @staticmethod
    def _pending(x):
        return x if hasattr(x, "materialize") else None

    def _skinny_input(self, x):
        """The nine input arguments of the few-token products: (x, h, norm weight, rows, eps)
        and (partial sums of squares, their tiles per row, eps, row length)."""
        pending = self._pending(x)
        if pending is None:
            return _ptr(x), None, None, None, 0.0, None, 0, 0.0, 0
        scaled = getattr(pending, "ss_part", None)
        if scaled is not None:
            return (_ptr(pending.x), None, None, None, 0.0, _ptr(scaled), scaled.shape[1],
                    float(pending.eps), pending.size)
        return (None, _ptr(pending.h), _ptr(pending.weight), _ptr(pending.rows), float(pending.eps),
                None, 0, 0.0, 0)

    @_timed("residual product")
    def linear_residual(self, x, weight, bias, h, ctx, name, then_norm=None):
        """h += x . weight^T (+ bias) in the float32 stream when the few-token kernel takes
        the shape (returns None); otherwise the product lands in the buffer `name` and is
        returned for the next norm to add. `then_norm` names the norm part that follows
        (it has `weight`, `eps`, `size`): the kernel then also leaves that norm's output, up
        to the division by the row's rms, in `ctx.prenormed` (a `PendingScaled`), where the
        norm part picks it up instead of launching."""
        m, k = x.shape
        n = weight.shape[0]
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16) and h.dtype == torch.float32
                and self.lib.mb_gemm_skinny_supports(m, n, k)):
            fuse = (then_norm is not None and self.fuse_next_norm and n % 4 == 0
                    and getattr(then_norm, "size", None) == n
                    and getattr(then_norm, "weight", None) is not None
                    and then_norm.weight.dtype == torch.bfloat16)
            normed = ctx.buffer("normed", m, n) if fuse else None
            sums = ctx.buffer("norm_sums", m, n // 16, dtype="float32") if fuse else None
            stable = self._last_stream_write != self.launches + self.library_calls
            check(self.lib.mb_gemm_skinny(
                *self._skinny_input(x), _ptr(weight), _ptr(bias), _ptr(h), 3, m, n, k,
                _ptr(then_norm.weight) if fuse else None, _ptr(normed), _ptr(sums), int(stable),
                _ptr(self._error_word()), self._stream()), "linear_residual (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or n * k >= self.fed_min_elements
            self._note_stream_write()
            if fuse:
                from ..parts.norm import PendingScaled

                ctx.prenormed = (then_norm, PendingScaled(normed, sums, h, then_norm.weight,
                                                          then_norm.eps, ctx, n))
            return None
        out = ctx.buffer(name, m, n)
        self.linear(x, weight, bias, out)
        return out

    @_timed("product")
    def linear(self, x, weight, bias, out):
        pending = self._pending(x)
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
            raise KernelError(f"linear: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> "
                              f"{tuple(out.shape)} do not fit")
        self._rows(weight), self._rows(out)
        all_bf16 = (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                    and (bias is None or bias.dtype == torch.bfloat16))
        if (all_bf16 and self.skinny and self.lib.mb_gemm_skinny_supports(m, n, k)
                and (n * k <= self.skinny_max_elements or self.gemm == "simt")):
            check(self.lib.mb_gemm_skinny(*self._skinny_input(x), _ptr(weight), _ptr(bias),
                                          _ptr(out), 0 if out.dtype == torch.bfloat16 else 1, m, n, k,
                                          None, None, None, 0, _ptr(self._error_word()),
                                          self._stream()),
                  "linear (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or n * k >= self.fed_min_elements
            return
        if pending is not None:
            x = pending.materialize()
        self._rows(x)
        if all_bf16 and self.gemm in ("tcgen05", "auto") and self.lib.mb_gemm_tcgen05_supports(m, n, k):
            # Measured inside a 2048-token step on B200 (weights cold in L2) the library is
            # ahead on the plain products (q/k/v 8.5 us, o 7.3 us, down 17 us against 12, 12
            # and 33 us), so "auto" leaves them to it; the gated product is where this
            # package's kernel wins (see linear_swiglu).
            if self.gemm == "tcgen05":
                check(self.lib.mb_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out),
                                               int(out.dtype == torch.float32), m, n, k,
                                               _ptr(self._error_word()), 0, self._stream()),
                      "linear (tcgen05)")
                self.launches += 1
                self._tc_pending = True
                return
        if self.gemm != "simt" and all_bf16:
            return self._library_linear(x, weight, bias, out)
        check(self.lib.mb_gemm_simt(_ptr(x), _flag(x.dtype), _ptr(weight), _flag(weight.dtype),
                                    _ptr(bias), _flag(bias.dtype) if bias is not None else 0,
                                    _ptr(out), _flag(out.dtype), m, n, k, self._stream()),
              "linear")
        self.launches += 1

    def _library_linear(self, x, weight, bias, out):
        """bfloat16 operands, float32 accumulation in cuBLAS; the result is rounded once, to
        bfloat16 or (for logits) kept in float32."""
        if out.dtype == torch.bfloat16:
            if bias is None:
                torch.mm(x, weight.t(), out=out)
            else:
                torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
            if bias is not None:
                out.add_(bias.float())
        self.library_calls += 1

    @_timed("gated product")
    def linear_swiglu(self, x, weight, out, ctx, ahead=None):
        """out = silu(x . gate^T) * (x . up^T) for `weight` = [gate rows; up rows]: one kernel
        for few tokens, product then gate otherwise. `ahead`: the matrix that the product
        behind this one will stream; the few-token kernel asks L2 for it once its own weights
        are in (`look_ahead_max_bytes` bounds what is asked for)."""
        m, k = x.shape
        width = out.shape[1]
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and self.lib.mb_gemm_skinny_supports(m, width, k)
                and 2 * width * k <= self.skinny_max_elements):
            bytes_ahead = 0
            if (ahead is not None and m >= self.look_ahead_min_tokens and ahead.is_cuda
                    and ahead.is_contiguous()
                    and ahead.numel() * ahead.element_size() <= self.look_ahead_max_bytes):
                bytes_ahead = ahead.numel() * ahead.element_size()
            check(self.lib.mb_gemm_skinny_swiglu(*self._skinny_input(x), _ptr(weight), _ptr(out),
                                                 m, width, k, _ptr(ahead) if bytes_ahead else None,
                                                 bytes_ahead, _ptr(self._error_word()),
                                                 self._stream()),
                  "linear_swiglu (skinny)")
            self.launches += 1
            self._tc_pending = self._tc_pending or 2 * width * k >= self.fed_min_elements
            return
        if self._pending(x) is not None:
            x = x.materialize()
        if (self.gemm in ("tcgen05", "auto") and x.dtype == torch.bfloat16
                and weight.dtype == torch.bfloat16 and m >= 256 and width % 8 == 0
                and ((2 * width * k <= self.gated_max_elements
                      and 2 * m * width * k >= self.gated_min_products) or self.gemm == "tcgen05")
                and self.lib.mb_gemm_tcgen05_supports(m, width, k)):
            if k >= self.pair_min_k and self.lib.mb_gemm_pair_supports(m, width, k):
                # pairs of SMs sharing one 256-row MMA: a CTA loads a third less per output
                check(self.lib.mb_gemm_pair(_ptr(x), _ptr(weight), None, _ptr(out), 2, m, width, k,
                                            None, 0, 0.0, 0, None, None, None, None,
                                            _ptr(self._error_word()), self._stream()),
                      "linear_swiglu (tcgen05 pairs)")
            else:
                check(self.lib.mb_gemm_tcgen05_persistent(_ptr(x), _ptr(weight), None, _ptr(out), 2, m,
                                                          width, k, _ptr(self._error_word()),
                                                          self._stream()), "linear_swiglu (tcgen05)")
            self.launches += 1
            self._tc_pending = True
            return
        gate_up = ctx.buffer("gate_up", m, 2 * width)
        self.linear(x, weight, None, gate_up)
        self.swiglu(gate_up, out)

    def qkv_rope_store(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                       batch, cache):
        """The packed q/k/v projection with bias, then rotation of q and k and the store of
        k and v into the cache pages: one kernel for few tokens, two otherwise."""
        m, k = x.shape
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        self._check_limits(cache, tables)
        if (self.skinny and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and (bias is None or bias.dtype == torch.bfloat16) and cache is not None
                and cache.k.dtype == torch.bfloat16
                and self.lib.mb_gemm_skinny_qkv_supports(m, k, head_dim, rot)):
            self._qkv_rope_fused(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, cos, sin,
                                 rot, batch, cache)
            return
        if self._pending(x) is not None:
            x = x.materialize()
        with self._as("q/k/v product"):
            self.linear(x, weight, bias, qkv)
        self.rope_cache_write(qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache)

    @_timed("q/k/v + rotary + store")
    def _qkv_rope_fused(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, cos, sin, rot,
                        batch, cache):
        m, k = x.shape
        xp, hp, wp, _rows, eps, ssp, sst, sse, ssk = self._skinny_input(x)
        check(self.lib.mb_gemm_skinny_qkv_rope(
            xp, hp, wp, eps, ssp, sst, sse, ssk, _ptr(weight), _ptr(bias), _ptr(qkv), _ptr(cos), _ptr(sin), rot,
            _ptr(batch.positions), _ptr(batch.seq_of_token), _ptr(cache.table),
            cache.table.shape[1], _ptr(cache.k), _ptr(cache.v), m, k, num_heads, num_kv_heads,
            head_dim, cache.page_size, int(cache.write), self._stream()),
            "qkv_rope_store (skinny)")
        self.launches += 1

    @_timed("gate")
    def swiglu(self, gate_up, out):
        check(self.lib.mb_swiglu(_ptr(gate_up), _ptr(out), out.shape[0], out.shape[1],
                                 _flag(out.dtype), self._stream()), "swiglu")
        self.launches += 1

    @_timed("rotary + store")
    def rope_cache_write(self, qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache):
        cos, sin = tables if tables is not None else (None, None)
        rot = 2 * cos.shape[1] if cos is not None else 0
        store = int(cache is not None and cache.write)
        self._check_limits(cache, tables)
        if cache is not None and cache.k.dtype != qkv.dtype:
            raise KernelError("rope_cache_write: pages and activations differ in dtype")
        check(self.lib.mb_rope_store(
            _ptr(qkv), _ptr(cos), _ptr(sin), rot, _ptr(batch.positions),
            _ptr(batch.seq_of_token), _ptr(cache.table) if cache is not None else None,
            cache.table.shape[1] if cache is not None else 0,
            _ptr(cache.k) if cache is not None else None,
            _ptr(cache.v) if cache is not None else None,
            qkv.shape[0], num_heads, num_kv_heads, head_dim,
            cache.page_size if cache is not None else 1, store, _flag(qkv.dtype),
            self._stream()), "rope_cache_write")
        self.launches += 1

    def _splits(self, batch, num_kv_heads, group, rows_per_block, keys_per_tile) -> int:
        """Divide the keys over more blocks when the batch alone cannot fill the device."""
        if getattr(batch, "attention_splits", None):
            return batch.attention_splits
        if self.decode_splits is not None:
            return max(1, self.decode_splits)
        tiles = -(-batch.max_q_len * group // rows_per_block)
        blocks = batch.num_seqs * tiles * num_kv_heads
        key_tiles = -(-batch.max_kv_len // keys_per_tile)
        if blocks >= self.sm_count or key_tiles < 4:
            return 1
        return max(1, min(key_tiles // 2, -(-2 * self.sm_count // blocks), 64))

    def graph_splits(self, sequences: int, num_kv_heads: int) -> int:
        """How many ways the keys of each sequence are split in a captured decode step of
        `sequences` rows: sized to fill the device whatever the lengths turn out to be."""
        if self.decode_splits:
            return max(1, int(self.decode_splits))
        rows = max(1, sequences * num_kv_heads)
        if rows <= self.graph_small_rows:
            return max(1, min(self.graph_max_ranges_small,
                              self.graph_blocks_per_sm_small * self.sm_count // rows))
        return max(1, -(-self.graph_blocks_per_sm_large * self.sm_count // rows))

    def _prompt_cluster(self, batch, num_kv_heads, group) -> int:
        """CTAs per row tile of the tensor-memory attention: the CTAs of a cluster share a
        row tile and split its keys (merged through distributed shared memory). It pays only
        while the row tiles alone leave SMs idle, that is for portions of a prompt: measured
        on B200 (14 heads over 2 KV heads of 64, context 2048, replayed from a graph) a prompt
        in portions of 256 tokens (30 row tiles a step) took 11.3 ms whole, 10.7 ms in pairs and
        10.5 in fours; in portions of 512 (58 row tiles) 6.13 and 6.13 ms; in one step of 2048
        tokens (228 row tiles) 2.8 ms whole, 3.5 in pairs, 4.5 in fours."""
        if self.prompt_cluster is not None:
            return self.prompt_cluster
        tokens_per_tile = max(1, 128 // group)
        row_tiles = batch.num_seqs * -(-batch.max_q_len // tokens_per_tile) * num_kv_heads
        if batch.max_kv_len < 4 * 128:
            return 1
        cluster = 1
        while cluster < 4 and row_tiles * cluster * 2 <= self.sm_count:
            cluster *= 2
        return cluster

    def _prompt_splits(self, batch, num_kv_heads, group) -> int:
        """Key ranges per row tile of a prompt portion. Cutting the keys (and merging the
        ranges afterwards) shortens the chain of the last, heaviest row tile, but on B200 a
        2048-token portion got slower with every cut (3.87 ms whole, 4.09 ms in two, 4.43 ms
        in eight: the float32 partial results cost more than the tail), so prompts are not
        cut unless `prompt_splits` says so."""
        if self.prompt_splits is not None:
            return max(1, self.prompt_splits)
        return 1

    @_timed("attention")
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                        window, out, kernel: str | None = None):
        """`kernel` forces "mma" or "simt"; by default bfloat16 with a head size the
        tensor-core kernel takes runs there, everything else on the CUDA cores."""
        group = num_heads // num_kv_heads
        tokens = qkv.shape[0]
        self._check_limits(cache)
        tc_ok = (qkv.dtype == torch.bfloat16 and self.lib.mb_attention_tcgen05_supports(
            head_dim, cache.page_size, num_heads, num_kv_heads, qkv.shape[1]))
        if kernel == "tcgen05" and not tc_ok:
            raise KernelError("the tensor-memory attention takes bfloat16, head sizes 64 and 128 and "
                              "pages of 8 to 128 tokens")
        # prompt portions (at least one full tile of rows) go to the tensor-memory kernel
        if tc_ok and (kernel == "tcgen05" or (kernel is None and self.attention == "auto"
                                              and batch.max_q_len * group >= 128)):
            check(self.lib.mb_paged_attention_tcgen05(
                _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), cache.k.shape[0],
                _ptr(cache.table), cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len),
                _ptr(out), tokens, batch.num_seqs, batch.max_q_len, num_heads, num_kv_heads,
                head_dim, cache.page_size, float(scale), int(window),
                self._prompt_cluster(batch, num_kv_heads, group), _ptr(self._error_word()),
                self._stream()), "paged_attention (tcgen05)")
            self.launches += 1
            self._tc_pending = True
            return
        use_mma = (qkv.dtype == torch.bfloat16 and self.lib.mb_attention_mma_supports(head_dim)
                   and kernel != "simt")
        if kernel == "mma" and not use_mma:
            raise KernelError(f"the tensor-core attention takes bfloat16 with head size 64 or "
                              f"128, not {qkv.dtype} with {head_dim}")
        if use_mma:
            small = batch.max_q_len * group <= 16
            if small:
                splits = self._splits(batch, num_kv_heads, group, 16, 64)
                if self.decode_clusters and splits < 32 and kernel is None and cache.page_size >= 2:
                    cluster = self._cluster_of(splits)
                    self._decode_cluster(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                                         window, out, cluster, None, False)
                    return
            else:
                splits = self._prompt_splits(batch, num_kv_heads, group)
        else:
            splits = self._splits(batch, num_kv_heads, group, 16, 32)
        floats = self.lib.mb_attention_scratch_floats(tokens, num_heads, head_dim, splits)
        scratch = self._scratch_for(floats) if floats else None
        common = (_ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                  cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len),
                  _ptr(batch.seq_of_token), _ptr(out), _ptr(scratch),
                  scratch.numel() if scratch is not None else 0, tokens, batch.num_seqs,
                  batch.max_q_len, num_heads, num_kv_heads, head_dim, cache.page_size, float(scale),
                  int(window), splits)
        if use_mma:
            counters = None
            if splits > 1 and small:
                counters = self._counters_for(batch.num_seqs * num_kv_heads)
            check(self.lib.mb_paged_attention_mma(*common, _ptr(counters), self._stream()),
                  "paged_attention (mma)")
            self.launches += 1 if (splits == 1 or counters is not None) else 2
            return
        else:
            check(self.lib.mb_paged_attention_simt(*common, _flag(qkv.dtype), self._stream()),
                  "paged_attention")
        self.launches += 1 if splits == 1 else 2

    @_timed("attention")
    def _decode_cluster(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                        out, cluster, tables, raw):
        cos, sin = tables if tables is not None else (None, None)
        self._check_limits(cache, tables)
        # blocks that walk many key tiles each (a large batch) get their tiles by TMA
        fed = self._long_ranges(batch, num_kv_heads, head_dim)
        if fed:
            self._tc_pending = True
        check(self.lib.mb_paged_attention_decode_cluster(
            _ptr(qkv), qkv.shape[1], _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
            cache.table.shape[1], _ptr(batch.q_start), _ptr(batch.kv_len), _ptr(out),
            qkv.shape[0], batch.num_seqs, batch.max_q_len, num_heads, num_kv_heads, head_dim,
            cache.page_size, float(scale), int(window), cluster, _ptr(cos), _ptr(sin), int(raw),
            int(cache.write), cache.k.shape[0] if fed else 0, _ptr(self._error_word()) if fed else None,
            self._stream()), "paged_attention (decode clusters)")
        self.launches += 1

    def _long_ranges(self, batch, num_kv_heads, head_dim=64) -> bool:
        """Whether the cluster decode kernel takes its TMA-fed form. Head size 64: when its
        blocks will walk many key tiles each, that is when the batch alone brings more
        (sequence, KV head) pairs than `graph_small_rows`, so that few key ranges per pair fill
        the device (for small batches every tile is in shared memory before the kernel in
        front is done, and 16 bytes per thread and copy are the faster way there). Head size
        128, whose tiles cost a thread twice the copies: from 16 pairs on (measured on B200
        inside the captured decode step, 1.5B sizes: 8 sequences 1.56 -> 1.34 ms, 16: 2.10 ->
        1.76; 4 sequences 1.23 -> 1.25, one 1.18 -> 1.22)."""
        if self.decode_long_ranges is not None:
            return bool(self.decode_long_ranges)
        pairs = batch.num_seqs * num_kv_heads
        if head_dim > 64:
            return pairs >= self.graph_small_rows
        return pairs > 2 * self.graph_small_rows

    @staticmethod
    def _cluster_of(splits: int) -> int:
        cluster = 1
        while cluster * 2 <= min(splits, 8):
            cluster *= 2
        return cluster

    def qkv_attention(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                      cache, scale, window, out):
        """Projection of q/k/v, rotation, store of the new keys and values, and attention over
        the cache. For decode-like batches (bfloat16, head size 64 or 128, whole-head rotation
        or none) the projection is the plain product for that many tokens (few tokens: as many
        blocks as row tiles, where the fused q/k/v kernel has one per head; more: the
        library's, and the rotary/store kernel's launch is saved), and the attention kernel rotates the
        queries as it loads them and rotates and stores the new keys itself; otherwise
        `qkv_rope_store` followed by `paged_attention`. Measured on B200 inside the captured
        decode step (2048-token contexts): Qwen2.5-0.5B sizes, head size 64: batch 8 0.671 ->
        0.660 ms, batch 1 0.667 -> 0.633 ms, batch 16 1.23 -> 1.11 ms, batch 32 1.27 -> 1.19 ms, batch 64 1.49 ->
        1.42 ms; head size 128: 1.5B sizes batch 16 2.18 -> 2.07 ms, 7B sizes batch 8 3.93 ->
        3.73 ms. Which head sizes gain is the kernel's to say (mb_attention_decode_raw_pays)."""
        m, k = x.shape
        group = num_heads // num_kv_heads
        cos = tables[0] if tables is not None else None
        fused = (self.decode_clusters and weight.dtype == torch.bfloat16
                 and x.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
                 and cache is not None and cache.write and cache.k.dtype == torch.bfloat16
                 and cache.page_size >= 2
                 and qkv.dtype == torch.bfloat16 and batch.max_q_len * group <= 16
                 and self.lib.mb_attention_mma_supports(head_dim)
                 and self.lib.mb_attention_decode_raw_pays(head_dim)
                 and (cos is None or 2 * cos.shape[1] == head_dim))
        splits = self._splits(batch, num_kv_heads, group, 16, 64) if fused else 0
        if not fused or splits >= 32:
            self.qkv_rope_store(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                                batch, cache)
            self.paged_attention(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                                 out)
            return
        with self._as("q/k/v product"):
            self.linear(x, weight, bias, qkv)
        self._decode_cluster(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window,
                             out, self._cluster_of(splits), tables, True)

    @_timed("sampling")
    def argmax(self, logits, out):
        rows = logits.shape[0]
        if self._argmax_scratch is None or self._argmax_scratch.numel() < rows * 128:
            if self._argmax_scratch is not None:
                self._retired.append(self._argmax_scratch)
            self._argmax_scratch = torch.empty(max(rows, 64) * 128, dtype=torch.float32,
                                               device=self.device)
        check(self.lib.mb_argmax(_ptr(logits), _ptr(out), rows, logits.shape[1],
                                 _ptr(self._argmax_scratch), self._stream()), "argmax")
        self.launches += 2 if logits.shape[1] >= 16384 else 1

    @_timed("sampling")
    def sample(self, logits, temperature, top_p, u, out):
        check(self.lib.mb_sample(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(u), _ptr(out),
                                 logits.shape[0], logits.shape[1], self._stream()), "sample")
        self.launches += 1
