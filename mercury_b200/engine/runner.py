"""The step function: run a batch of (sequence, its next tokens) from the cache and return
the logits at the wanted places.

`ModelRunner` owns the model's weights, the page tensors, the per-request state tensors,
the cache manager and the activation buffers. `step(entries)` is the only way tokens go
through the model: trace replay, the scheduler's engine and the benchmarks all call it.
The reference's counterpart is `ModelRunner.execute` (mercury/runner.py:106-178), which
runs one forward per prompt and another for the decode batch and samples inside; here one
pass takes prompt portions and decode tokens together and sampling is a separate call.
"""

from __future__ import annotations

import time
from pathlib import Path

import torch

from ..cache.manager import CacheManager, OutOfPages, Sequence
from ..config.model_config import ModelConfig, architecture_named, read_model_config
from ..models.model import Model
from ..parts.base import PartSetup
from ..weights.loader import check_tensors, read_checkpoint
from .batch import BatchBuffers, StepBatch, StepEntry


class Workspace:
    """Activation buffers by name, allocated once for the largest step and handed out as
    row slices, so that addresses stay the same from step to step."""

    # buffers whose row count follows what a step asks for (logits of the wanted rows), not
    # the step's token count: they start small and grow
    ROW_SIZED = ("logits", "normed_rows")

    def __init__(self, device, dtype, max_rows: int):
        self.device = device
        self.dtype = dtype
        self.max_rows = max_rows
        self._buffers: dict[tuple, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []   # outgrown buffers: captured graphs still use them

    def get(self, name: str, rows: int, cols: int, dtype=None) -> torch.Tensor:
        dt = self.dtype if dtype is None else (torch.float32 if dtype == "float32" else dtype)
        key = (name, cols, dt)
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            if buf is not None:
                self._retired.append(buf)
                capacity = max(rows, 2 * buf.shape[0])
            else:
                capacity = max(rows, 64) if name in self.ROW_SIZED else max(rows, self.max_rows)
            buf = torch.empty((capacity, cols), dtype=dt, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]


class StepContext:
    """What parts see during one step: the kernels, the batch, buffers, the page size."""

    def __init__(self, ops, workspace: Workspace, page_size: int, dtype):
        self.ops = ops
        self.workspace = workspace
        self.page_size = page_size
        self.dtype = dtype
        self.batch: StepBatch | None = None
        self.prenormed = None      # (norm part, its output) left by the product before it

    def buffer(self, name: str, rows: int, cols: int, dtype=None) -> torch.Tensor:
        return self.workspace.get(name, rows, cols, dtype)


class ModelRunner:
    def __init__(
        self,
        model: str | Path | None = None,
        *,
        dtype: torch.dtype = torch.bfloat16,
        device: str = "cuda",
        page_size: int = 16,
        num_pages: int = 256,
        max_seqs: int = 8,
        max_step_tokens: int = 2048,
        max_model_len: int | None = None,
        ops=None,
        config: ModelConfig | None = None,
        tensors: dict[str, torch.Tensor] | None = None,
        cuda_graphs: bool = True,
        poison_pages: bool = False,
    ):
        """`model` is a folder with config.json and safetensors; or pass `config` and
        `tensors` (a `{name: tensor}` dictionary) directly. `ops` is the kernel set; by
        default the CUDA kernels, which refuse to load without a GPU. `poison_pages` is a
        debugging aid: every page is filled with NaN when it gets its first holder and when
        it goes back to the free list, so that a kernel that reads a key it should not see
        (beyond a sequence's length, on a page of another request, left by an earlier
        owner) yields NaN instead of a plausible number."""
        self.device = torch.device(device)
        self.dtype = dtype
        if config is None:
            _entry, config = read_model_config(model)
        self.config = config
        entry = architecture_named(config.architecture)
        self.spec = entry.describe(config)
        self.model = Model(self.spec)
        specs = self.model.tensor_specs()
        if tensors is None:
            tensors = read_checkpoint(model, specs, self.model.optional_tensors())
        else:
            check_tensors({n: (tuple(t.shape), t.is_floating_point()) for n, t in tensors.items()},
                          specs, self.model.optional_tensors())
        if ops is None:
            from ..kernels.ops import CudaOps

            ops = CudaOps(self.device)
        self.ops = ops
        self.max_model_len = min(max_model_len or self.spec.max_positions, self.spec.max_positions)
        setup = PartSetup(self.device, dtype, ops, self.max_model_len)
        self.model.load(tensors, setup)

        self.page_size = page_size
        self.max_seqs = max_seqs
        self.max_step_tokens = max_step_tokens
        self.cache = CacheManager(self.model.group_windows, num_pages, page_size, max_seqs)
        self.kv_layers: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        for cache_id, layer in self.model.cache_layers.items():
            pages = self.cache.pools[layer.group].num_pages
            store = torch.zeros(
                (2, pages, layer.need.num_kv_heads, page_size, layer.need.head_dim),
                dtype=dtype, device=self.device)
            self.kv_layers[cache_id] = (store[0], store[1])
        self.states: dict[tuple[int, int], torch.Tensor] = {
            key: torch.zeros((max_seqs, *need.shape), dtype=need.dtype, device=self.device)
            for key, need in self.model.state_needs.items()
        }
        self.has_state = bool(self.states)
        self.poison_pages = bool(poison_pages)
        if self.poison_pages:
            self.cache.keep_journal()
            for k, v in self.kv_layers.values():
                k.fill_(float("nan"))
                v.fill_(float("nan"))
        max_pages = -(-self.max_model_len // page_size)
        self.buffers = BatchBuffers(self.device, max_step_tokens, max_seqs, max_pages,
                                    max(1, len(self.model.group_windows)),
                                    pin=self.device.type == "cuda",
                                    append_only=[w == 0 for w in self.model.group_windows] or None)
        self.workspace = Workspace(self.device, dtype, max_step_tokens)
        self.ctx = StepContext(ops, self.workspace, page_size, dtype)
        self.steps = 0
        self.max_pages = max_pages
        # (the checked build of the kernels copies its limits from host memory before every
        # attention call and is read back after every step: it runs without graphs)
        self.use_graphs = (cuda_graphs and self.device.type == "cuda" and self.model.capturable
                           and not getattr(ops, "checked", False))
        self._graphs: dict[int, tuple] = {}
        self.dependent_launch_buckets = 16   # largest batch bucket captured with dependent launch
        self.graph_replays = 0
        self.graph_launches = 0      # kernels run by replayed graphs
        self._shape_graphs: dict[tuple, tuple] = {}   # other steps, by the shape of the batch
        self._shape_seen: dict[tuple, int] = {}
        self.max_shape_graphs = 16
        # opt-in: every step runs eagerly with CUDA events around each kernel-set call, and
        # `last_kernel_ms` holds the step's milliseconds per class of call (a step so timed
        # waits for the device; this is for looking at a step, not for serving)
        self.time_kernels = False
        self.last_prepare_s = 0.0          # host seconds the last step's preparation took
        self.last_kernel_ms: dict[str, float] = {}

    # ------------------------------------------------------------------ sizes

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def kv_bytes_per_token(self) -> int:
        """Bytes of keys and values one token occupies over all cache layers
        (mercury/config.py:73-81)."""
        elem = torch.finfo(self.dtype).bits // 8
        return sum(2 * l.need.num_kv_heads * l.need.head_dim * elem
                   for l in self.model.cache_layers.values())

    # ------------------------------------------------------------------ sequences

    def open(self, seq_id: str) -> Sequence:
        return self.cache.open(seq_id)

    def close(self, seq: Sequence) -> None:
        self.cache.close(seq)
        self._poison()

    def _poison(self) -> None:
        """Overwrite with NaN the pages that changed hands since the last call."""
        if not self.poison_pages:
            return
        for group, pages in enumerate(self.cache.drain_journal()):
            if not pages:
                continue
            index = torch.tensor(pages, dtype=torch.long, device=self.device)
            for cache_id, layer in self.model.cache_layers.items():
                if layer.group == group:
                    for side in self.kv_layers[cache_id]:
                        side.index_fill_(0, index, float("nan"))

    def _reset_fresh_state(self) -> None:
        fresh, self.cache.fresh_slots = self.cache.fresh_slots, []
        if self.states and fresh:
            index = torch.tensor(fresh, dtype=torch.long, device=self.device)
            for state in self.states.values():
                state.index_fill_(0, index, 0)

    # ------------------------------------------------------------------ the step

    def prepare(self, entries: list[StepEntry], sampled: torch.Tensor | None = None,
                **capacities) -> StepBatch:
        """Provide pages for the entries' tokens and put the batch on the device. Token ids
        that an entry marks as `late` are taken on the device from `sampled`, the tokens the
        step before has sampled (and the host may not have read yet)."""
        started = time.perf_counter()
        for e in entries:
            if not e.tokens:
                raise ValueError(f"{e.seq.seq_id}: an entry needs at least one token")
            end = e.seq.num_computed + len(e.tokens)
            if end > self.max_model_len:
                raise ValueError(f"{e.seq.seq_id}: {end} tokens exceed max_model_len "
                                 f"{self.max_model_len}")
            if not self.cache.ensure(e.seq, end):
                raise OutOfPages(
                    f"{e.seq.seq_id}: no pages left for tokens up to {end} "
                    f"(available per group: {self.cache.num_available()})")
        self._reset_fresh_state()
        self._poison()
        batch = self.buffers.build(entries, self.page_size, **capacities)
        if batch.late_tokens:
            if sampled is None:
                raise ValueError("an entry's token is to come from the step before, but its "
                                 "sampled tokens were not given")
            self.ops.patch_tokens(batch.token_ids, batch.token_from, sampled)
        self.last_prepare_s = time.perf_counter() - started
        return batch

    def run(self, batch: StepBatch) -> torch.Tensor | None:
        """The model pass over a prepared batch; float32 logits `[wanted, vocab]` or None."""
        self.ctx.batch = batch
        pin = getattr(self.ops, "pin_stream", None)
        if pin is None:
            return self.model.forward(self.ctx, self.kv_layers, self.states)
        pin()
        try:
            return self.model.forward(self.ctx, self.kv_layers, self.states)
        finally:
            self.ops.unpin_stream()

    def finish(self, entries: list[StepEntry]) -> None:
        """Book the tokens as computed: full pages become shareable, passed pages go back."""
        for e in entries:
            self.cache.advance(e.seq, e.seq.num_computed + len(e.tokens), e.hashes)
        self.steps += 1

    def launch_count(self, replayed: bool = True) -> int:
        """Kernels launched so far by this runner's kernel set: its own and the library's,
        and (with `replayed`) those inside replayed graphs, which no Python call sees."""
        direct = getattr(self.ops, "launches", 0) + getattr(self.ops, "library_calls", 0)
        return direct + (self.graph_launches if replayed else 0)

    # ------------------------------------------------------------------ decode graphs

    def _bucket(self, count: int) -> int:
        size = 1
        while size < count:
            size *= 2
        return min(size, self.max_seqs)

    def _graph_splits(self, bucket: int) -> int | None:
        """How many ways the keys of each sequence are split in a captured step of `bucket`
        sequences: the grid is fixed at capture, so the kernel set sizes it for its device
        (`graph_splits`); a kernel set without an opinion decides per launch."""
        choose = getattr(self.ops, "graph_splits", None)
        if choose is None:
            return None
        kv_heads = max((l.need.num_kv_heads for l in self.model.cache_layers.values()), default=1)
        return choose(bucket, kv_heads)

    def _decode_with_graph(self, entries: list[StepEntry], sampled=None) -> torch.Tensor | None:
        """Decode-only steps (one token per entry) replay a CUDA graph captured once per
        batch-size bucket: the launch sequence is fixed and everything that varies (tokens,
        positions, block tables, lengths) is read by the kernels from the step's device
        buffer, whose layout is fixed by the bucket."""
        bucket = self._bucket(len(entries))
        wanted = [i for i, e in enumerate(entries) if e.want]
        capacities = dict(token_capacity=bucket, seq_capacity=bucket, page_capacity=self.max_pages,
                          row_capacity=bucket)
        # every row of the bucket gets logits; rows nobody asked for are dropped below
        batch = self.prepare(entries, sampled, **capacities)
        batch.attention_splits = self._graph_splits(bucket)
        held = self._graphs.get(bucket)
        if held is None:
            self.run(batch)                       # warm-up: allocates buffers, loads kernels
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = self.launch_count(replayed=False)
            # Inside a captured decode step every kernel may be scheduled while the one in
            # front drains (programmatic dependent launch): the kernels prefetch weights and
            # cached keys before they wait. Prompt steps run without it: their grids are
            # larger than the device and early blocks would only take room (the same holds
            # for decode batches beyond 16, whose products are the library's).
            dependent = (getattr(self.ops, "set_dependent_launch", None)
                         if bucket <= self.dependent_launch_buckets else None)
            if dependent is not None:
                dependent(True)
            try:
                with torch.cuda.graph(graph):
                    logits = self.run(batch)
            finally:
                if dependent is not None:
                    dependent(False)
            kernels = self.launch_count(replayed=False) - before
            held = self._graphs[bucket] = (graph, logits, kernels)
        graph, logits, kernels = held
        graph.replay()
        self.graph_replays += 1
        self.graph_launches += kernels
        # kernels with bounded waits (TMA-fed products) report through an error word; inside a
        # graph nobody looks at it, so it is read now and then (a read is a synchronisation)
        check = getattr(self.ops, "check_errors", None)
        if check is not None and self.graph_replays % 256 == 0:
            self.ops._tc_pending = True
            check()
        self.finish(entries)
        if not wanted:
            return None
        if len(wanted) == len(entries):
            return logits[:len(entries)]
        return logits[torch.tensor(wanted, device=self.device)]

    def _step_with_shape_graph(self, entries: list[StepEntry], key: tuple,
                               sampled=None) -> torch.Tensor | None:
        """Steps other than pure decoding are captured per batch shape: the launch sequence
        of a step depends only on (tokens, sequences, longest portion, wanted rows), and a
        server cutting prompts into portions of one size sees the same shapes again and
        again. A shape is captured the second time it is seen; at most `max_shape_graphs`
        are kept. Without this a 2048-token step is bound by the Python launch loop."""
        tokens, seqs, _max_q, rows = key
        batch = self.prepare(entries, sampled, token_capacity=tokens, seq_capacity=seqs,
                             page_capacity=self.max_pages)
        batch.attention_splits = self._graph_splits(seqs)
        held = self._shape_graphs.get(key)
        if held is None:
            if len(self._shape_graphs) >= self.max_shape_graphs:
                self._shape_graphs.pop(next(iter(self._shape_graphs)))
            self.run(batch)                       # warm-up outside the capture
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = self.launch_count(replayed=False)
            with torch.cuda.graph(graph):
                logits = self.run(batch)
            kernels = self.launch_count(replayed=False) - before
            held = self._shape_graphs[key] = (graph, logits, kernels)
        graph, logits, kernels = held
        graph.replay()
        self.graph_replays += 1
        self.graph_launches += kernels
        # the graph may hold kernels with bounded waits, which report through an error word;
        # reading it waits for the device, and a step of prompt portions that nobody reads
        # back would otherwise never let the host prepare the next step meanwhile (four
        # portions of 512 tokens took 6.8 ms with a read per step where they take 4.1 ms
        # without): so it is read now and then, as in the decode path
        check = getattr(self.ops, "check_errors", None)
        if check is not None and self.graph_replays % 64 == 0:
            if getattr(self.ops, "gemm", "library") != "library":
                self.ops._tc_pending = True
            check()
        self.finish(entries)
        return logits if rows else None

    @torch.inference_mode()
    def step(self, entries: list[StepEntry], sampled: torch.Tensor | None = None
             ) -> torch.Tensor | None:
        """Run exactly the tokens given, as one batch, from the cache that earlier steps
        left; returns the logits at the wanted places in the order of the entries and of
        each entry's `want` (None if nothing is wanted). The tensor returned is a view of a
        buffer that the next step overwrites. `sampled` (device int32) supplies the token
        ids of entries marked `late`."""
        timing = self.time_kernels and hasattr(self.ops, "begin_timing")
        if timing:
            self.ops.begin_timing()
            try:
                batch = self.prepare(entries, sampled)
                logits = self.run(batch)
            finally:
                self.last_kernel_ms = self.ops.end_timing()
            self.ops.check_errors()
            self.finish(entries)
            return logits
        if (self.use_graphs and len(entries) <= self.max_seqs
                and all(len(e.tokens) == 1 and e.want in ([], [0]) for e in entries)):
            return self._decode_with_graph(entries, sampled)
        if self.use_graphs:
            key = (sum(len(e.tokens) for e in entries), len(entries),
                   max(len(e.tokens) for e in entries), sum(len(e.want) for e in entries))
            if key in self._shape_graphs or self._shape_seen.get(key, 0) >= 1:
                return self._step_with_shape_graph(entries, key, sampled)
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            self._shape_seen[key] = 1
        batch = self.prepare(entries, sampled)
        logits = self.run(batch)
        check = getattr(self.ops, "check_errors", None)
        if check is not None:
            check()
        self.finish(entries)
        return logits


def kv_bytes_per_token_of(folder, dtype: torch.dtype) -> int:
    """Cache bytes per token of the model under `folder`, without loading its weights."""
    entry, config = read_model_config(folder)
    model = Model(entry.describe(config))
    elem = torch.finfo(dtype).bits // 8
    return sum(2 * l.need.num_kv_heads * l.need.head_dim * elem for l in model.cache_layers.values())
