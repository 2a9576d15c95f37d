"""What a part of a model is, and the registries that parts are chosen from.

A model is put together from parts: a mixer (attention here), a feed-forward, norms, a
position encoding, and the arrangement of these in a block. A part gets every size and
constant as a constructor parameter, declares the checkpoint tensors it owns, and never
learns which model it is in. Which part a layer uses is data (`PartSpec`: a registered
kind plus its parameters), so one model may use different mixers and feed-forwards in
different layers.

Interfaces
----------
Embedding (`register_embedding`):
    forward(token_ids, ctx) -> Tensor         the float32 residual stream [T, hidden]

Head (`register_head`):
    forward(rows, ctx) -> Tensor              float32 logits [rows, vocab] of normalised rows

Every part:
    tensor_specs() -> list[TensorSpec]        the checkpoint tensors it reads, by full name
    load(tensors, setup)                      take (and pack) them; `setup` is a `PartSetup`
    capturable                                True if forward() can be recorded in a CUDA graph

Mixer (`register_mixer`):
    cache_need() -> CacheNeed | None          pages of keys and values it wants, if any
    state_need() -> StateNeed | None          fixed-size per-request state it wants, if any
    forward(x, ctx, cache, state) -> Tensor   x: [T, hidden] in the activation dtype;
                                              `cache` is a `LayerCache` or None, `state` a
                                              `[slots, *shape]` tensor or None

FeedForward (`register_feed_forward`):
    forward(x, ctx) -> Tensor

Two optional protocols let a mixer or feed-forward fuse with its neighbours; a part that
declares neither is handed a plain tensor and returns its output, as above.
    accepts_pending_norm = True    x may be a `PendingNorm` (parts/norm.py): the norm before
                                   the part has not run, the part's first kernel does it
    adds_to_residual = True        forward(..., residual=h, then_norm=norm) may add the output
                                   into the float32 stream itself and return None; it may
                                   also leave `then_norm`'s output in `ctx.prenormed`

Norm (`register_norm`):
    add_norm(h, delta, ctx, rows=None, defer=False) -> Tensor | PendingNorm
        h: [T, hidden] float32 residual stream, updated in place to h + delta when delta is
        given; returns norm(h) in the activation dtype. With `rows` (int32 indices) only
        those rows are normalised and returned, and h is left as it was.

PositionEncoding (`register_position_encoding`):
    fused_form() -> "rotary" | "identity" | None   what the rotate-and-store kernels can do
                                              for this encoding: rotate by its tables, leave
                                              q and k as they are, or nothing (then `apply`)
    rotary_tables() -> (cos, sin) | None      float32 [positions, rotary_dim/2] tables for
                                              the fused rotate-and-store kernel, or None
    apply(qkv, layout, ctx)                   for encodings the fused kernel does not cover:
                                              changes q and k of the packed rows in place

Arrangement (`register_arrangement`): how mixers, feed-forward and norms sit in a block.
    mixers() -> list[Mixer]                   every mixer of the block, in a fixed order; a
                                              `LayerCall` names one cache layer per mixer
    parts() -> list[Part]                     everything that owns checkpoint tensors
    forward(h, delta, ctx, caches, states) -> Tensor
                                              `caches[i]` / `states[i]` belong to `mixers()[i]`
                                              (None where that mixer wants none); returns the
                                              new pending delta (None if it is already in the
                                              stream); an arrangement with `first_norm()`
                                              also takes `next_norm=`
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part expects. `kind` is "float" or "int"; `init` says how the
    random-weights mode fills it: "normal" = N(0, std), "ones_normal" = 1 + N(0, std)."""

    name: str
    shape: tuple[int, ...]
    kind: str = "float"
    init: str = "normal"
    std: float = 0.02


@dataclass(frozen=True)
class PartSpec:
    """A registered kind of part and the parameters to build it with."""

    kind: str
    params: dict = field(default_factory=dict)


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per token. `window` = 0 keeps every key; a positive
    window keeps the last `window` (pages behind it are given back)."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one `shape` tensor of `dtype` per live request,
    zeroed when the request is admitted."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PartSetup:
    """What a part may know of its surroundings when it loads: where tensors live, the
    activation dtype, the kernels, and how many positions the engine will ever ask for."""

    device: torch.device
    dtype: torch.dtype
    ops: Any
    max_positions: int
    _by_name: dict = field(default_factory=dict)
    _derived: dict = field(default_factory=dict)

    def place(self, tensor: torch.Tensor) -> torch.Tensor:
        """Move a checkpoint tensor to the device under the storage rule: in the float32
        engine every floating tensor becomes float32; in the bfloat16 engine 16-bit tensors
        are held in bfloat16 and a tensor stored in 32-bit stays 32-bit; integer tables
        become int32."""
        if tensor.is_floating_point():
            if self.dtype == torch.float32 or tensor.dtype == torch.float32:
                target = torch.float32
            else:
                target = torch.bfloat16
        else:
            target = torch.int32
        return tensor.to(device=self.device, dtype=target).contiguous()

    def place_named(self, tensors: dict, name: str) -> torch.Tensor:
        """`place(tensors[name])`, once per checkpoint tensor: two parts that read the same
        tensor (a head tied to the embedding table) share one buffer on the device."""
        if name not in self._by_name:
            self._by_name[name] = self.place(tensors[name])
        return self._by_name[name]

    def derived(self, key: tuple, make: Callable[[], Any]) -> Any:
        """A table computed from constants (rotation angles, say), made once per `key` and
        shared by every part that asks for the same one."""
        if key not in self._derived:
            self._derived[key] = make()
        return self._derived[key]


@dataclass
class LayerCache:
    """One cache layer as a mixer sees it: K and V pages `[pages, kv_heads, page_size,
    head_dim]`, the block table of its group for this step `[sequences, max_pages]` int32
    (-1 where a page was given back), and whether this call stores new keys or only reads
    what another layer stored."""

    k: torch.Tensor
    v: torch.Tensor
    page_size: int
    table: torch.Tensor
    write: bool = True


class Part:
    # Whether forward() may be recorded into a CUDA graph: it must launch the same kernels
    # whatever the batch holds and never read device memory from the host. Parts that do
    # not say so are assumed unsafe, and a model holding one runs without graphs.
    capturable = False

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor], setup: PartSetup) -> None:
        pass


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def skips_cached_prefix(self) -> bool:
        """Whether a request may start behind a prefix whose pages another request left in
        the cache, so that this mixer never sees the prefix's tokens. True for a mixer whose
        memory of earlier tokens is in the pages alone; a mixer with state of its own has to
        run every token."""
        return self.state_need() is None

    def forward(self, x, ctx, cache, state):  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):  # pragma: no cover - interface
        raise NotImplementedError


class Norm(Part):
    def add_norm(self, h, delta, ctx, rows=None):  # pragma: no cover - interface
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids, ctx):  # pragma: no cover - interface
        raise NotImplementedError


class Head(Part):
    def forward(self, rows, ctx):  # pragma: no cover - interface
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_form(self) -> str | None:
        return None

    def rotary_tables(self):
        return None

    def apply(self, qkv, layout, ctx) -> None:
        pass


# ------------------------------------------------------------------------------ registries

_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position_encoding": {},
    "arrangement": {},
    "embedding": {},
    "head": {},
}


def _register(family: str, kind: str, factory: Callable[..., Any]) -> None:
    _REGISTRIES[family][kind] = factory


def register_mixer(kind: str, factory) -> None:
    _register("mixer", kind, factory)


def register_feed_forward(kind: str, factory) -> None:
    _register("feed_forward", kind, factory)


def register_norm(kind: str, factory) -> None:
    _register("norm", kind, factory)


def register_position_encoding(kind: str, factory) -> None:
    _register("position_encoding", kind, factory)


def register_arrangement(kind: str, factory) -> None:
    _register("arrangement", kind, factory)


def register_embedding(kind: str, factory) -> None:
    _register("embedding", kind, factory)


def register_head(kind: str, factory) -> None:
    _register("head", kind, factory)


def build_part(family: str, spec: PartSpec):
    """Instantiate `spec.kind` of `family` with `spec.params` as keyword arguments."""
    table = _REGISTRIES[family]
    if spec.kind not in table:
        raise KeyError(
            f"no {family} of kind {spec.kind!r} is registered; known: {', '.join(sorted(table))}"
        )
    return table[spec.kind](**spec.params)
