"""A model as data: which parts make each block, and the order in which blocks run.

`schedule` is the execution order, one `LayerCall` per step of the stack. A call names the
block to run and the cache layer its mixer uses; the same block may be called twice (each
call with a cache layer of its own), and a call may read the cache layer that an earlier
call stored (`writes_cache=False`) instead of storing its own keys.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int | None = None
    writes_cache: bool = True


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_weight: str
    blocks: list[PartSpec]
    schedule: list[LayerCall]
    final_norm: PartSpec
    head_weight: str | None
    eos_token_ids: tuple[int, ...] = ()
    extra: dict = field(default_factory=dict)
