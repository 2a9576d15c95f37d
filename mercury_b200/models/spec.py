"""A model as data: which parts make each block, and the order in which blocks run.

`schedule` is the execution order, one `LayerCall` per step of the stack. A call names the
block to run and the cache layer its mixer uses; the same block may be called twice (each
call with a cache layer of its own), and a call may read the cache layer that an earlier
call stored (`writes_cache=False`) instead of storing its own keys. For a block with
several mixers `cache` is a tuple, one entry (or None) per mixer in the order of the
block's `mixers()`.

The embedding and the head are parts like the others (`PartSpec`s of the "embedding" and
"head" families). `optional_tensors` names checkpoint tensors that may be present although
no part reads them (a tied model's stored copy of its head).
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int | tuple | None = None
    writes_cache: bool = True

    def caches(self, mixers: int) -> tuple:
        """One cache layer (or None) per mixer of the block."""
        if isinstance(self.cache, tuple):
            if len(self.cache) != mixers:
                raise ValueError(f"block {self.block} has {mixers} mixers but its call names "
                                 f"{len(self.cache)} cache layers")
            return self.cache
        return (self.cache,) + (None,) * (mixers - 1)


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    blocks: list[PartSpec]
    schedule: list[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    optional_tensors: tuple[str, ...] = ()
    eos_token_ids: tuple[int, ...] = ()
    extra: dict = field(default_factory=dict)
