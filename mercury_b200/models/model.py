"""The generic model: an embedding, blocks run in the order the schedule gives, a final
norm on the rows whose logits are wanted, and the output head. It knows parts and their
interfaces only; which architecture it is running is in the `ModelSpec` it was given."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import PartSetup, build_part
from ..parts.base import CacheNeed, LayerCache, StateNeed, TensorSpec
from ..parts.embedding import OutputHead, TokenEmbedding
from .spec import ModelSpec


@dataclass(frozen=True)
class CacheLayer:
    """One cache layer: what it stores and which group's pages it lies on."""

    need: CacheNeed
    group: int


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = TokenEmbedding(spec.vocab_size, spec.hidden_size, spec.embedding_weight)
        self.blocks = [build_part("arrangement", b) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = OutputHead(spec.vocab_size, spec.hidden_size, spec.head_weight)
        self._plan_caches()
        self.capturable = all(part.capturable for part in self._parts()) and all(
            getattr(block.mixer, "position", None) is None or block.mixer.position.capturable
            for block in self.blocks)

    # ------------------------------------------------------------------ layout of caches

    def _plan_caches(self) -> None:
        needs: dict[int, CacheNeed] = {}
        for call in self.spec.schedule:
            mixer = self.blocks[call.block].mixer
            need = mixer.cache_need()
            if need is None:
                continue
            if call.cache is None:
                raise ValueError(f"block {call.block} keeps keys but its call names no cache layer")
            if call.writes_cache:
                if call.cache in needs:
                    raise ValueError(f"cache layer {call.cache} is stored by two calls")
                needs[call.cache] = need
        for call in self.spec.schedule:
            mixer = self.blocks[call.block].mixer
            if mixer.cache_need() is not None and call.cache not in needs:
                raise ValueError(f"cache layer {call.cache} is read but no call stores it")
        self.group_windows: list[int] = []
        self.cache_layers: dict[int, CacheLayer] = {}
        for cache_id in sorted(needs):
            window = needs[cache_id].window
            if window not in self.group_windows:
                self.group_windows.append(window)
            self.cache_layers[cache_id] = CacheLayer(needs[cache_id], self.group_windows.index(window))
        self.state_needs: dict[int, StateNeed] = {}
        for index, call in enumerate(self.spec.schedule):
            need = self.blocks[call.block].mixer.state_need()
            if need is not None:
                self.state_needs[index] = need

    # ------------------------------------------------------------------ weights

    def _parts(self):
        yield self.embedding
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> list[TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for part in self._parts():
            for spec in part.tensor_specs():
                specs.setdefault(spec.name, spec)
        return list(specs.values())

    def optional_tensors(self) -> set[str]:
        """Tensors a checkpoint may carry although this model has no home for them: a tied
        model's copy of the head (mercury/model/loader.py:88-91)."""
        return {"lm_head.weight"} if self.spec.head_weight is None else set()

    def load(self, tensors: dict[str, torch.Tensor], setup: PartSetup) -> None:
        self.embedding.load(tensors, setup)
        for block in self.blocks:
            for part in block.parts():
                part.load(tensors, setup)
        self.final_norm.load(tensors, setup)
        self.head.load(tensors, setup, tied_table=self.embedding.table)

    def weight_bytes(self) -> int:
        seen: dict[int, int] = {}
        for part in self._parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor):
                    seen[value.data_ptr()] = value.numel() * value.element_size()
        return sum(seen.values())

    # ------------------------------------------------------------------ one pass

    def forward(self, ctx, kv_layers: dict[int, tuple], states: dict[int, torch.Tensor]):
        """Run the tokens of `ctx.batch`; returns float32 logits `[wanted rows, vocab]`, or
        None when no row is wanted. `kv_layers[c]` is (K pages, V pages) of cache layer c."""
        batch = ctx.batch
        h = self.embedding.forward(batch.token_ids, ctx)
        delta = None
        for index, call in enumerate(self.spec.schedule):
            block = self.blocks[call.block]
            cache = None
            if call.cache is not None and call.cache in self.cache_layers:
                k, v = kv_layers[call.cache]
                group = self.cache_layers[call.cache].group
                cache = LayerCache(k, v, ctx.page_size, batch.tables[group], call.writes_cache)
            # the norm that opens the next call's block, which this block's last product
            # may compute ahead (the final norm picks rows, so it is left alone)
            following = None
            if index + 1 < len(self.spec.schedule):
                nxt = self.blocks[self.spec.schedule[index + 1].block]
                following = getattr(nxt, "first_norm", lambda: None)()
            if following is not None:
                delta = block.forward(h, delta, ctx, cache, states.get(index), next_norm=following)
            else:
                delta = block.forward(h, delta, ctx, cache, states.get(index))
        if batch.num_logit_rows == 0:
            return None
        rows = self.final_norm.add_norm(h, delta, ctx, rows=batch.logit_rows, defer=True)
        return self.head.forward(rows, ctx)
