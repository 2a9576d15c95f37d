"""The generic model: an embedding, blocks run in the order the schedule gives, a final
norm on the rows whose logits are wanted, and the output head. It knows parts and their
interfaces only; which architecture it is running is in the `ModelSpec` it was given."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts import PartSetup, build_part
from ..parts.base import CacheNeed, LayerCache, StateNeed, TensorSpec
from .spec import ModelSpec


@dataclass(frozen=True)
class CacheLayer:
    """One cache layer: what it stores and which group's pages it lies on."""

    need: CacheNeed
    group: int


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.blocks = [build_part("arrangement", b) for b in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self._plan_caches()
        self.capturable = all(part.capturable for part in self._parts()) and all(
            getattr(mixer, "position", None) is None or mixer.position.capturable
            for block in self.blocks for mixer in block.mixers())
        # a request may start behind another request's cached pages only if every mixer's
        # memory of the prefix lies in those pages
        self.skips_cached_prefix = all(mixer.skips_cached_prefix()
                                       for block in self.blocks for mixer in block.mixers())

    # ------------------------------------------------------------------ layout of caches

    def _calls(self):
        """(schedule index, call, [(mixer index, mixer, cache layer id)])."""
        for index, call in enumerate(self.spec.schedule):
            mixers = self.blocks[call.block].mixers()
            yield index, call, list(zip(range(len(mixers)), mixers, call.caches(len(mixers))))

    def _plan_caches(self) -> None:
        needs: dict[int, CacheNeed] = {}
        for _index, call, mixers in self._calls():
            for _m, mixer, cache_id in mixers:
                need = mixer.cache_need()
                if need is None:
                    continue
                if cache_id is None:
                    raise ValueError(f"block {call.block} keeps keys but its call names no cache layer")
                if call.writes_cache:
                    if cache_id in needs:
                        raise ValueError(f"cache layer {cache_id} is stored by two calls")
                    needs[cache_id] = need
        for _index, _call, mixers in self._calls():
            for _m, mixer, cache_id in mixers:
                if mixer.cache_need() is not None and cache_id not in needs:
                    raise ValueError(f"cache layer {cache_id} is read but no call stores it")
        self.group_windows: list[int] = []
        self.cache_layers: dict[int, CacheLayer] = {}
        for cache_id in sorted(needs):
            window = needs[cache_id].window
            if window not in self.group_windows:
                self.group_windows.append(window)
            self.cache_layers[cache_id] = CacheLayer(needs[cache_id], self.group_windows.index(window))
        # per-request state, keyed by (schedule index, mixer index within the block)
        self.state_needs: dict[tuple[int, int], StateNeed] = {}
        for index, _call, mixers in self._calls():
            for m, mixer, _cache_id in mixers:
                need = mixer.state_need()
                if need is not None:
                    self.state_needs[(index, m)] = need

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
        """Tensors a checkpoint may carry although this model has no home for them, as the
        model's description lists them (a tied model's copy of the head,
        mercury/model/loader.py:88-91)."""
        return set(self.spec.optional_tensors)

    def load(self, tensors: dict[str, torch.Tensor], setup: PartSetup) -> None:
        for part in self._parts():
            part.load(tensors, setup)

    def weight_bytes(self) -> int:
        seen: dict[int, int] = {}
        for part in self._parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor):
                    seen[value.data_ptr()] = value.numel() * value.element_size()
        return sum(seen.values())

    # ------------------------------------------------------------------ one pass

    def forward(self, ctx, kv_layers: dict[int, tuple], states: dict[tuple, torch.Tensor]):
        """Run the tokens of `ctx.batch`; returns float32 logits `[wanted rows, vocab]`, or
        None when no row is wanted. `kv_layers[c]` is (K pages, V pages) of cache layer c;
        `states[(i, m)]` the state tensor of mixer m of schedule entry i."""
        batch = ctx.batch
        h = self.embedding.forward(batch.token_ids, ctx)
        delta = None
        schedule = self.spec.schedule
        for index, call in enumerate(schedule):
            block = self.blocks[call.block]
            count = len(block.mixers())
            caches = []
            for cache_id in call.caches(count):
                if cache_id is None or cache_id not in self.cache_layers:
                    caches.append(None)
                    continue
                k, v = kv_layers[cache_id]
                group = self.cache_layers[cache_id].group
                caches.append(LayerCache(k, v, ctx.page_size, batch.tables[group], call.writes_cache))
            own = [states.get((index, m)) for m in range(count)]
            # the norm that opens the next call's block, which this block's last product
            # may compute ahead (the final norm picks rows, so it is left alone)
            following = None
            if index + 1 < len(schedule):
                nxt = self.blocks[schedule[index + 1].block]
                following = getattr(nxt, "first_norm", lambda: None)()
            if following is not None:
                delta = block.forward(h, delta, ctx, caches, own, next_norm=following)
            else:
                delta = block.forward(h, delta, ctx, caches, own)
        if batch.num_logit_rows == 0:
            return None
        rows = self.final_norm.add_norm(h, delta, ctx, rows=batch.logit_rows, defer=True)
        return self.head.forward(rows, ctx)
