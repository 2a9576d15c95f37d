"""A minimal stand for running one part on the GPU: a step context over one or more
sequences that start from an empty cache."""

from __future__ import annotations

import torch

from mercury_b200.cache import CacheManager
from mercury_b200.engine.batch import BatchBuffers, StepEntry
from mercury_b200.engine.runner import StepContext, Workspace
from mercury_b200.parts import PartSetup
from mercury_b200.parts.base import LayerCache


class PartStand:
    def __init__(self, dtype, page_size=16, num_pages=32, windows=(0,), max_tokens=256):
        from mercury_b200.kernels.ops import CudaOps

        self.device = torch.device("cuda")
        self.dtype = dtype
        self.ops = CudaOps(self.device)
        self.setup = PartSetup(self.device, dtype, self.ops, 512)
        self.cache = CacheManager(list(windows), num_pages, page_size, 4)
        self.buffers = BatchBuffers(self.device, max_tokens, 4, 64, len(windows), pin=True)
        self.ctx = StepContext(self.ops, Workspace(self.device, dtype, max_tokens), page_size, dtype)
        self.page_size = page_size
        self.num_pages = num_pages

    def batch_for(self, lengths):
        """One fresh sequence per length, all tokens new; returns the entries too."""
        entries = []
        for i, n in enumerate(lengths):
            seq = self.cache.open(f"s{len(self.cache.live)}-{i}")
            assert self.cache.ensure(seq, n)
            entries.append(StepEntry(seq, [0] * n, []))
        self.ctx.batch = self.buffers.build(entries, self.page_size)
        return entries

    def continue_with(self, entries, counts):
        """The next `counts[i]` tokens of each sequence of `entries`, after the tokens it has
        run so far were booked as computed."""
        following = []
        for e, n in zip(entries, counts):
            self.cache.advance(e.seq, e.seq.num_computed + len(e.tokens))
            assert self.cache.ensure(e.seq, e.seq.num_computed + n)
            following.append(StepEntry(e.seq, [0] * n, []))
        self.ctx.batch = self.buffers.build(following, self.page_size)
        return following

    def layer_cache(self, kv_heads, head_dim, group=0):
        k = torch.zeros((self.num_pages, kv_heads, self.page_size, head_dim), dtype=self.dtype,
                        device=self.device)
        return LayerCache(k, torch.zeros_like(k), self.page_size, self.ctx.batch.tables[group], True)
