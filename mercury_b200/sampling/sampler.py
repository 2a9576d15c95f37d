"""From logits to token ids.

Greedy rows take the argmax (lowest index among equal maxima); the others sample from
softmax(logits / max(T, 1e-5)) cut by top-p (mercury/sampling.py:17-35) by inverse CDF in
index order. The uniform number of a draw depends only on the request's seed and on how
many tokens it has produced, never on what else is in the batch, so a request's tokens
are the same however it is batched; the reference draws from one generator shared by the
whole batch (mercury/runner.py:66-68, mercury/sampling.py:34).
"""

from __future__ import annotations

import zlib

import torch

from .params import SamplingParams

_MASK = (1 << 64) - 1


def draw_uniform(seed: int, index: int) -> float:
    """u in [0, 1): the splitmix64 finaliser of seed * 2^32 + index, top 24 bits."""
    z = (((seed & 0xFFFFFFFF) << 32) | (index & 0xFFFFFFFF)) & _MASK
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def request_seed(params: SamplingParams, engine_seed: int, rid: str) -> int:
    """The request's own seed if it gave one, else one derived from the engine's seed and
    the request id."""
    if params.seed is not None:
        return int(params.seed) & 0xFFFFFFFF
    return (zlib.crc32(rid.encode()) ^ (engine_seed * 0x9E3779B1)) & 0xFFFFFFFF


class Sampler:
    """`begin` launches the kernels of one batch and the copy of its tokens to the host;
    `finish` waits for that copy. Two sets of buffers alternate, so that the tokens of one
    batch stay on the device (where the next step may take its inputs from them) and on
    their way to the host while the next batch is being sampled."""

    def __init__(self, ops, device, max_rows: int):
        self.ops = ops
        self.device = torch.device(device)
        pin = self.device.type == "cuda"
        self.host = torch.zeros((2, 3, max_rows), dtype=torch.float32, pin_memory=pin)
        self.dev = torch.zeros((2, 3, max_rows), dtype=torch.float32, device=self.device)
        self.tokens = torch.zeros((2, max_rows), dtype=torch.int32, device=self.device)
        self.tokens_host = torch.zeros((2, max_rows), dtype=torch.int32, pin_memory=pin)
        self._copied = [torch.cuda.Event(), torch.cuda.Event()] if pin else None
        self._turn = 0

    def begin(self, logits: torch.Tensor, rows: list[tuple[SamplingParams, int, int]]
              ) -> tuple[int, int]:
        """`rows[i]` = (params, seed, output index) of the request that logits row i belongs
        to. Returns a handle for `finish` and `on_device`."""
        count = len(rows)
        turn = self._turn
        self._turn ^= 1
        if count == 0:
            return turn, 0
        out = self.tokens[turn, :count]
        if all(p.greedy for p, _s, _i in rows):
            self.ops.argmax(logits, out)
        else:
            host = self.host[turn, :, :count]
            for i, (p, seed, index) in enumerate(rows):
                host[0, i] = p.temperature
                host[1, i] = p.top_p
                host[2, i] = 0.0 if p.greedy else draw_uniform(seed, index)
            dev = self.dev[turn, :, :count]
            dev.copy_(host, non_blocking=True)
            self.ops.sample(logits, dev[0], dev[1], dev[2], out)
        self.tokens_host[turn, :count].copy_(out, non_blocking=True)
        if self._copied is not None:
            self._copied[turn].record()
        return turn, count

    def on_device(self, handle: tuple[int, int]) -> torch.Tensor:
        """The sampled tokens of a batch as they lie on the device (int32)."""
        turn, count = handle
        return self.tokens[turn, :count]

    def finish(self, handle: tuple[int, int]) -> list[int]:
        """One token id per row, on the host."""
        turn, count = handle
        if count == 0:
            return []
        if self._copied is not None:
            self._copied[turn].synchronize()
        return self.tokens_host[turn, :count].tolist()

    def sample(self, logits: torch.Tensor, rows: list[tuple[SamplingParams, int, int]]) -> list[int]:
        return self.finish(self.begin(logits, rows))
