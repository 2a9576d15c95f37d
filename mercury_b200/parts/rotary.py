"""Rotary position encoding with the NeoX pairing of halves.

Table as in mercury/model/rope.py:37-47: inv_freq[i] = theta^(-2i/d), angle = position *
inv_freq, both in float32; the table is kept in float32 (the reference rounds it to the
activation dtype) and covers as many positions as the engine will serve
(mercury/model/loader.py:101). `rotary_dim` is the number of leading features of a head
that are rotated; Qwen2 rotates the whole head.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    capturable = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most {head_dim}")
        self.cos = None
        self.sin = None

    def load(self, tensors, setup):
        def tables():
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            inv_freq = 1.0 / (self.theta ** exponent)
            positions = torch.arange(setup.max_positions, dtype=torch.float32)
            angles = torch.outer(positions, inv_freq)
            return (angles.cos().to(setup.device).contiguous(),
                    angles.sin().to(setup.device).contiguous())

        # every layer with the same constants reads the same pair of tables
        self.cos, self.sin = setup.derived(
            ("rotary", self.rotary_dim, self.theta, setup.max_positions, str(setup.device)), tables)

    def fused_form(self):
        return "rotary"

    def rotary_tables(self):
        return self.cos, self.sin


class NoPositionEncoding(PositionEncoding):
    capturable = True

    def __init__(self, **_ignored):
        pass

    def fused_form(self):
        return "identity"


register_position_encoding("rotary", RotaryEncoding)
register_position_encoding("none", NoPositionEncoding)
