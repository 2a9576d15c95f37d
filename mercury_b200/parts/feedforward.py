"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases
(mercury/model/qwen2.py:34-42, with act = SiLU). Gate and up are held as one packed matrix
`[2 * intermediate, hidden]` (gate rows first) so that one product feeds both."""

from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


class GatedFeedForward(FeedForward):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str,
                 activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation {activation!r} is not built; only 'silu'")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.prefix = prefix
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + "gate_proj.weight", (i, h)),
            TensorSpec(p + "up_proj.weight", (i, h)),
            TensorSpec(p + "down_proj.weight", (h, i)),
        ]

    def load(self, tensors, setup):
        p = self.prefix
        gate = setup.place(tensors[p + "gate_proj.weight"])
        up = setup.place(tensors[p + "up_proj.weight"])
        widest = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        self.gate_up_weight = torch.cat([gate.to(widest), up.to(widest)], dim=0).contiguous()
        self.down_weight = setup.place(tensors[p + "down_proj.weight"])

    def forward(self, x, ctx, residual=None, then_norm=None):
        tokens = x.shape[0]
        act = ctx.buffer("ff_act", tokens, self.intermediate_size)
        ctx.ops.linear_swiglu(x, self.gate_up_weight, act, ctx, ahead=self.down_weight)
        if residual is not None:
            return ctx.ops.linear_residual(act, self.down_weight, None, residual, ctx, "ff_out",
                                           then_norm=then_norm)
        out = ctx.buffer("ff_out", tokens, self.hidden_size)
        ctx.ops.linear(act, self.down_weight, None, out)
        return out


register_feed_forward("gated", GatedFeedForward)
