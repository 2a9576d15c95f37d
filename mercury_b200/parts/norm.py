"""RMSNorm fused with the residual sum.

The formula is mercury/model/qwen2.py:27-31: the pending delta is added to the residual
stream, the sum is the new residual, and the sum is normalised by rsqrt(mean(x^2) + eps)
and scaled by the weight. The reference adds in the activation dtype on its plain path and
in float32 on its fused path (mercury/kernels/rmsnorm_quant.py:40-46); here the stream
itself is float32, so nothing is rounded between layers.
"""

from __future__ import annotations

from .base import Norm, TensorSpec, register_norm


class PendingNorm:
    """A norm that has not run yet: the float32 stream, the weight and eps (and optionally
    which rows). A consumer whose kernel can normalise its input on the fly takes this
    instead of a tensor and saves the norm's own launch; any other consumer calls
    `materialize()` and gets the normalised rows."""

    def __init__(self, h, weight, eps, rows, ctx, size):
        self.h, self.weight, self.eps, self.rows, self.ctx, self.size = h, weight, eps, rows, ctx, size
        self.shape = ((h.shape[0] if rows is None else rows.shape[0]), size)
        self.dtype = ctx.dtype

    def materialize(self):
        count = self.shape[0]
        out = self.ctx.buffer("normed" if self.rows is None else "normed_rows", count, self.size)
        self.ctx.ops.add_rmsnorm(self.h, None, self.weight, self.eps, out, self.rows)
        return out


class PendingScaled(PendingNorm):
    """A norm whose output exists up to the division by the row's rms: `x` holds the stream
    times the norm weight (bfloat16) and `ss_part` [rows, tiles] the stream's sums of
    squares per 16-column tile, both left by the product that updated the stream. A product
    that takes this multiplies its result rows by 1/rms (a row scale commutes with the
    product); any other consumer calls `materialize()`, which runs the norm from the
    stream."""

    def __init__(self, x, ss_part, h, weight, eps, ctx, size):
        super().__init__(h, weight, eps, None, ctx, size)
        self.x, self.ss_part = x, ss_part


class RMSNorm(Norm):
    capturable = True

    def __init__(self, size: int, eps: float, weight_name: str, init_std: float = 0.05):
        self.size = size
        self.eps = eps
        self.weight_name = weight_name
        self.init_std = init_std
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size,), init="ones_normal", std=self.init_std)]

    def load(self, tensors, setup):
        self.weight = setup.place(tensors[self.weight_name])

    def add_norm(self, h, delta, ctx, rows=None, defer=False):
        """`defer=True` says that the consumer takes a `PendingNorm`; one is returned when
        nothing has to be added first and the kernels can fuse the norm for this many rows."""
        pre = getattr(ctx, "prenormed", None)
        if pre is not None:
            ctx.prenormed = None
            if pre[0] is self and delta is None and rows is None:
                # the product before this norm already left its output (up to the row scale)
                return pre[1] if defer else pre[1].materialize()
        count = h.shape[0] if rows is None else rows.shape[0]
        if (defer and delta is None
                and getattr(ctx.ops, "can_fuse_norm", lambda *a: False)(count, self.size, self.weight)):
            return PendingNorm(h, self.weight, self.eps, rows, ctx, self.size)
        out = ctx.buffer("normed" if rows is None else "normed_rows", count, self.size)
        ctx.ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out


register_norm("rmsnorm", RMSNorm)
