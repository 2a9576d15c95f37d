"""Grouped-query attention over the paged cache.

Formulas of mercury/model/qwen2.py:45-69: q, k and v projections (bias on all three when
`qkv_bias`), position encoding on q and k after the bias and before the keys are stored,
keys and values stored before attending (mercury/model/attention.py:127, :154) so that a
portion sees its own keys, softmax(q.k * scale) over the keys j <= p, query head h reading
KV head h // (heads / kv_heads), and an output projection. The three projections are held
as one packed matrix so that one product feeds them.
"""

from __future__ import annotations

import torch

from .base import CacheNeed, Mixer, PartSpec, TensorSpec, build_part, register_mixer


class GroupedQueryAttention(Mixer):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        prefix: str,
        qkv_bias: bool = True,
        out_bias: bool = False,
        window: int = 0,
        position_encoding: PartSpec | None = None,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.prefix = prefix
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = int(window)
        self.position = build_part(
            "position_encoding", position_encoding or PartSpec("none", {})
        )
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.qkv_weight = self.qkv_b = self.out_weight = self.out_b = None

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self):
        p, h = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q_proj.weight", (self.q_size, h)),
            TensorSpec(p + "k_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "v_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "o_proj.weight", (h, self.q_size)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(p + "q_proj.bias", (self.q_size,)),
                TensorSpec(p + "k_proj.bias", (self.kv_size,)),
                TensorSpec(p + "v_proj.bias", (self.kv_size,)),
            ]
        if self.out_bias:
            specs.append(TensorSpec(p + "o_proj.bias", (h,)))
        return specs + self.position.tensor_specs()      # a learned encoding owns tensors too

    def load(self, tensors, setup):
        p = self.prefix

        def packed(suffix):
            parts = [setup.place(tensors[p + name + suffix]) for name in ("q_proj", "k_proj", "v_proj")]
            widest = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            return torch.cat([t.to(widest) for t in parts], dim=0).contiguous()

        self.qkv_weight = packed(".weight")
        self.qkv_b = packed(".bias") if self.qkv_bias else None
        self.out_weight = setup.place(tensors[p + "o_proj.weight"])
        self.out_b = setup.place(tensors[p + "o_proj.bias"]) if self.out_bias else None
        self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state, residual=None, then_norm=None):
        tokens = x.shape[0]
        ops = ctx.ops
        qkv = ctx.buffer("qkv", tokens, self.q_size + 2 * self.kv_size)
        form = self.position.fused_form()
        tables = self.position.rotary_tables() if form == "rotary" else None
        attended = ctx.buffer("attended", tokens, self.q_size)
        fused = getattr(ops, "qkv_attention", None)
        if fused is not None and form is not None:
            # projection, bias, rotation, store into the pages and attention: the kernels
            # choose how to share the work between them
            fused(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads, self.num_kv_heads,
                  self.head_dim, tables, ctx.batch, cache, self.scale, self.window, attended)
            return self._project_out(attended, ctx, residual, then_norm, tokens)
        if form is not None:
            # projection, bias, rotation and the store into the pages, fused where it pays
            ops.qkv_rope_store(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads,
                               self.num_kv_heads, self.head_dim, tables, ctx.batch, cache)
        else:
            if hasattr(x, "materialize"):
                x = x.materialize()
            ops.linear(x, self.qkv_weight, self.qkv_b, qkv)
            self.position.apply(qkv, (self.num_heads, self.num_kv_heads, self.head_dim), ctx)
            ops.rope_cache_write(qkv, self.num_heads, self.num_kv_heads, self.head_dim, None,
                                 ctx.batch, cache)
        ops.paged_attention(
            qkv, self.num_heads, self.num_kv_heads, self.head_dim, ctx.batch, cache,
            self.scale, self.window, attended,
        )
        return self._project_out(attended, ctx, residual, then_norm, tokens)

    def _project_out(self, attended, ctx, residual, then_norm, tokens):
        ops = ctx.ops
        if residual is not None:
            return ops.linear_residual(attended, self.out_weight, self.out_b, residual, ctx,
                                       "mixer_out", then_norm=then_norm)
        out = ctx.buffer("mixer_out", tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, self.out_b, out)
        return out


register_mixer("grouped_query_attention", GroupedQueryAttention)
