"""Parts that are not Qwen2's, defined HERE and plugged into the engine without a change to
the package: a position encoding that goes through `apply()` (and owns a checkpoint
tensor), a feed-forward that routes each token to one of several experts, an arrangement
with two mixers side by side (attention and a mixer with state of its own, each with its own
cache layer or state slot), and rotary encoding over a part of the head. None of them is a
model of anyone's; they show what the interfaces carry."""

from __future__ import annotations

import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen2 as P
import replay_cases
from mercury_b200.config import ModelConfig, register_architecture
from mercury_b200.models import LayerCall, ModelSpec
from mercury_b200.parts import (FeedForward, Mixer, PartSpec, PositionEncoding, StateNeed, TensorSpec,
                                build_part, register_arrangement, register_feed_forward,
                                register_mixer, register_position_encoding)
from mercury_b200.parts.base import LayerCache
from mercury_b200.trace_run import replay
from mercury_b200.weights import write_random_model
from part_harness import PartStand

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).bfloat16()


# ------------------------------------------------------------------ rotary over part of a head

def plain_partial_rope(x, positions, rotary_dim, theta):
    """x: [T, heads, d]: the first `rotary_dim` features of each head are rotated as a head
    of that size would be (pairs i, i + rotary_dim/2), the rest pass through."""
    angles = P.plain_rope_angles(positions, rotary_dim, theta)
    turned = P.plain_rope(x[..., :rotary_dim], angles)
    return torch.cat((turned, x[..., rotary_dim:]), dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("head_dim,rotary_dim", [(64, 32), (48, 16), (128, 64)])
def test_attention_with_rotary_over_part_of_the_head(dtype, head_dim, rotary_dim):
    """Prompt portions, then one more token per sequence (the few-token kernels), with
    `rotary_dim < head_dim`: the fused kernels refuse such a head and the chain falls back
    to the kernels that take it."""
    hidden, heads, kv_heads, theta = 72, 4, 2, 10000.0
    stand = PartStand(dtype)
    mixer = build_part("mixer", PartSpec("grouped_query_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
        "scale": head_dim ** -0.5, "prefix": "a.",
        "position_encoding": PartSpec("rotary", {"head_dim": head_dim, "theta": theta,
                                                 "rotary_dim": rotary_dim})}))
    weights = {s.name: rand(s.shape, 10 + i, 0.15) for i, s in enumerate(mixer.tensor_specs())}
    mixer.load(weights, stand.setup)
    assert mixer.position.rotary_tables()[0].shape[1] == rotary_dim // 2
    lengths = [50, 7]
    entries = stand.batch_for(lengths)
    x = rand((sum(lengths) + len(lengths), hidden), 5)
    cache = stand.layer_cache(kv_heads, head_dim)
    got = [mixer.forward(x[:sum(lengths)].cuda().to(dtype), stand.ctx, cache, None).clone()]
    stand.continue_with(entries, [1, 1])
    cache = LayerCache(cache.k, cache.v, cache.page_size, stand.ctx.batch.tables[0], True)
    got.append(mixer.forward(x[sum(lengths):].cuda().to(dtype), stand.ctx, cache, None).clone())
    w = {k: v.double() for k, v in weights.items()}
    at = 0
    for s, n in enumerate(lengths):
        rows = torch.cat((x[at:at + n], x[sum(lengths) + s:sum(lengths) + s + 1])).double()
        positions = torch.arange(n + 1)
        q = (rows @ w["a.q_proj.weight"].T + w["a.q_proj.bias"]).view(n + 1, heads, head_dim)
        k = (rows @ w["a.k_proj.weight"].T + w["a.k_proj.bias"]).view(n + 1, kv_heads, head_dim)
        v = (rows @ w["a.v_proj.weight"].T + w["a.v_proj.bias"]).view(n + 1, kv_heads, head_dim)
        q = plain_partial_rope(q, positions, rotary_dim, theta)
        k = plain_partial_rope(k, positions, rotary_dim, theta)
        want = P.plain_attention(q, k, v, head_dim ** -0.5).reshape(n + 1, -1) @ w["a.o_proj.weight"].T
        both = torch.cat((got[0][at:at + n], got[1][s:s + 1])).double().cpu()
        err = float((both - want).abs().max() / want.abs().max())
        assert err <= TOL[dtype], f"sequence {s}: relative error {err:.2e}"
        at += n


# ------------------------------------------------------------------ the toy parts

class AddedPositions(PositionEncoding):
    """q and k of every head get a learned vector of their position added (a checkpoint
    tensor [positions, head_dim]). No kernel of the package knows this encoding, so the
    attention part calls `apply()`, which works on the packed rows in place."""

    def __init__(self, head_dim: int, positions: int, weight_name: str):
        self.head_dim, self.positions, self.weight_name = head_dim, positions, weight_name

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.positions, self.head_dim), std=0.3)]

    def load(self, tensors, setup):
        self.table = setup.place(tensors[self.weight_name])

    def apply(self, qkv, layout, ctx):
        heads, kv_heads, d = layout
        tokens = qkv.shape[0]
        added = self.table[ctx.batch.positions[:tokens].long()].float()[:, None, :]
        both = qkv[:, :(heads + kv_heads) * d].view(tokens, heads + kv_heads, d)
        both.copy_((both.float() + added).to(qkv.dtype))


class RoutedFeedForward(FeedForward):
    """Each token goes to the expert whose router logit is largest (float32), and gets that
    expert's matrix times the token, weighted by the softmax probability of the choice."""

    def __init__(self, hidden_size: int, experts: int, prefix: str):
        self.hidden_size, self.experts, self.prefix = hidden_size, experts, prefix

    def tensor_specs(self):
        h, p = self.hidden_size, self.prefix
        return [TensorSpec(p + "router", (self.experts, h), std=0.5)] + [
            TensorSpec(p + f"expert{e}", (h, h), std=0.1) for e in range(self.experts)]

    def load(self, tensors, setup):
        self.router = setup.place(tensors[self.prefix + "router"])
        self.matrices = [setup.place(tensors[self.prefix + f"expert{e}"]) for e in range(self.experts)]

    def forward(self, x, ctx):
        logits = x.float() @ self.router.float().T
        probs = torch.softmax(logits, dim=-1)
        choice = logits.argmax(dim=-1)
        out = ctx.buffer("routed_out", x.shape[0], self.hidden_size)
        for e, matrix in enumerate(self.matrices):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                picked = ctx.buffer("routed_rows", rows.numel(), self.hidden_size)
                ctx.ops.linear(x[rows].contiguous(), matrix, None, picked)
                out[rows] = (picked.float() * probs[rows, e, None]).to(out.dtype)
        return out


class DecayingSum(Mixer):
    """state <- decay * state + x_t * w_in ;  out_t = state * w_out, one float32 vector per
    request in the slot the cache manager gave it."""

    def __init__(self, hidden_size: int, decay: float, prefix: str):
        self.hidden_size, self.decay, self.prefix = hidden_size, decay, prefix

    def state_need(self):
        return StateNeed((self.hidden_size,), torch.float32)

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "w_in", (self.hidden_size,), init="ones_normal", std=0.1),
                TensorSpec(self.prefix + "w_out", (self.hidden_size,), init="ones_normal", std=0.1)]

    def load(self, tensors, setup):
        self.w_in = setup.place(tensors[self.prefix + "w_in"]).float()
        self.w_out = setup.place(tensors[self.prefix + "w_out"]).float()

    def forward(self, x, ctx, cache, state):
        batch = ctx.batch
        out = ctx.buffer("decay_out", x.shape[0], self.hidden_size)
        starts, slots = batch.q_start.tolist(), batch.slots.tolist()
        for s in range(batch.num_seqs):
            for t in range(starts[s], starts[s + 1]):
                state[slots[s]] = self.decay * state[slots[s]] + x[t].float() * self.w_in
                out[t] = (state[slots[s]] * self.w_out).to(out.dtype)
        return out


class SideBySideBlock:
    """One norm, then every mixer and the feed-forward on the same normalised input; their
    sum is the block's delta. Two mixers: `caches[i]` and `states[i]` are mixer i's."""

    def __init__(self, mixers: list, feed_forward: PartSpec, norm: PartSpec):
        self._mixers = [build_part("mixer", m) for m in mixers]
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.norm = build_part("norm", norm)

    def mixers(self):
        return self._mixers

    def parts(self):
        return [self.norm, *self._mixers, self.feed_forward]

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        x = self.norm.add_norm(h, delta, ctx)
        total = torch.zeros((x.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
        for mixer, cache, state in zip(self._mixers, caches, states):
            total += mixer.forward(x, ctx, cache, state).float()
        total += self.feed_forward.forward(x, ctx).float()
        out = ctx.buffer("side_by_side", x.shape[0], x.shape[1])
        out.copy_(total.to(out.dtype))
        return out


@dataclass(frozen=True)
class ZooConfig(ModelConfig):
    hidden_size: int = 48
    vocab_size: int = 101

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["architectures"][0], raw["hidden_size"], raw["vocab_size"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                "vocab_size": self.vocab_size}


HEADS, KV_HEADS, HEAD_DIM, EXPERTS, DECAY, POSITIONS = 3, 1, 16, 3, 0.8, 256


def describe_zoo(cfg: ZooConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("rmsnorm", {"size": h, "eps": 1e-6, "weight_name": name})

    def attention(prefix, position):
        return PartSpec("grouped_query_attention", {
            "hidden_size": h, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
            "scale": HEAD_DIM ** -0.5, "prefix": prefix, "position_encoding": position})

    side = PartSpec("side_by_side", {
        "mixers": [attention("l0.attn.", PartSpec("rotary", {"head_dim": HEAD_DIM, "theta": 10000.0})),
                   PartSpec("decaying_sum_2", {"hidden_size": h, "decay": DECAY, "prefix": "l0.decay."})],
        "feed_forward": PartSpec("routed", {"hidden_size": h, "experts": EXPERTS, "prefix": "l0.ff."}),
        "norm": norm("l0.norm")})
    plain = PartSpec("pre_norm", {
        "mixer": attention("l1.attn.", PartSpec("added_positions", {
            "head_dim": HEAD_DIM, "positions": POSITIONS, "weight_name": "l1.attn.positions"})),
        "feed_forward": PartSpec("gated", {"hidden_size": h, "intermediate_size": 64, "prefix": "l1.mlp."}),
        "mixer_norm": norm("l1.n1"), "feed_forward_norm": norm("l1.n2")})
    part = lambda kind, name: PartSpec(kind, {"vocab_size": cfg.vocab_size, "hidden_size": h,
                                              "weight_name": name})
    return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, max_positions=POSITIONS,
                     embedding=part("lookup", "embed"), blocks=[side, plain],
                     # the side-by-side block names a cache layer for its attention and none
                     # for the mixer that keeps state instead
                     schedule=[LayerCall(0, cache=(0, None)), LayerCall(1, cache=1)],
                     final_norm=norm("final_norm"), head=part("linear", "head"))


def plain_zoo(tensors, cfg, tokens):
    """The toy model whole, in float64."""
    w = {k: v.double() for k, v in tensors.items()}
    count = len(tokens)
    positions = torch.arange(count)
    h = w["embed"][torch.tensor(tokens)]

    def heads_of(x, prefix):
        q = (x @ w[prefix + "q_proj.weight"].T + w[prefix + "q_proj.bias"]).view(count, HEADS, HEAD_DIM)
        k = (x @ w[prefix + "k_proj.weight"].T + w[prefix + "k_proj.bias"]).view(count, KV_HEADS, HEAD_DIM)
        v = (x @ w[prefix + "v_proj.weight"].T + w[prefix + "v_proj.bias"]).view(count, KV_HEADS, HEAD_DIM)
        return q, k, v

    def attend(q, k, v, prefix):
        return P.plain_attention(q, k, v, HEAD_DIM ** -0.5).reshape(count, -1) @ w[prefix + "o_proj.weight"].T

    # block 0: attention, decaying sum and routed experts side by side
    x = P.plain_rmsnorm(h, w["l0.norm"], 1e-6)
    q, k, v = heads_of(x, "l0.attn.")
    angles = P.plain_rope_angles(positions, HEAD_DIM, 10000.0)
    attended = attend(P.plain_rope(q, angles), P.plain_rope(k, angles), v, "l0.attn.")
    state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    decayed = torch.empty_like(x)
    for t in range(count):
        state = DECAY * state + x[t] * w["l0.decay.w_in"]
        decayed[t] = state * w["l0.decay.w_out"]
    logits = x @ w["l0.ff.router"].T
    probs = torch.softmax(logits, dim=-1)
    choice = logits.argmax(dim=-1)
    routed = torch.stack([(w[f"l0.ff.expert{int(e)}"] @ x[t]) * probs[t, e] for t, e in enumerate(choice)])
    h = h + attended + decayed + routed
    # block 1: pre-norm attention with added positions, gated feed-forward
    x = P.plain_rmsnorm(h, w["l1.n1"], 1e-6)
    q, k, v = heads_of(x, "l1.attn.")
    added = w["l1.attn.positions"][positions][:, None, :]
    h = h + attend(q + added, k + added, v, "l1.attn.")
    h = h + P.plain_mlp(P.plain_rmsnorm(h, w["l1.n2"], 1e-6), w, "l1.mlp.")
    return P.plain_rmsnorm(h, w["final_norm"], 1e-6) @ w["head"].T


def test_toy_parts_run_through_replay(tmp_path):
    from mercury_b200.engine.runner import ModelRunner
    from safetensors.torch import load_file

    register_position_encoding("added_positions", AddedPositions)
    register_feed_forward("routed", RoutedFeedForward)
    register_mixer("decaying_sum_2", DecayingSum)
    register_arrangement("side_by_side", SideBySideBlock)
    register_architecture("ToyZooForCausalLM", ZooConfig, describe_zoo)
    cfg = ZooConfig("ToyZooForCausalLM")
    folder = write_random_model(tmp_path / "zoo", cfg, seed=8)
    tensors = load_file(str(folder / "model.safetensors"))
    assert "l1.attn.positions" in tensors and "l0.ff.expert2" in tensors
    gen = torch.Generator().manual_seed(2)
    requests = {f"z{i}": torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
                for i, n in enumerate((40, 23, 64, 31, 50))}
    want = {rid: plain_zoo(tensors, cfg, toks).numpy() for rid, toks in requests.items()}
    for mode in ("whole", "decode_tail", "portions", "mixed"):
        runner = ModelRunner(folder, dtype=torch.float32, device="cuda", page_size=16, num_pages=16,
                             max_seqs=4, max_step_tokens=256, max_model_len=256, poison_pages=True)
        assert not runner.use_graphs, "parts that do not declare themselves capturable run eagerly"
        assert len(runner.kv_layers) == 2 and list(runner.states) == [(0, 1)]
        assert not runner.model.skips_cached_prefix
        builder = getattr(replay_cases, mode)
        steps, rows = builder(requests, 256, seed=4) if mode == "mixed" else builder(requests)
        out = tmp_path / mode
        replay(runner, [json.dumps(s) for s in steps], out, lambda _line: None)
        for step, expected in rows.items():
            got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(expected), cfg.vocab_size)
            for row, (rid, pos) in enumerate(expected):
                err = np.abs(got[row] - want[rid][pos]).max() / np.abs(want[rid]).max()
                assert err < 3e-5, (mode, step, rid, pos, err)
        runner.cache.check_invariants()
        assert runner.cache.leaked_pages() == 0
