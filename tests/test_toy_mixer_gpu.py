"""A mixer with per-request state of its own, defined HERE, is registered, built from a
model folder and stepped through the ordinary runner and replay, beside an attention layer
in the same model, without a change to the package."""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import pytest
import torch

import replay_cases
from mercury_b200.config import ModelConfig, register_architecture
from mercury_b200.models import LayerCall, ModelSpec
from mercury_b200.parts import Mixer, PartSpec, StateNeed, TensorSpec, register_mixer
from mercury_b200.trace_run import replay
from mercury_b200.weights import write_random_model

pytestmark = pytest.mark.gpu


class DecayingSumMixer(Mixer):
    """state <- decay * state + x_t * w_in ;  out_t = state * w_out. The state is one
    float32 vector per request, kept in the slot the cache manager gave the request."""

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
        out = ctx.buffer("toy_out", x.shape[0], self.hidden_size)
        starts, slots = batch.q_start.tolist(), batch.slots.tolist()
        for s in range(batch.num_seqs):
            for t in range(starts[s], starts[s + 1]):
                state[slots[s]] = self.decay * state[slots[s]] + x[t].float() * self.w_in
                out[t] = (state[slots[s]] * self.w_out).to(out.dtype)
        return out


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden_size: int = 48
    vocab_size: int = 97
    decay: float = 0.9

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["architectures"][0], raw["hidden_size"], raw["vocab_size"], raw["decay"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size,
                "vocab_size": self.vocab_size, "decay": self.decay}


def describe_toy(cfg: ToyConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name: PartSpec("rmsnorm", {"size": h, "eps": 1e-6, "weight_name": name})
    ff = lambda p: PartSpec("gated", {"hidden_size": h, "intermediate_size": 64, "prefix": p})
    attention = PartSpec("grouped_query_attention", {
        "hidden_size": h, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "scale": 0.25,
        "prefix": "layers.0.attn.",
        "position_encoding": PartSpec("rotary", {"head_dim": 16, "theta": 10000.0})})
    toy = PartSpec("decaying_sum", {"hidden_size": h, "decay": cfg.decay, "prefix": "layers.1.toy."})
    blocks = [PartSpec("pre_norm", {"mixer": m, "feed_forward": ff(f"layers.{i}.mlp."),
                                    "mixer_norm": norm(f"layers.{i}.n1"),
                                    "feed_forward_norm": norm(f"layers.{i}.n2")})
              for i, m in enumerate((attention, toy))]
    return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size, max_positions=512,
                     embedding=PartSpec("lookup", {"vocab_size": cfg.vocab_size, "hidden_size": h,
                                                   "weight_name": "embed"}),
                     blocks=blocks,
                     schedule=[LayerCall(0, cache=0), LayerCall(1), LayerCall(0, cache=1)],
                     final_norm=norm("final_norm"),
                     head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": h,
                                              "weight_name": "head"}))


def plain_toy(tensors, cfg, tokens):
    """The toy model whole, in float64, written out here."""
    import plain_qwen2 as P

    w = {k: v.double() for k, v in tensors.items()}
    h = w["embed"][torch.tensor(tokens)]
    positions = torch.arange(len(tokens))
    acfg = {"heads": 3, "kv_heads": 1, "head_dim": 16, "theta": 10000.0}

    def mlp(x, p):
        g = x @ w[p + "gate_proj.weight"].T
        return (g * torch.sigmoid(g) * (x @ w[p + "up_proj.weight"].T)) @ w[p + "down_proj.weight"].T

    def attention_block(h):
        x = P.plain_rmsnorm(h, w["layers.0.n1"], 1e-6)
        h = h + P.plain_attention_layer(x, w, "layers.0.attn.", {**acfg}, positions, 0)
        return h + mlp(P.plain_rmsnorm(h, w["layers.0.n2"], 1e-6), "layers.0.mlp.")

    h = attention_block(h)
    x = P.plain_rmsnorm(h, w["layers.1.n1"], 1e-6)
    state = torch.zeros(cfg.hidden_size, dtype=torch.float64)
    mixed = torch.empty_like(x)
    for t in range(len(tokens)):
        state = cfg.decay * state + x[t] * w["layers.1.toy.w_in"]
        mixed[t] = state * w["layers.1.toy.w_out"]
    h = h + mixed
    h = h + mlp(P.plain_rmsnorm(h, w["layers.1.n2"], 1e-6), "layers.1.mlp.")
    h = attention_block(h)                      # block 0 again, with a cache layer of its own
    return P.plain_rmsnorm(h, w["final_norm"], 1e-6) @ w["head"].T


def test_toy_mixer_is_registered_built_and_stepped(tmp_path):
    from mercury_b200.engine.runner import ModelRunner
    from safetensors.torch import load_file

    register_mixer("decaying_sum", DecayingSumMixer)
    register_architecture("ToyStateForCausalLM", ToyConfig, describe_toy)
    cfg = ToyConfig("ToyStateForCausalLM")
    folder = write_random_model(tmp_path / "toy", cfg, seed=5)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyStateForCausalLM"]
    tensors = load_file(str(folder / "model.safetensors"))
    gen = torch.Generator().manual_seed(1)
    requests = {f"t{i}": torch.randint(0, 97, (n,), generator=gen).tolist()
                for i, n in enumerate((40, 23, 64, 31, 50))}
    want = {rid: plain_toy(tensors, cfg, toks).numpy() for rid, toks in requests.items()}
    for mode in ("whole", "portions", "mixed"):
        runner = ModelRunner(folder, dtype=torch.float32, device="cuda", page_size=16,
                             num_pages=16, max_seqs=4, max_step_tokens=256, max_model_len=256)
        assert runner.has_state and len(runner.states) == 1 and len(runner.kv_layers) == 2
        builder = getattr(replay_cases, mode)
        steps, rows = builder(requests, 256, seed=4) if mode == "mixed" else builder(requests)
        out = tmp_path / mode
        replay(runner, [json.dumps(s) for s in steps], out, lambda _line: None)
        import numpy as np

        for step, expected in rows.items():
            got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(expected), 97)
            for row, (rid, pos) in enumerate(expected):
                err = np.abs(got[row] - want[rid][pos]).max() / np.abs(want[rid]).max()
                assert err < 3e-5, (mode, step, rid, pos, err)
        runner.cache.check_invariants()
        assert runner.cache.leaked_pages() == 0
