"""Each part alone on the GPU against the plain function of the same part."""

from __future__ import annotations

import pytest
import torch

import plain_qwen2 as P
from mercury_b200.parts import PartSpec, build_part
from part_harness import PartStand

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).bfloat16()


def check(got, want, dtype, what):
    err = float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max())
    assert err <= TOL[dtype], f"{what}: relative error {err:.2e}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_rmsnorm_part(dtype):
    stand = PartStand(dtype)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 100, "eps": 1e-5, "weight_name": "w"}))
    weight = rand((100,), 0, 0.05) + 1
    norm.load({"w": weight}, stand.setup)
    h = torch.randn((13, 100), generator=torch.Generator().manual_seed(1))
    delta = rand((13, 100), 2)
    h_dev = h.cuda()
    out = norm.add_norm(h_dev, delta.cuda().to(dtype), stand.ctx)
    summed = h.double() + delta.double()
    check(out, P.plain_rmsnorm(summed, weight.double(), 1e-5), dtype, "norm")
    check(h_dev, summed, torch.float32, "residual")
    rows = torch.tensor([12, 3], dtype=torch.int32).cuda()
    picked = norm.add_norm(h_dev, None, stand.ctx, rows=rows)
    check(picked, P.plain_rmsnorm(summed[[12, 3]], weight.double(), 1e-5), dtype, "selected rows")


def test_rotary_tables_follow_the_plain_angles():
    stand = PartStand(torch.float32)
    rope = build_part("position_encoding", PartSpec("rotary", {"head_dim": 48, "theta": 50000.0}))
    rope.load({}, stand.setup)
    cos, sin = rope.rotary_tables()
    angles = P.plain_rope_angles(torch.arange(512), 48, 50000.0)
    assert cos.shape == (512, 24)
    assert torch.allclose(cos.cpu(), angles.cos(), atol=1e-6)
    assert torch.allclose(sin.cpu(), angles.sin(), atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embedding_and_head(dtype):
    stand = PartStand(dtype)
    table = rand((331, 80), 3)
    emb = build_part("embedding", PartSpec("lookup", {"vocab_size": 331, "hidden_size": 80,
                                                      "weight_name": "e"}))
    emb.load({"e": table}, stand.setup)
    entries = stand.batch_for([9])
    ids = torch.randint(0, 331, (9,), dtype=torch.int32).cuda()
    h = emb.forward(ids, stand.ctx)
    assert h.dtype == torch.float32
    assert torch.equal(h.cpu(), P.plain_embedding(table.float(), ids.cpu().long()))
    # a head that names the embedding's tensor is tied to it: one buffer for both
    head = build_part("head", PartSpec("linear", {"vocab_size": 331, "hidden_size": 80,
                                                  "weight_name": "e"}))
    head.load({"e": table}, stand.setup)
    assert head.weight.data_ptr() == emb.table.data_ptr()
    rows = rand((4, 80), 4).cuda().to(dtype)
    logits = head.forward(rows, stand.ctx)
    assert logits.dtype == torch.float32
    check(logits, rows.double().cpu() @ table.double().T, dtype, "tied head")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, 0), (6, 2, 48, 20), (7, 1, 64, 0)])
def test_attention_part(dtype, heads, kv_heads, head_dim, window):
    hidden = 72
    stand = PartStand(dtype, windows=(window,))
    mixer = build_part("mixer", PartSpec("grouped_query_attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
        "scale": head_dim ** -0.5, "prefix": "a.", "window": window,
        "position_encoding": PartSpec("rotary", {"head_dim": head_dim, "theta": 10000.0})}))
    weights = {s.name: rand(s.shape, 10 + i, 0.15) for i, s in enumerate(mixer.tensor_specs())}
    mixer.load(weights, stand.setup)
    lengths = [50, 7]
    stand.batch_for(lengths)
    x = rand((sum(lengths), hidden), 5)
    cache = stand.layer_cache(kv_heads, head_dim)
    out = mixer.forward(x.cuda().to(dtype), stand.ctx, cache, None)
    cfg = {"heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "theta": 10000.0}
    w = {k: v.double() for k, v in weights.items()}
    at = 0
    for n in lengths:
        want = P.plain_attention_layer(x[at:at + n].double(), w, "a.", cfg, torch.arange(n), window)
        check(out[at:at + n], want, dtype, f"attention over {n} tokens")
        at += n


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_feed_forward_part(dtype):
    stand = PartStand(dtype)
    ff = build_part("feed_forward", PartSpec("gated", {"hidden_size": 72, "intermediate_size": 200,
                                                      "prefix": "m."}))
    weights = {s.name: rand(s.shape, 20 + i, 0.1) for i, s in enumerate(ff.tensor_specs())}
    ff.load(weights, stand.setup)
    x = rand((11, 72), 6)
    out = ff.forward(x.cuda().to(dtype), stand.ctx)
    check(out, P.plain_mlp(x.double(), {k: v.double() for k, v in weights.items()}, "m."), dtype, "mlp")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_pre_norm_block(dtype):
    hidden, heads, kv_heads, head_dim = 64, 4, 2, 16
    stand = PartStand(dtype)
    prefix = "model.layers.0."
    norm = lambda n: PartSpec("rmsnorm", {"size": hidden, "eps": 1e-6, "weight_name": prefix + n + ".weight"})
    block = build_part("arrangement", PartSpec("pre_norm", {
        "mixer": PartSpec("grouped_query_attention", {
            "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads,
            "head_dim": head_dim, "scale": head_dim ** -0.5, "prefix": prefix + "self_attn.",
            "position_encoding": PartSpec("rotary", {"head_dim": head_dim, "theta": 10000.0})}),
        "feed_forward": PartSpec("gated", {"hidden_size": hidden, "intermediate_size": 128,
                                           "prefix": prefix + "mlp."}),
        "mixer_norm": norm("input_layernorm"), "feed_forward_norm": norm("post_attention_layernorm")}))
    weights = {}
    for part in block.parts():
        for i, s in enumerate(part.tensor_specs()):
            weights[s.name] = rand(s.shape, 30 + len(weights), 0.1) + (1 if s.init == "ones_normal" else 0)
        part.load(weights, stand.setup)
    stand.batch_for([33])
    h = torch.randn((33, hidden), generator=torch.Generator().manual_seed(7))
    h_dev = h.cuda()
    delta = block.forward(h_dev, None, stand.ctx, [stand.layer_cache(kv_heads, head_dim)], [None])
    cfg = {"heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "theta": 10000.0,
           "eps": 1e-6, "windows": [0]}
    want = P.plain_layer(h.double(), {k: v.double() for k, v in weights.items()}, 0, cfg, torch.arange(33))
    check(h_dev.double() + delta.double(), want, dtype, "block output")
