"""A plain, slow implementation of the Qwen2 decoder: the oracle of the test-suite.

Whole sequences only, no cache, no batching, one function for each part, every step
written out. It shares no code with the `mercury_b200` package: it reads a config
dictionary (the keys of config.json) and a `{tensor name: tensor}` dictionary directly.
Each function cites the file and line of RishDevs/mercury whose formula it restates.

The arithmetic runs in `dtype` (float64 by default, so that the oracle's own rounding is
far below what the engine's 32-bit path is held to; `tests/golden/make_golden.py` runs it
in float32 beside the reference's own CPU model). It runs where its weights are: on the
CPU by default; the tests of real layer widths hand it float64 weights on the GPU, where the
same plain PyTorch functions finish a 2048-token sequence in a moment.

Where the reference has no formula (it never reads `sliding_window`), the rule used is
stated at the function.
"""

from __future__ import annotations

import torch


# ----------------------------------------------------------------------------- config

def plain_config(raw: dict) -> dict:
    """The numbers the forward pass needs, with the reference's defaults.

    mercury/config.py:45-71: `num_key_value_heads` defaults to the number of heads,
    `head_dim` to hidden // heads, `rms_norm_eps` to 1e-6, `rope_theta` to 10000.0,
    `tie_word_embeddings` to False. The window keys are this engine's addition (the
    reference ignores them): layer i is windowed iff `use_sliding_window` and
    i >= `max_window_layers`.
    """
    heads = raw["num_attention_heads"]
    hidden = raw["hidden_size"]
    layers = raw["num_hidden_layers"]
    use_window = bool(raw.get("use_sliding_window", False))
    window = int(raw.get("sliding_window") or 0)
    first_windowed = int(raw.get("max_window_layers", layers))
    return {
        "hidden": hidden,
        "intermediate": raw["intermediate_size"],
        "layers": layers,
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim") or hidden // heads,
        "vocab": raw["vocab_size"],
        "eps": raw.get("rms_norm_eps", 1e-6),
        "theta": float(raw.get("rope_theta", 10000.0)),
        "tied": bool(raw.get("tie_word_embeddings", False)),
        "windows": [
            window if (use_window and window > 0 and i >= first_windowed) else 0
            for i in range(layers)
        ],
    }


# ----------------------------------------------------------------------------- parts

def plain_embedding(table: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """Row lookup, no scaling and no position term (mercury/model/qwen2.py:100, :109)."""
    return table[token_ids]


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight (mercury/model/qwen2.py:29-31)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def plain_rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """angle[p, i] = p * theta^(-2i/d), computed in float32 as the reference's table is
    (mercury/model/rope.py:37-45), then handed on in the oracle's dtype."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    return torch.outer(positions.to(torch.float32), inv_freq)


def plain_rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(-second half, first half): the NeoX pairing (mercury/model/rope.py:6-8)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def plain_rope(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d]; x*cos + rotate_half(x)*sin with the angle table repeated over
    both halves (mercury/model/rope.py:11-17, :46-47)."""
    table = torch.cat((angles, angles), dim=-1).to(x.dtype)
    cos = table.cos().unsqueeze(1)
    sin = table.sin().unsqueeze(1)
    return x * cos + plain_rotate_half(x) * sin


def plain_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: float,
    window: int = 0,
) -> torch.Tensor:
    """q: [T, n_q, d]; k, v: [T, n_kv, d], all positions 0..T-1 of one sequence.

    Query head h reads KV head h // (n_q / n_kv) (mercury/model/attention.py:26-29);
    scores are scaled by `scale` (= d^-0.5, mercury/model/qwen2.py:54); key j is seen
    from position p iff j <= p (mercury/model/attention.py:97-99); masked scores are
    -inf before the softmax (tests/test_attention.py:25-35 of the reference).
    `window` > 0 additionally hides keys with j <= p - window, so a query sees itself and
    the window-1 keys before it; the reference has no window, this is the engine's rule.
    """
    tokens, n_q, _ = q.shape
    group = n_q // k.shape[1]
    out = torch.empty_like(q)
    pos = torch.arange(tokens, device=q.device)
    hidden = pos[None, :] > pos[:, None]
    if window > 0:
        hidden = hidden | (pos[None, :] <= pos[:, None] - window)
    for head in range(n_q):
        kv_head = head // group
        scores = (q[:, head, :] @ k[:, kv_head, :].T) * scale
        scores = scores.masked_fill(hidden, float("-inf"))
        weights = torch.softmax(scores, dim=-1)
        out[:, head, :] = weights @ v[:, kv_head, :]
    return out


def plain_attention_layer(x, w, prefix, cfg, positions, window):
    """q/k/v with bias, rotate q and k, attend, output projection without bias
    (mercury/model/qwen2.py:57-69)."""
    tokens = x.shape[0]
    n_q, n_kv, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = x @ w[prefix + "q_proj.weight"].T + w[prefix + "q_proj.bias"]
    k = x @ w[prefix + "k_proj.weight"].T + w[prefix + "k_proj.bias"]
    v = x @ w[prefix + "v_proj.weight"].T + w[prefix + "v_proj.bias"]
    q = q.view(tokens, n_q, d)
    k = k.view(tokens, n_kv, d)
    v = v.view(tokens, n_kv, d)
    angles = plain_rope_angles(positions, d, cfg["theta"])
    q = plain_rope(q, angles)
    k = plain_rope(k, angles)
    attended = plain_attention(q, k, v, d ** -0.5, window)
    return attended.reshape(tokens, n_q * d) @ w[prefix + "o_proj.weight"].T


def plain_mlp(x, w, prefix):
    """down(silu(gate(x)) * up(x)), no biases (mercury/model/qwen2.py:41-42)."""
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ w[prefix + "down_proj.weight"].T


def plain_layer(h, w, index, cfg, positions):
    """Pre-norm block: h += attention(norm(h)); h += mlp(norm(h)). The reference carries
    the sum as a deferred residual (mercury/model/qwen2.py:82-94); the value is the same."""
    prefix = f"model.layers.{index}."
    x = plain_rmsnorm(h, w[prefix + "input_layernorm.weight"], cfg["eps"])
    h = h + plain_attention_layer(
        x, w, prefix + "self_attn.", cfg, positions, cfg["windows"][index]
    )
    x = plain_rmsnorm(h, w[prefix + "post_attention_layernorm.weight"], cfg["eps"])
    h = h + plain_mlp(x, w, prefix + "mlp.")
    return h


def plain_hidden(raw_config: dict, weights: dict, token_ids, dtype=torch.float64):
    """Final-norm hidden states [T, H] of one whole sequence, computed on the device the
    weights lie on (converting them to `dtype` costs nothing if they already are)."""
    cfg = plain_config(raw_config)
    w = {name: t.to(dtype) for name, t in weights.items() if t.is_floating_point()}
    device = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    positions = torch.arange(ids.numel(), device=device)
    h = plain_embedding(w["model.embed_tokens.weight"], ids)
    for index in range(cfg["layers"]):
        h = plain_layer(h, w, index, cfg, positions)
    return plain_rmsnorm(h, w["model.norm.weight"], cfg["eps"]), w, cfg


def plain_logits(raw_config: dict, weights: dict, token_ids, dtype=torch.float64):
    """Logits [T, V] at every position of one whole sequence: hidden times the embedding
    table when tied, else times lm_head.weight (mercury/model/qwen2.py:145-150)."""
    hidden, w, cfg = plain_hidden(raw_config, weights, token_ids, dtype)
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return hidden @ head.T


def plain_logits_at(raw_config: dict, weights: dict, token_ids, rows, dtype=torch.float64):
    """Logits [len(rows), V] at the positions `rows` only: the whole sequence goes through
    the layers, the head is applied to the chosen rows (a [T, V] matrix of a real
    vocabulary would not be worth building)."""
    hidden, w, cfg = plain_hidden(raw_config, weights, token_ids, dtype)
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    index = torch.as_tensor(list(rows), dtype=torch.long, device=hidden.device)
    return hidden[index] @ head.T


# ----------------------------------------------------------------------------- sampling

def plain_uniform(seed: int, index: int) -> float:
    """The engine's documented draw: u in [0, 1) from (request seed, output index), by the
    splitmix64 finaliser over seed * 2^32 + index, top 24 bits. The reference draws with
    torch.multinomial from one shared generator (mercury/sampling.py:34), which no other
    implementation can reproduce; only the distribution is the reference's."""
    mask = (1 << 64) - 1
    z = ((seed & 0xFFFFFFFF) << 32 | (index & 0xFFFFFFFF)) & mask
    z = (z + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def plain_probabilities(logits: torch.Tensor, temperature: float, top_p: float = 1.0):
    """softmax(logits / max(T, 1e-5)) in float64 (mercury/sampling.py:28-29), then top-p:
    in descending order drop every token whose predecessors already hold more than top_p
    (the token that crosses stays), renormalise (mercury/sampling.py:6-14, :33)."""
    scaled = logits.to(torch.float64) / max(temperature, 1e-5)
    probs = torch.softmax(scaled, dim=-1)
    if top_p < 1.0:
        ordered, index = probs.sort(descending=True)
        before = ordered.cumsum(-1) - ordered
        ordered = ordered.masked_fill(before > top_p, 0.0)
        probs = torch.zeros_like(probs).scatter_(0, index, ordered)
    return probs / probs.sum()


def plain_sample(logits: torch.Tensor, temperature: float, top_p: float, u: float) -> int:
    """Greedy iff temperature <= 0 (mercury/request.py:21-23; lowest index on ties);
    otherwise the first index whose cumulative probability exceeds u."""
    if temperature <= 0.0:
        return int(torch.argmax(logits))
    cdf = plain_probabilities(logits, temperature, top_p).cumsum(-1)
    return int(min(torch.searchsorted(cdf, torch.tensor(u, dtype=cdf.dtype), right=True),
                   logits.numel() - 1))


def plain_generate(raw_config, weights, prompt, max_tokens, temperature=0.0, top_p=1.0,
                   seed=0, dtype=torch.float64):
    """Recompute the whole sequence for every new token."""
    tokens = list(prompt)
    out = []
    for index in range(max_tokens):
        logits = plain_logits(raw_config, weights, tokens, dtype)[-1]
        token = plain_sample(logits, temperature, top_p, plain_uniform(seed, index))
        tokens.append(token)
        out.append(token)
    return out

