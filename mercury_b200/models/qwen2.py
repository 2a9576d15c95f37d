"""The Qwen2 dense decoder described in parts (mercury/model/qwen2.py:34-150).

Every layer is a pre-norm block of grouped-query attention (bias on q, k and v, none on
the output projection, rotary positions over the whole head, scale head_dim^-0.5) and a
SiLU-gated feed-forward; one RMSNorm closes the stack; the head is tied to the embedding
when `tie_word_embeddings` says so. Tensor names are the checkpoint's own, so no renaming
table exists (mercury/model/loader.py:66-76). Layers from `max_window_layers` on are
windowed when `use_sliding_window` is set, which the reference never reads.
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config, register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec


def describe_qwen2(config: Qwen2Config) -> ModelSpec:
    blocks = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        rotary = PartSpec("rotary", {"head_dim": config.head_dim, "theta": config.rope_theta})
        mixer = PartSpec("grouped_query_attention", {
            "hidden_size": config.hidden_size,
            "num_heads": config.num_attention_heads,
            "num_kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "scale": config.head_dim ** -0.5,
            "prefix": prefix + "self_attn.",
            "qkv_bias": True,
            "out_bias": False,
            "window": config.layer_window(index),
            "position_encoding": rotary,
        })
        feed_forward = PartSpec("gated", {
            "hidden_size": config.hidden_size,
            "intermediate_size": config.intermediate_size,
            "prefix": prefix + "mlp.",
            "activation": config.hidden_act,
        })

        def norm(name):
            return PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps,
                                        "weight_name": prefix + name + ".weight"})

        blocks.append(PartSpec("pre_norm", {
            "mixer": mixer,
            "feed_forward": feed_forward,
            "mixer_norm": norm("input_layernorm"),
            "feed_forward_norm": norm("post_attention_layernorm"),
        }))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("lookup", {"vocab_size": config.vocab_size,
                                      "hidden_size": config.hidden_size,
                                      "weight_name": "model.embed_tokens.weight"}),
        blocks=blocks,
        schedule=[LayerCall(block=i, cache=i) for i in range(config.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps,
                                        "weight_name": "model.norm.weight"}),
        # a tied head reads the embedding's tensor; such a checkpoint may still carry a
        # copy under the head's own name, which nothing reads (mercury/model/loader.py:88-91)
        head=PartSpec("linear", {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size,
                                 "weight_name": "model.embed_tokens.weight"
                                 if config.tie_word_embeddings else "lm_head.weight"}),
        optional_tensors=("lm_head.weight",) if config.tie_word_embeddings else (),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, describe_qwen2)
