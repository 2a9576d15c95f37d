"""Typed architecture configurations, read from the architecture's own config.json keys.

Every size and constant of a model comes from here; no part of the engine carries one.
`Qwen2Config` holds the field set of mercury/config.py:22-37 (`ModelConfig`) with the same
defaults for absent keys (mercury/config.py:56-70), plus the keys the reference silently
ignores and this engine either honours (the sliding window) or checks (`hidden_act`,
`rope_scaling`, `attention_bias`).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Callable


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key named."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    architecture: str

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The config.json dictionary that `from_dict` reads back to an equal object."""
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    hidden_act: str = "silu"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        def need(key: str) -> Any:
            if key not in raw:
                raise ConfigError(f"config.json has no {key!r}, which Qwen2 needs")
            return raw[key]

        arch = (raw.get("architectures") or ["Qwen2ForCausalLM"])[0]
        heads = int(need("num_attention_heads"))
        hidden = int(need("hidden_size"))
        layers = int(need("num_hidden_layers"))
        kv_heads = int(raw.get("num_key_value_heads", heads))
        head_dim = int(raw.get("head_dim") or hidden // heads)
        eos = raw.get("eos_token_id", [])
        if eos is None:
            eos = []
        if isinstance(eos, int):
            eos = [eos]

        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r}: the Qwen2 feed-forward here is SiLU-gated only")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is set; scaled rotary embeddings are not built")
        if raw.get("attention_bias", True) is False:
            raise ConfigError("attention_bias=false: Qwen2 carries a bias on q, k and v")
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads={heads} is not a multiple of num_key_value_heads={kv_heads}"
            )
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim={head_dim} must be even for rotary embeddings")

        use_window = bool(raw.get("use_sliding_window", False))
        window = int(raw.get("sliding_window") or 0)
        if use_window and window <= 0:
            raise ConfigError("use_sliding_window is true but sliding_window is not positive")
        return cls(
            architecture=arch,
            hidden_size=hidden,
            intermediate_size=int(need("intermediate_size")),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=int(need("vocab_size")),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_ids=tuple(int(t) for t in eos),
            bos_token_id=raw.get("bos_token_id"),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=int(raw.get("max_window_layers", layers)),
            hidden_act=act,
        )

    def layer_window(self, layer: int) -> int:
        """Window of one layer in tokens, 0 for full attention: with `use_sliding_window`
        the layers from `max_window_layers` on see only the last `sliding_window` keys."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out


# --------------------------------------------------------------------------- the registry

@dataclass(frozen=True)
class Architecture:
    """What the engine knows about one architecture name: how to read its config.json and
    how to turn that configuration into a model description (`ModelSpec`)."""

    name: str
    config_class: type
    describe: Callable[[ModelConfig], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, describe: Callable) -> None:
    """Add an architecture. `describe(config)` returns the `ModelSpec` to build."""
    _ARCHITECTURES[name] = Architecture(name, config_class, describe)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def architecture_named(name: str) -> Architecture:
    _load_builtin()
    entry = _ARCHITECTURES.get(name)
    if entry is None:
        raise ConfigError(
            f"architecture {name!r} is not registered; known: {', '.join(sorted(_ARCHITECTURES))}"
        )
    return entry


def _load_builtin() -> None:
    # The built-in model descriptions register themselves when imported.
    from .. import models  # noqa: F401


def read_model_config(folder: str | Path) -> tuple[Architecture, ModelConfig]:
    """Parse `<folder>/config.json` with the class its `architectures[0]` is registered to.

    The reference falls back to "Qwen2ForCausalLM" when the key is absent
    (mercury/config.py:46); so does this.
    """
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    raw = json.loads(path.read_text())
    return config_from_dict(raw)


def config_from_dict(raw: dict) -> tuple[Architecture, ModelConfig]:
    name = (raw.get("architectures") or ["Qwen2ForCausalLM"])[0]
    entry = architecture_named(name)
    return entry, entry.config_class.from_dict(raw)


def config_fields(config: ModelConfig) -> dict:
    return {f.name: getattr(config, f.name) for f in fields(config)}
