"""Random weights: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has no such mode; its tests fill a model by hand with
`normal_(std=0.05)` under `torch.manual_seed(7)` (tests/test_runner.py:52-55 of the
reference). Here each tensor is drawn from its own generator, seeded from the seed and the
tensor's name, so a tensor's values do not depend on which other tensors exist: matrices,
biases and embeddings are N(0, std) and norm weights 1 + N(0, std), as each part declares.
Values are drawn in float32 and stored as bfloat16 (or float32 on request); the 32-bit
engine then runs exactly the values the bfloat16 engine runs.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from ..config.model_config import ModelConfig, architecture_named
from ..parts.base import TensorSpec


def _generator_for(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int.from_bytes(digest, "big") >> 1)
    return gen


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, vocab_limit: int = 0):
    gen = _generator_for(seed, spec.name)
    if spec.kind == "int":
        return torch.randint(0, max(1, vocab_limit), spec.shape, generator=gen, dtype=torch.int32)
    values = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * spec.std
    if spec.init == "ones_normal":
        values = values + 1.0
    return values.to(dtype)


def random_tensors(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16,
                   std: float | None = None) -> dict[str, torch.Tensor]:
    """`{name: tensor}` for every tensor the architecture's model declares. `std`
    overrides the spread of the N(0, std) tensors (norm weights keep their own)."""
    from ..models.model import Model

    entry = architecture_named(config.architecture)
    model = Model(entry.describe(config))
    out = {}
    for spec in model.tensor_specs():
        if std is not None and spec.init == "normal":
            spec = TensorSpec(spec.name, spec.shape, spec.kind, spec.init, std)
        out[spec.name] = random_tensor(spec, seed, dtype)
    return out


def write_random_model(folder: str | Path, config: ModelConfig, seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float | None = None) -> Path:
    """Create `folder` with config.json and model.safetensors; returns the folder."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    tensors = {k: v.contiguous() for k, v in random_tensors(config, seed, dtype, std).items()}
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder
