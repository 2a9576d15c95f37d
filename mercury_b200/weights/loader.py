"""Checkpoint tensors from safetensors, by tensor name.

File discovery follows mercury/model/loader.py:34-45 (an index file's shard list, else
model.safetensors, else every *.safetensors). Names are matched against what the model's
parts declare (`Model.tensor_specs()`), strictly in both directions; where the reference
stops at the first fault (mercury/model/loader.py:77-91), this collects all of them and
raises ONE error that lists missing tensors, unexpected tensors and wrong shapes.

Tensors come back on the CPU in their stored dtype; the storage rule (what stays 32-bit,
what becomes bfloat16, integer tables as int32) is applied where a part places them
(`PartSetup.place`).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open

from ..parts.base import TensorSpec


class WeightError(RuntimeError):
    """A checkpoint that does not fit the model; the message lists every fault."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {tuple(got)}, the model expects {tuple(want)}")
        for name, got, want in self.wrong_kind:
            lines.append(f"  wrong type: {name} is {got}, the model expects a {want} tensor")
        super().__init__("\n".join(lines))


def weight_files(folder: Path) -> list[Path]:
    index = folder / "model.safetensors.index.json"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        return sorted({folder / name for name in weight_map.values()})
    single = folder / "model.safetensors"
    if single.exists():
        return [single]
    shards = sorted(folder.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no safetensors weights under {folder}")
    return shards


def check_tensors(found: dict[str, tuple[tuple[int, ...], bool]], specs: list[TensorSpec],
                  optional: set[str] = frozenset()) -> None:
    """`found[name]` = (shape, is floating point). Raises `WeightError` unless the names are
    exactly the declared ones (plus `optional`) with the declared shapes."""
    wanted = {s.name: s for s in specs}
    missing = sorted(set(wanted) - set(found))
    unexpected = sorted(set(found) - set(wanted) - set(optional))
    wrong_shape, wrong_kind = [], []
    for name in sorted(set(found) & set(wanted)):
        shape, floating = found[name]
        if tuple(shape) != tuple(wanted[name].shape):
            wrong_shape.append((name, shape, wanted[name].shape))
        if floating != (wanted[name].kind == "float"):
            wrong_kind.append((name, "floating" if floating else "integer", wanted[name].kind))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(missing, unexpected, wrong_shape, wrong_kind)


def read_checkpoint(folder: str | Path, specs: list[TensorSpec],
                    optional: set[str] = frozenset()) -> dict[str, torch.Tensor]:
    """Every declared tensor of the checkpoint under `folder`, checked against `specs`."""
    folder = Path(folder)
    handles = [safe_open(str(f), framework="pt", device="cpu") for f in weight_files(folder)]
    where: dict[str, int] = {}
    found: dict[str, tuple[tuple[int, ...], bool]] = {}
    for number, handle in enumerate(handles):
        for name in handle.keys():
            piece = handle.get_slice(name)
            where[name] = number
            found[name] = (tuple(piece.get_shape()), piece.get_dtype().startswith(("F", "BF")))
    check_tensors(found, specs, optional)
    return {s.name: handles[where[s.name]].get_tensor(s.name) for s in specs}
