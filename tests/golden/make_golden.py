"""Make the golden logits: run RishDevs/mercury's own model code on the CPU in float32 on
the tiny random models of the test-suite and store the logits of one sequence each.

    python tests/golden/make_golden.py /path/to/mercury/checkout

The reference is imported from the path given (its `mercury` package must be importable
there; nothing is installed). Its `Qwen2ForCausalLM` is filled with this repository's
seeded random tensors by name and driven through its `ModelRunner.forward_prompt`, i.e.
its own paged prefill path. Output: tiny_<name>.f32 (little-endian float32 [T, vocab]) and
tiny_<name>.json (config, tokens, shape) beside this script.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    from mercury.allocator import BlockAllocator
    from mercury.config import EngineConfig, ModelConfig
    from mercury.model.qwen2 import Qwen2ForCausalLM
    from mercury.runner import ModelRunner

    from tiny import RAW, random_tokens, tiny_model

    # (name, tokens): D and E add one KV head under 7 and under 32 query heads, head sizes
    # 64 and 80; C is left out, its sliding window is not something the reference computes
    for name, length in (("A", 40), ("B", 40), ("D", 24), ("E", 24)):
        raw, _cfg, tensors = tiny_model(name)
        ref_cfg = ModelConfig.from_dict(raw)
        model = Qwen2ForCausalLM(ref_cfg, fused_norm=False).to(torch.float32).eval()
        params = dict(model.named_parameters())
        assert set(params) == set(tensors), sorted(set(params) ^ set(tensors))
        with torch.no_grad():
            for key, value in tensors.items():
                params[key].copy_(value.float())
        engine_cfg = EngineConfig(model="tiny", device="cpu", dtype="float32", num_blocks=16,
                                  block_size=16, max_model_len=128, fused_rmsnorm=False)
        model.init_rotary("cpu", torch.float32, 128)
        runner = ModelRunner(engine_cfg, alloc=BlockAllocator(16, 16), model=model,
                             model_config=ref_cfg)
        tokens = random_tokens(length, RAW[name]["vocab_size"], 9)
        logits = runner.forward_prompt(tokens, all_positions=True)
        logits.numpy().astype("<f4").tofile(HERE / f"tiny_{name}.f32")
        (HERE / f"tiny_{name}.json").write_text(json.dumps(
            {"config": raw, "tokens": tokens, "shape": list(logits.shape)}, indent=1) + "\n")
        print(name, tuple(logits.shape), float(logits.abs().max()))


if __name__ == "__main__":
    main(sys.argv[1])
