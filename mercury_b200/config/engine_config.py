"""Engine knobs, with the reference's names where it has them (mercury/config.py:84-113).

Kept with their meaning: `model`, `device`, `dtype`, `block_size`, `num_blocks`,
`gpu_memory_fraction`, `max_running`, `prefill_budget`, `max_model_len`, `policy`,
`aging_tokens_per_s`, `max_wait_s`, `scan_limit`, `cryptographic_hashes`, `seed`,
`debug_invariants`. New, because this engine cuts prompts into portions and the reference
does not: `max_batched_tokens` (tokens of one step, decode tokens included) and
`prefill_chunk` (most tokens of one prompt in one step). `cuda_graphs` replays decode-only
steps from captured graphs. `prefix_caching` switches the hash lookup at admission.
`lookahead` lets the engine launch a step before it has read the tokens of the step in front.
`debug_poison_pages` fills cache pages with NaN whenever they change hands. `time_kernels`
runs every step eagerly with CUDA events around each class of kernel call and books the
milliseconds in the step records (for looking at a step, not for serving).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

import torch

POLICIES = ("fcfs", "lpm", "lpm_aging")

_DTYPE_BY_NAME = {
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
}


def engine_dtype(name: str) -> torch.dtype:
    """bfloat16 (what serving uses) or float32 (a true 32-bit path). The reference also
    lists float16 (mercury/config.py:11-19); this engine's kernels are not built for it."""
    if name not in _DTYPE_BY_NAME:
        raise ValueError(f"unsupported dtype {name!r}; choose bfloat16 or float32")
    return _DTYPE_BY_NAME[name]


@dataclass
class EngineConfig:
    model: str = ""
    device: str = "cuda"
    dtype: str = "bfloat16"

    block_size: int = 16
    num_blocks: int = 4096
    gpu_memory_fraction: float = 0.85

    max_running: int = 64
    prefill_budget: int = 8192
    max_batched_tokens: int = 8192
    prefill_chunk: int = 2048
    max_model_len: int = 8192

    policy: str = "fcfs"
    aging_tokens_per_s: float = 2000.0
    max_wait_s: float = 5.0
    scan_limit: int = 128

    prefix_caching: bool = True
    cryptographic_hashes: bool = False
    cuda_graphs: bool = True
    lookahead: bool = True
    seed: int = 0
    debug_invariants: bool = False
    debug_poison_pages: bool = False
    time_kernels: bool = False
    max_step_records: int = 500_000

    def __post_init__(self) -> None:
        if self.policy not in POLICIES:
            raise ValueError(f"policy must be one of {POLICIES}, got {self.policy!r}")
        engine_dtype(self.dtype)
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValueError("block_size must be a positive power of two")
        if self.max_running <= 0:
            raise ValueError("max_running must be positive")
        if self.max_batched_tokens < self.max_running:
            raise ValueError(
                f"max_batched_tokens ({self.max_batched_tokens}) must hold one decode token for "
                f"each of max_running ({self.max_running}) requests"
            )
        if self.prefill_chunk <= 0:
            raise ValueError("prefill_chunk must be positive")

    @property
    def torch_dtype(self) -> torch.dtype:
        return engine_dtype(self.dtype)

    @property
    def kv_capacity_tokens(self) -> int:
        return self.num_blocks * self.block_size

    def validate_against(self, max_position_embeddings: int) -> None:
        """The two start-up guards of mercury/config.py:133-145: a request may not outgrow
        the position table, and the pool must hold one request of full length, or that
        request would preempt itself for ever."""
        if self.max_model_len > max_position_embeddings:
            raise ValueError(
                f"max_model_len {self.max_model_len} exceeds the model's "
                f"{max_position_embeddings} positions"
            )
        if self.kv_capacity_tokens < self.max_model_len:
            raise ValueError(
                f"the page pool holds {self.kv_capacity_tokens} tokens but one request may "
                f"reach {self.max_model_len}; raise num_blocks above "
                f"{self.max_model_len // self.block_size} or lower max_model_len"
            )

    def to_dict(self) -> dict:
        return asdict(self)


def blocks_for_capacity(num_tokens: int, block_size: int = 16) -> int:
    """Pages that hold `num_tokens` (mercury/config.py:160-161)."""
    return max(1, -(-int(num_tokens) // block_size))


def autosize_blocks(kv_bytes_per_token: int, engine_cfg: EngineConfig, reserve_bytes: int = 0,
                    device_index: int = 0) -> int:
    """Pages that fit in what is left of the device after `reserve_bytes` (the weights),
    times `gpu_memory_fraction` (mercury/config.py:164-185)."""
    free, _total = torch.cuda.mem_get_info(device_index)
    budget = int(max(0, free - reserve_bytes) * engine_cfg.gpu_memory_fraction)
    blocks = budget // (kv_bytes_per_token * engine_cfg.block_size)
    if blocks < 1:
        raise RuntimeError(
            f"only {free / 2**30:.1f} GiB free and {reserve_bytes / 2**30:.1f} GiB reserved; "
            f"no room for a cache"
        )
    return int(blocks)
