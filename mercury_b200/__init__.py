"""mercury_b200: a single-GPU inference engine for the Qwen2 decoder on NVIDIA B200."""

from .config import EngineConfig, ModelConfig, Qwen2Config, register_architecture  # noqa: F401
from .engine import Engine, ModelRunner, StepEntry, StreamEvent  # noqa: F401
from .sampling import SamplingParams  # noqa: F401

__version__ = "0.1.0"
