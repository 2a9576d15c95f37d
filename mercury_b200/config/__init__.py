from .engine_config import (  # noqa: F401
    POLICIES,
    EngineConfig,
    autosize_blocks,
    blocks_for_capacity,
    engine_dtype,
)
from .model_config import (  # noqa: F401
    Architecture,
    ConfigError,
    ModelConfig,
    Qwen2Config,
    architecture_named,
    config_from_dict,
    known_architectures,
    read_model_config,
    register_architecture,
)
