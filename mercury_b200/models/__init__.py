"""Model descriptions. Importing this package registers the built-in architectures."""

from . import qwen2  # noqa: F401
from .model import Model  # noqa: F401
from .spec import LayerCall, ModelSpec  # noqa: F401
