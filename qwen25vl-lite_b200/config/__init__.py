"""Typed configuration, the model-as-data spec, and the architecture registry."""

from .engine_config import EngineConfig  # noqa: F401
from .registry import (Architecture, known_architectures, register_architecture,  # noqa: F401
                       resolve_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
from .text_config import ConfigError, Qwen25VLTextConfig, read_config_json  # noqa: F401
