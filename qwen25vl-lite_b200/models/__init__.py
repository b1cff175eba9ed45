"""Model assembly and the architectures this engine knows.  Importing registers them."""

from . import qwen2_5_vl  # noqa: F401
from .decoder import DecoderModel, StopRuntime  # noqa: F401
