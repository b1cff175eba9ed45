"""qwen25vl-lite for B200: a single-GPU inference engine for the Qwen2.5-VL text decoder.

``config``    typed configuration, the model-as-data spec, the architecture registry
``weights``   safetensors reading/writing, loading by tensor name, random models
``parts``     norm, position encoding, mixer, feed-forward, block: what layers are made of
``models``    generic decoder assembly and the architectures that are registered
``cache``     pages, groups, block tables, per-request state slots
``engine``    step function, scheduler, ``LLM``, trace replay
``sampling``  sampling parameters and the device sampler
``ops``       build and bindings of the CUDA kernels in ``csrc``
``cli``       the ``qwen25vl-lite`` command line
"""

__version__ = "0.1.0"

from .config import EngineConfig, Qwen25VLTextConfig, register_architecture, resolve_architecture  # noqa: F401,E402
from .sampling import SamplingParams  # noqa: F401,E402
from . import models  # noqa: F401,E402  (registers the architectures)
from .engine import LLM, LLMEngine, ModelRunner, RequestOutput  # noqa: F401,E402
from .weights import WeightsError, load_model, write_random_model  # noqa: F401,E402
