"""Loading a model folder: config.json -> architecture -> model, tensors by name.

Name handling follows the reference's ``map_hf_name`` (src/qwen25vl_lite/model.py:52-73):
a decoder tensor may carry any of the architecture's prefixes.  Error handling is stricter
than the reference, which counts unknown tensors and skips them silently
(model.py:390-394) and lists at most eight missing ones (model.py:420-426): here one
``WeightsError`` lists every missing tensor, every unexpected one and every wrong shape.

Storage: matrices and the embedding are held in the engine's dtype (bfloat16 for serving,
float32 for the 32-bit path); vectors that enter float32 arithmetic (norm weights, biases)
are held in float32, which keeps a 32-bit tensor 32-bit and widens a bfloat16 one exactly.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.registry import resolve_architecture
from ..config.text_config import read_config_json
from .safetensors_io import SafetensorsFile, open_model_files

TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class WeightsError(RuntimeError):
    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"the weights under {model_dir!r} do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def canonical_name(raw: str, spec) -> Tuple[str, bool]:
    """(name without the architecture's prefix, whether the tensor is one to ignore)."""
    for p in spec.ignored_prefixes:
        if raw.startswith(p):
            return raw, True
    if raw in spec.unprefixed_names:
        return raw, False
    for p in sorted(spec.name_prefixes, key=len, reverse=True):
        if p and raw.startswith(p):
            return raw[len(p):], False
    return raw, False


def load_model(model_dir: str, dtype: str = "float32", device: str = "cuda:0"):
    """Returns ``(typed config, DecoderModel with weights on the device)``."""
    from ..models.decoder import DecoderModel

    if dtype not in TORCH_DTYPES:
        raise ValueError(f"dtype must be one of {sorted(TORCH_DTYPES)}, got {dtype!r}")
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    cfg = arch.config_from_dict(raw)
    model = DecoderModel(arch.build_spec(cfg))
    files = open_model_files(model_dir)
    where: Dict[str, Tuple[SafetensorsFile, str]] = {}
    unexpected: List[str] = []
    expected = model.expected_tensors()
    for f in files:
        for raw_name in f.names():
            name, ignore = canonical_name(raw_name, model.spec)
            if ignore:
                continue
            if name not in expected or name in where:
                unexpected.append(raw_name)
            else:
                where[name] = (f, raw_name)
    missing = [n for n, ts in expected.items() if n not in where and not ts.optional]
    wrong = []
    for name, (f, raw_name) in where.items():
        if tuple(f.shape(raw_name)) != tuple(expected[name].shape):
            wrong.append(f"{raw_name}: file has {list(f.shape(raw_name))}, model needs {list(expected[name].shape)}")
        elif not f.dtype(raw_name).is_floating_point:
            wrong.append(f"{raw_name}: file stores {f.dtype(raw_name)}, model needs a floating-point tensor")
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, sorted(missing), sorted(unexpected), sorted(wrong))

    def get_tensor(name: str) -> torch.Tensor:
        f, raw_name = where[name]
        return f.tensor(raw_name)

    model.load(get_tensor, set(where), device, TORCH_DTYPES[dtype])
    return cfg, model
