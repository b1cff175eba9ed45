"""Random-weights mode: a model folder (config.json + model.safetensors) from a
configuration and a seed.

The reference has no such mode in the engine; its tests let ``transformers`` initialise a
tiny model and save it (tests/conftest.py:75-86, scripts/make_tiny_model.py:22-54).  Here
the distributions are fixed: matrices and embeddings N(0, std), norm weights 1 + N(0, std),
biases N(0, std), std = 0.02, drawn tensor by tensor in the order of the model's tensor
list from one ``torch.Generator`` seeded with the seed.  The folder is written with the
``model.language_model.`` prefix that Qwen2.5-VL releases use.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterator, Tuple

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

STD = 0.02


def _draw(ts, gen: torch.Generator, device) -> torch.Tensor:
    t = torch.randn(ts.shape, generator=gen, dtype=torch.float32, device=device) * STD
    if ts.init == "norm":
        t += 1.0
    return t


def random_tensors(model, seed: int, device="cpu") -> Iterator[Tuple[str, Any, torch.Tensor]]:
    """Yields (canonical name, TensorSpec, float32 tensor) for every required tensor."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, ts in model.expected_tensors().items():
        if ts.optional:
            continue
        yield name, ts, _draw(ts, gen, device)


def write_random_model(model_dir: str, config_json: Dict[str, Any], seed: int, storage_dtype: str = "float32",
                       prefix: str = "model.language_model.") -> str:
    """Writes ``config.json`` and ``model.safetensors`` under ``model_dir``."""
    from ..models.decoder import DecoderModel

    arch = resolve_architecture(config_json)
    cfg = arch.config_from_dict(config_json)
    model = DecoderModel(arch.build_spec(cfg))
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[storage_dtype]
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config_json, fh, indent=1)
    unprefixed = set(model.spec.unprefixed_names)

    def named():
        for name, _, t in random_tensors(model, seed):
            yield (name if name in unprefixed else prefix + name), t.to(dtype)

    write_safetensors(os.path.join(model_dir, "model.safetensors"), named(),
                      metadata={"format": "pt", "seed": str(seed), "init": f"normal std {STD}"})
    return model_dir


def load_random_model(config_json: Dict[str, Any], seed: int, dtype: str = "bfloat16", device: str = "cuda:0"):
    """The same model without a folder: tensors are drawn on ``device`` (another stream of
    numbers than the CPU generator of ``write_random_model``) and handed to the parts.
    For benchmarks of sizes whose file would take minutes to write."""
    from ..models.decoder import DecoderModel

    arch = resolve_architecture(config_json)
    cfg = arch.config_from_dict(config_json)
    model = DecoderModel(arch.build_spec(cfg))
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    expected = model.expected_tensors()
    names = {n for n, ts in expected.items() if not ts.optional}
    target = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]

    def get_tensor(name: str) -> torch.Tensor:
        ts = expected[name]
        t = _draw(ts, gen, device)
        return t if ts.init != "matrix" else t.to(target)

    model.load(get_tensor, names, device, target)
    return cfg, model
