"""Decoding settings of one request.  Fields, defaults and checks are the reference's
``SamplingParams`` (src/qwen25vl_lite/sampling.py:16-41); ``temperature == 0`` is greedy.
String ``stop`` sequences need a tokenizer, which the engine does not have; like the
reference's engine (src/qwen25vl_lite/engine.py:517-525) it refuses them."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = -1
    max_tokens: int = 512
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    min_p: float = 0.0
    seed: Optional[int] = None
    stop: Sequence[str] = field(default_factory=tuple)
    stop_token_ids: Sequence[int] = field(default_factory=tuple)
    ignore_eos: bool = False

    # (field, what its value must satisfy, the rule in words); the same rules as sampling.py:30-41
    _RULES = (
        ("temperature", lambda v: v >= 0, "0 (greedy) or more"),
        ("top_p", lambda v: 0.0 < v <= 1.0, "above 0 and at most 1"),
        ("max_tokens", lambda v: v >= 1, "at least 1"),
        ("repetition_penalty", lambda v: v > 0, "above 0 (1 switches it off)"),
        ("min_p", lambda v: 0.0 <= v <= 1.0, "between 0 and 1"),
    )

    def validate(self) -> None:
        for name, holds, rule in self._RULES:
            value = getattr(self, name)
            if not holds(value):
                raise ValueError(f"SamplingParams.{name} = {value!r}: must be {rule}")

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @property
    def has_filters(self) -> bool:
        return self.temperature > 0 and ((self.top_k and self.top_k > 0) or self.min_p > 0 or self.top_p < 1.0)
