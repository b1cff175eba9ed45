"""Typed configuration of the Qwen2.5-VL text decoder, read from the model's own config.json.

Restates what zhangjianbang-nb/qwen25vl-lite reads (src/qwen25vl_lite/config.py:77-95 for
the text fields, :163-178 for where the rope keys and the tie flag may sit), with two
differences that are deliberate:

* sizes are never defaulted.  The reference fills every absent key with the 3B value
  (config.py:81-95), so a flat config silently becomes a 3B model; here a missing size is
  an error that names the key.
* ``use_sliding_window: true`` is refused.  The reference parses ``sliding_window`` /
  ``use_sliding_window`` and derives ``layer_types()`` (config.py:93-94, 105-109) but its
  attention never consults them (src/qwen25vl_lite/text.py:156-175), so a file that sets the
  flag would silently run full attention there.  Here it is an error that says so, instead of
  logits that nobody asked for; ``sliding_window`` itself is kept as read.
* ``eos_token_id`` defaults to 151645 when config.json has none, as config.py:147,188 does.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

REQUIRED_SIZES = (
    "hidden_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "intermediate_size",
    "vocab_size",
    "rms_norm_eps",
    "rope_theta",
    "mrope_section",
)


DEFAULT_EOS_TOKEN_ID = 151645      # the reference's default (src/qwen25vl_lite/config.py:147,188)


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can build."""


@dataclass(frozen=True)
class Qwen25VLTextConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    mrope_section: Tuple[int, ...]
    tie_word_embeddings: bool = True
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    eos_token_id: Optional[int] = DEFAULT_EOS_TOKEN_ID
    max_position_embeddings: Optional[int] = None

    # ---- derived -------------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        """hidden_size // num_attention_heads; no ``head_dim`` key is read (config.py:97-99)."""
        return self.hidden_size // self.num_attention_heads

    @property
    def num_key_value_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def num_params(self) -> int:
        """Parameter count, as config.py:120-134 accounts it."""
        h, d, inter = self.hidden_size, self.head_dim, self.intermediate_size
        per_layer = h * self.num_attention_heads * d + self.num_attention_heads * d
        per_layer += 2 * (h * self.num_key_value_heads * d + self.num_key_value_heads * d)
        per_layer += self.num_attention_heads * d * h + 3 * h * inter + 2 * h
        total = self.vocab_size * h + per_layer * self.num_hidden_layers + h
        if not self.tie_word_embeddings:
            total += self.vocab_size * h
        return total

    # ---- validation ----------------------------------------------------------------
    def validate(self) -> None:
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                     "intermediate_size", "vocab_size"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads {self.num_attention_heads}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 or sum(self.mrope_section) * 2 != self.head_dim:
            raise ConfigError(
                f"mrope_section {list(self.mrope_section)} must sum to head_dim/2 = {self.head_dim / 2:g}")
        if len(self.mrope_section) != 3:
            raise ConfigError(f"mrope_section needs three entries (t, h, w), got {list(self.mrope_section)}")
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        if self.use_sliding_window:
            raise ConfigError(
                "use_sliding_window=true is not supported: the decoder this engine restates never applies a window "
                "(it parses the key and attends to every key); set use_sliding_window to false")

    # ---- reading / writing ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen25VLTextConfig":
        """``raw`` is a whole config.json.  Sizes come from ``text_config`` when present,
        else from the top level; the rope keys from ``rope_scaling`` / ``rope_parameters``
        (either level) or a plain key; the tie flag from the text block, then the top level."""
        text = dict(raw.get("text_config") or {})
        flat = not text
        if flat:
            text = dict(raw)
        for key in ("rope_scaling", "rope_parameters"):
            block = raw.get(key) or text.get(key)
            if isinstance(block, dict):
                for k in ("mrope_section", "rope_theta"):
                    if k in block:
                        text.setdefault(k, block[k])
        for k in ("rope_theta", "mrope_section"):
            if k in raw:
                text.setdefault(k, raw[k])
        missing = [k for k in REQUIRED_SIZES if text.get(k) is None]
        if missing:
            where = "config.json" if flat else "config.json (text_config)"
            raise ConfigError(f"{where} lacks required key(s): {', '.join(missing)}")
        tie = text.get("tie_word_embeddings", raw.get("tie_word_embeddings", True))
        eos = raw.get("eos_token_id", text.get("eos_token_id", DEFAULT_EOS_TOKEN_ID))
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        window = text.get("sliding_window")
        cfg = cls(
            hidden_size=int(text["hidden_size"]),
            num_hidden_layers=int(text["num_hidden_layers"]),
            num_attention_heads=int(text["num_attention_heads"]),
            num_key_value_heads=int(text["num_key_value_heads"]),
            intermediate_size=int(text["intermediate_size"]),
            vocab_size=int(text["vocab_size"]),
            rms_norm_eps=float(text["rms_norm_eps"]),
            rope_theta=float(text["rope_theta"]),
            mrope_section=tuple(int(s) for s in text["mrope_section"]),
            tie_word_embeddings=bool(tie),
            sliding_window=None if window is None else int(window),
            use_sliding_window=bool(text.get("use_sliding_window", False)),
            eos_token_id=None if eos is None else int(eos),
            max_position_embeddings=(None if text.get("max_position_embeddings") is None
                                     else int(text["max_position_embeddings"])),
        )
        cfg.validate()
        return cfg

    def to_config_json(self, architecture: str) -> Dict[str, Any]:
        """A config.json in the layout Qwen2.5-VL releases use: sizes under ``text_config``,
        the section under ``rope_scaling``, the tie flag at the top."""
        text = asdict(self)
        text.pop("tie_word_embeddings")
        text.pop("eos_token_id")
        section = list(text.pop("mrope_section"))
        text = {k: v for k, v in text.items() if v is not None}
        text["rope_scaling"] = {"type": "mrope", "mrope_section": section}
        out: Dict[str, Any] = {
            "architectures": [architecture],
            "model_type": "qwen2_5_vl",
            "tie_word_embeddings": self.tie_word_embeddings,
            "text_config": text,
        }
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = model_dir if model_dir.endswith(".json") else os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json under {model_dir!r}; --model must name a model folder")
    with open(path, "r", encoding="utf-8") as fh:
        return json.load(fh)
