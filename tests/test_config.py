"""Configuration: where keys are read, what is required, the registry."""

import copy
import json

import pytest

from qwen25vl_lite.config import ConfigError, Qwen25VLTextConfig, known_architectures, resolve_architecture
from tiny_models import TINY_A, TINY_B, TINY_C


def test_reads_text_config_and_rope_scaling():
    cfg = Qwen25VLTextConfig.from_dict(TINY_B)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (192, 3, 6, 1)
    assert cfg.head_dim == 32 and cfg.mrope_section == (4, 6, 6) and cfg.rope_theta == 1e6
    assert cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    assert cfg.sliding_window == 4096 and cfg.use_sliding_window is False


def test_flat_config_and_rope_parameters_and_top_level_keys():
    flat = dict(TINY_A["text_config"])
    section = flat.pop("rope_scaling")["mrope_section"]
    theta = flat.pop("rope_theta")
    flat.update(architectures=TINY_A["architectures"], rope_parameters={"mrope_section": section, "rope_theta": theta})
    assert Qwen25VLTextConfig.from_dict(flat) == Qwen25VLTextConfig.from_dict(TINY_A)
    nested = copy.deepcopy(TINY_A)
    del nested["text_config"]["rope_scaling"]
    nested["mrope_section"] = section
    assert Qwen25VLTextConfig.from_dict(nested).mrope_section == (2, 3, 3)


def test_no_size_is_defaulted():
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                "intermediate_size", "vocab_size", "rms_norm_eps", "rope_theta"):
        raw = copy.deepcopy(TINY_A)
        del raw["text_config"][key]
        with pytest.raises(ConfigError, match=key):
            Qwen25VLTextConfig.from_dict(raw)
    raw = copy.deepcopy(TINY_A)
    del raw["text_config"]["rope_scaling"]
    with pytest.raises(ConfigError, match="mrope_section"):
        Qwen25VLTextConfig.from_dict(raw)


def test_validation():
    def broken(**kw):
        raw = copy.deepcopy(TINY_A)
        raw["text_config"].update(kw)
        return raw
    for raw in (broken(num_attention_heads=3), broken(num_key_value_heads=3),
                broken(rope_scaling={"mrope_section": [2, 3, 4]}), broken(rope_scaling={"mrope_section": [4, 4]}),
                broken(use_sliding_window=True, sliding_window=None)):
        with pytest.raises(ConfigError):
            Qwen25VLTextConfig.from_dict(raw)


def test_use_sliding_window_is_refused_and_no_layer_of_the_architecture_windows():
    """The reference parses the flag and attends to every key (text.py:156-175); here the flag is
    an error, and a config.json of this architecture can never switch a window on."""
    raw = copy.deepcopy(TINY_A)
    raw["text_config"].update(use_sliding_window=True, sliding_window=24)
    with pytest.raises(ConfigError, match="use_sliding_window=true is not supported"):
        Qwen25VLTextConfig.from_dict(raw)
    arch = resolve_architecture(TINY_A)
    spec = arch.build_spec(arch.config_from_dict(TINY_B))          # sliding_window 4096, flag false
    assert all(layer.mixer.params["window"] is None for layer in spec.layers)


def test_eos_token_id_defaults_as_in_the_reference():
    assert Qwen25VLTextConfig.from_dict(TINY_A).eos_token_id == 151645          # config.py:147,188
    raw = copy.deepcopy(TINY_A)
    raw["eos_token_id"] = [7, 9]
    assert Qwen25VLTextConfig.from_dict(raw).eos_token_id == 7


def test_round_trip_and_param_count():
    cfg = Qwen25VLTextConfig.from_dict(TINY_B)
    again = Qwen25VLTextConfig.from_dict(json.loads(json.dumps(cfg.to_config_json(TINY_B["architectures"][0]))))
    assert again == cfg
    h, d, i, v = 192, 32, 320, 512
    per_layer = h * 6 * d + 6 * d + 2 * (h * d + d) + 6 * d * h + 3 * h * i + 2 * h
    assert cfg.num_params() == v * h + 3 * per_layer + h + v * h


def test_registry():
    assert "Qwen2_5_VLForConditionalGeneration" in known_architectures()
    arch = resolve_architecture(TINY_A)
    spec = arch.build_spec(arch.config_from_dict(TINY_B))
    assert len(spec.layers) == 3 and [s.layer for s in spec.schedule] == [0, 1, 2]
    windowed = resolve_architecture(TINY_C)                        # an architecture the tests register
    spec = windowed.build_spec(windowed.config_from_dict(TINY_C))
    assert spec.layers[0].mixer.params["window"] == 24 and spec.layers[1].mixer.params["window"] is None
    with pytest.raises(ValueError, match="unknown architecture.*known architectures.*Qwen2_5_VL"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ValueError, match="architectures"):
        resolve_architecture({})


def test_missing_config_file(tmp_path):
    from qwen25vl_lite.config import read_config_json
    with pytest.raises(FileNotFoundError, match="config.json"):
        read_config_json(str(tmp_path))
