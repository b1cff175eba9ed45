"""Qwen2.5-VL text decoder as a ``ModelSpec``.

Layer make-up after the reference (src/qwen25vl_lite/text.py:188-215): every layer is a
pre-norm residual block of GQA attention (biased q/k/v, unbiased o) and a SwiGLU
feed-forward with two RMSNorms; a final RMSNorm; a head that is the embedding table when
``tie_word_embeddings``.  Checkpoint names follow src/qwen25vl_lite/model.py:52-73: the
decoder's tensors may carry ``model.language_model.``, ``language_model.``, ``model.`` or
no prefix, ``lm_head.weight`` never does, and ``visual.*`` belongs to the vision tower,
which this engine does not build.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.text_config import Qwen25VLTextConfig

ARCHITECTURE = "Qwen2_5_VLForConditionalGeneration"


def build_spec(cfg: Qwen25VLTextConfig, layer_windows=None) -> ModelSpec:
    """``layer_windows``: a window per layer (None = all keys) for builders of *other*
    architectures that reuse this make-up; this architecture's own config.json never sets one
    (the reference parses ``sliding_window`` and attends to every key,
    src/qwen25vl_lite/text.py:156-175)."""
    h, d = cfg.hidden_size, cfg.head_dim
    layers = []
    if layer_windows is None:
        layer_windows = [None] * cfg.num_hidden_layers
    if len(layer_windows) != cfg.num_hidden_layers:
        raise ValueError(f"{len(layer_windows)} windows for {cfg.num_hidden_layers} layers")
    for i, window in enumerate(layer_windows):
        layers.append(LayerSpec(
            block="prenorm_residual",
            mixer=PartSpec("gqa_attention", dict(hidden_size=h, num_heads=cfg.num_attention_heads,
                                                 num_kv_heads=cfg.num_key_value_heads, head_dim=d,
                                                 qkv_bias=True, out_bias=False, window=window), "self_attn."),
            feed_forward=PartSpec("swiglu", dict(hidden_size=h, intermediate_size=cfg.intermediate_size), "mlp."),
            norms=(PartSpec("rmsnorm", dict(dim=h, eps=cfg.rms_norm_eps), "input_layernorm."),
                   PartSpec("rmsnorm", dict(dim=h, eps=cfg.rms_norm_eps), "post_attention_layernorm.")),
            prefix=f"layers.{i}.",
        ))
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=h), "embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(dim=h, eps=cfg.rms_norm_eps), "norm."),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=h, tied=cfg.tie_word_embeddings),
                      "lm_head."),
        position=PartSpec("mrope", dict(head_dim=d, theta=cfg.rope_theta, sections=cfg.mrope_section)),
        name_prefixes=("model.language_model.", "language_model.", "model.", ""),
        ignored_prefixes=("model.visual.", "visual."),
        unprefixed_names=("lm_head.weight",),
    )


register_architecture(ARCHITECTURE, Qwen25VLTextConfig.from_dict, build_spec, replace=True)
