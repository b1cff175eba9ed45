"""The tiny configurations of the test-suite and helpers that write them as model folders.

tiny-A and tiny-B differ in every size and option (layers, width, heads and groups, head
size, feed-forward width, vocabulary, theta, sections, eps, tied or not, page size).  tiny-D
has the head size of the released models (128) and a feed-forward wider than 4,096, which puts
the kernels that serve those models on the whole-model comparisons: the tcgen05 prefill
attention, the fused decode attention at head size 128, the K-sliced chain products and the
4 KB-row streaming product.

tiny-C and tiny-E belong to another architecture, defined here and registered from here: the
same layer make-up with a sliding window on the layers of even index.  The Qwen2.5-VL
architecture itself never windows (its config.json cannot switch one on), so the window of the
attention part is exercised the way any other part would be: by a model that asks for it.

All use random weights from the engine's random-weights mode; folders are made in temporary
directories and never committed.
"""

from __future__ import annotations

ARCH = "Qwen2_5_VLForConditionalGeneration"
WINDOWED_ARCH = "TinyWindowedDecoder"


def _config(hidden, layers, heads, kv_heads, inter, vocab, theta, section, eps, tie, window, use_window, eos=None,
            arch=ARCH, layer_windows=None):
    cfg = {
        "architectures": [arch],
        "model_type": "qwen2_5_vl",
        "tie_word_embeddings": tie,
        "text_config": {
            "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "intermediate_size": inter, "vocab_size": vocab,
            "rms_norm_eps": eps, "rope_theta": theta,
            "rope_scaling": {"type": "mrope", "mrope_section": list(section)},
            "sliding_window": window, "use_sliding_window": use_window,
        },
    }
    if eos is not None:
        cfg["eos_token_id"] = eos
    if layer_windows is not None:
        cfg["text_config"]["layer_windows"] = list(layer_windows)
    return cfg


# 2 layers, hidden 64, 4 query / 2 kv heads, head 16, inter 128, vocab 256, tied
TINY_A = _config(64, 2, 4, 2, 128, 256, 10000.0, (2, 3, 3), 1e-6, True, 32768, False)
# 3 layers, hidden 192, 6 query / 1 kv head (MQA), head 32, inter 320, vocab 512, untied
TINY_B = _config(192, 3, 6, 1, 320, 512, 1000000.0, (4, 6, 6), 1e-5, False, 4096, False)
# 4 layers, hidden 240, 5 query / 5 kv heads (MHA), head 48, inter 136, vocab 300 (no power of two
# anywhere), window 24 on the even layers (the windowed architecture)
TINY_C = _config(240, 4, 5, 5, 136, 300, 50000.0, (8, 8, 8), 1e-5, False, 24, False, arch=WINDOWED_ARCH,
                 layer_windows=[24, None, 24, None])
# 2 layers, hidden 512, 4 query / 2 kv heads, head 128, inter 4224 (K of the down projection beyond
# 4,096: three slices in the chain kernel, 4 KB rows in the streaming kernel), vocab 640, untied
TINY_D = _config(512, 2, 4, 2, 4224, 640, 1000000.0, (16, 24, 24), 1e-6, False, 32768, False)
# 3 layers, hidden 384, 6 query / 2 kv heads, head 64, inter 416, vocab 333, tied, window 24 (less
# than two pages of 16) on layers 0 and 2 (the windowed architecture)
TINY_E = _config(384, 3, 6, 2, 416, 333, 10000.0, (8, 12, 12), 1e-6, True, 24, False, arch=WINDOWED_ARCH,
                 layer_windows=[24, None, 24])

# config, weight seed, page size
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 16), "E": (TINY_E, 4, 16)}

# bfloat16 replay against the float64 plain decoder on the same bfloat16-rounded weights: the
# largest difference of any logit that any replay test showed on a B200 (whole, last 32 one by
# one, portions, mixed, many live requests, long decoding), per configuration.  The tests allow
# three times that, so that a wrong key among a hundred or a window's edge off by one (1e-3 to
# 1e-2 on these logits) does not hide under rounding.  The 32-bit path showed at most 4.3e-6.
MEASURED_BF16_ERROR = {"A": 2.2e-3, "B": 6.8e-3, "C": 6.6e-3, "D": 1.7e-2, "E": 1.1e-2}
BF16_TOLERANCE = {name: 3 * err for name, err in MEASURED_BF16_ERROR.items()}


def register_windowed_architecture():
    """Registers ``TinyWindowedDecoder``: the Qwen2.5-VL layer make-up with the windows that
    ``text_config.layer_windows`` lists (None = all keys).  Nothing of the package is changed."""
    from qwen25vl_lite.config import Qwen25VLTextConfig, register_architecture
    from qwen25vl_lite.models.qwen2_5_vl import build_spec

    class WindowedConfig:
        def __init__(self, base, windows):
            self.base, self.windows = base, tuple(windows)
            self.eos_token_id = base.eos_token_id

        @classmethod
        def from_dict(cls, raw):
            return cls(Qwen25VLTextConfig.from_dict(raw), raw["text_config"]["layer_windows"])

    register_architecture(WINDOWED_ARCH, WindowedConfig.from_dict, lambda c: build_spec(c.base, c.windows), replace=True)


register_windowed_architecture()


def make_model_dir(tmp_dir: str, name: str, storage_dtype: str = "float32") -> str:
    import os

    from qwen25vl_lite.weights import write_random_model

    cfg, seed, _ = TINY[name]
    return write_random_model(os.path.join(str(tmp_dir), f"tiny-{name}-{storage_dtype}"), cfg, seed, storage_dtype)
