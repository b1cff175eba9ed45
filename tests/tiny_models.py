"""The tiny configurations of the test-suite and helpers that write them as model folders.

tiny-A and tiny-B differ in every size and option (layers, width, heads and groups, head
size, feed-forward width, vocabulary, theta, sections, eps, tied or not, page size);
tiny-C adds the sliding window.  All use random weights from the engine's random-weights
mode; folders are made in temporary directories and never committed.
"""

from __future__ import annotations

ARCH = "Qwen2_5_VLForConditionalGeneration"


def _config(hidden, layers, heads, kv_heads, inter, vocab, theta, section, eps, tie, window, use_window, eos=None):
    cfg = {
        "architectures": [ARCH],
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
    return cfg


# 2 layers, hidden 64, 4 query / 2 kv heads, head 16, inter 128, vocab 256, tied
TINY_A = _config(64, 2, 4, 2, 128, 256, 10000.0, (2, 3, 3), 1e-6, True, 32768, False)
# 3 layers, hidden 192, 6 query / 1 kv head (MQA), head 32, inter 320, vocab 512, untied
TINY_B = _config(192, 3, 6, 1, 320, 512, 1000000.0, (4, 6, 6), 1e-5, False, 4096, False)
# 4 layers, hidden 240, 5 query / 5 kv heads (MHA), head 48, inter 136, vocab 300 (no power of two
# anywhere), window 24 on the even layers
TINY_C = _config(240, 4, 5, 5, 136, 300, 50000.0, (8, 8, 8), 1e-5, False, 24, True)

TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16)}   # config, weight seed, page size


def make_model_dir(tmp_dir: str, name: str, storage_dtype: str = "float32") -> str:
    import os

    from qwen25vl_lite.weights import write_random_model

    cfg, seed, _ = TINY[name]
    return write_random_model(os.path.join(str(tmp_dir), f"tiny-{name}-{storage_dtype}"), cfg, seed, storage_dtype)
