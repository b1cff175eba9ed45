"""The plain implementation against the reference's own decoder (committed outputs under
tests/golden, made by tests/golden/make_golden.py) and against itself."""

import os

import numpy as np
import pytest

from plain import decoder as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_decoder(model_dirs, name):
    gold = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    cfg, w = plain.load_model_dir(model_dirs[name])
    logits = plain.forward_logits(cfg, w, gold["token_ids"], gold["positions"])
    assert logits.shape == gold["logits"].shape
    assert np.abs(logits - gold["logits"]).max() < 2e-5
    # float64 arithmetic on the same weights agrees too: the oracle is not rounding-lucky
    cfg, w64 = plain.load_model_dir(model_dirs[name], np.float64)
    assert np.abs(plain.forward_logits(cfg, w64, gold["token_ids"], gold["positions"]) - gold["logits"]).max() < 2e-5


def test_prompt_positions_match_reference_rope_index():
    gold = np.load(os.path.join(GOLDEN, "tiny_B.npz"))
    start, t, h, w = (int(v) for v in gold["image"])
    pos, delta = plain.prompt_positions(len(gold["token_ids"]), [(start, t, h, w)])
    assert np.array_equal(pos, gold["positions"])
    assert delta == int(gold["rope_delta"]) == -8
    gold_a = np.load(os.path.join(GOLDEN, "tiny_A.npz"))
    pos, delta = plain.prompt_positions(len(gold_a["token_ids"]))
    assert np.array_equal(pos, gold_a["positions"]) and delta == 0


def test_engine_prompt_positions_match_reference_rope_index():
    from qwen25vl_lite.parts.position import prompt_positions

    gold = np.load(os.path.join(GOLDEN, "tiny_B.npz"))
    pos, delta = prompt_positions(len(gold["token_ids"]), [tuple(int(v) for v in gold["image"])])
    assert np.array_equal(pos, gold["positions"]) and delta == -8


def test_window_hides_old_keys():
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((12, 2, 16)) for _ in range(3))
    full = plain.causal_attention(q, k, v)
    win = plain.causal_attention(q, k, v, window=4)
    assert np.allclose(full[:4], win[:4])           # the first 4 queries see the same keys
    assert not np.allclose(full[8:], win[8:])
    # a window of 4 at query 11 is attention over keys 8..11 alone
    alone = plain.causal_attention(q[8:], k[8:], v[8:])
    assert np.allclose(alone[-1], win[-1])


def test_sampler_restatement():
    logits = np.random.default_rng(1).standard_normal(300).astype(np.float32)
    assert plain.sample(logits, 0.0) == int(np.argmax(logits))
    a = plain.sample(logits, 0.8, seed=2, token_index=0)
    assert a == plain.sample(logits, 0.8, seed=2, token_index=0)
    draws = {plain.sample(logits, 1.5, seed=2, token_index=i) for i in range(40)}
    assert len(draws) > 5
    # Gumbel-max draws follow softmax(logits / T): check frequencies on a small vocabulary
    small = np.asarray([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    counts = np.bincount([plain.sample(small, 1.0, seed=7, token_index=i) for i in range(4000)], minlength=4)
    p = np.exp(small) / np.exp(small).sum()
    assert np.abs(counts / 4000 - p).max() < 0.03
    # filters
    s = plain.filter_scores(small, top_k=2)
    assert np.isinf(s[2:]).all() and np.isfinite(s[:2]).all()
    s = plain.filter_scores(small, top_p=0.7)       # p = .64 .24 .09 .03: keeps the crossing token
    assert np.isfinite(s[:2]).all() and np.isinf(s[2:]).all()
    s = plain.filter_scores(small, min_p=0.2)       # keeps p >= 0.2 * 0.64
    assert np.isfinite(s[:2]).all() and np.isinf(s[2:]).all()
    out = plain.apply_penalties(small, [0, 0, 3], repetition=2.0, presence=0.5, frequency=0.25)
    assert np.allclose(out, [2.0 / 2 - 0.5 - 0.5, 1.0, 0.0, -1.0 * 2 - 0.5 - 0.25])
