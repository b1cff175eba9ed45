"""The true 32-bit path at the layer sizes of the released 3B model (hidden 2048, 16 query / 2 kv
heads of 128, feed-forward 11008, vocabulary 151,936, tied head) against the plain decoder in
float64: every way of cutting and batching, one request with an image run (3-axis positions);
and the whole 36-layer model in 32-bit on the device.

The reference's tested path is float32 end to end (src/qwen25vl_lite/engine.py:63,
src/qwen25vl_lite/cli.py:637); these are the sizes its formulas are written for
(src/qwen25vl_lite/config.py:81-95).  Two layers keep the float64 oracle to a few seconds."""

import numpy as np
import pytest

import replay_util as ru
from plain import decoder as plain

pytestmark = pytest.mark.gpu

CONFIG_3B = {
    "architectures": ["Qwen2_5_VLForConditionalGeneration"], "model_type": "qwen2_5_vl", "tie_word_embeddings": True,
    "text_config": {"hidden_size": 2048, "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 2,
                    "intermediate_size": 11008, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
                    "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
                    "sliding_window": 32768, "use_sliding_window": False},
}
VOCAB = 151936
LENGTHS = (33, 70, 129, 48)
IMAGE_REQUEST, IMAGE_SPAN = "r1", (9, 2, 3, 4)          # 24 tokens of request r1 are a t2 x h3 x w4 grid


@pytest.fixture(scope="module")
def full_size(tmp_path_factory):
    """(model folder, requests, their positions, float64 oracle logits).  Made once."""
    from qwen25vl_lite.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("full-size") / "two-layers-3b-f32"), CONFIG_3B, 5, "float32")
    rng = np.random.default_rng(31)
    reqs = {f"r{i}": rng.integers(0, VOCAB, size=n).tolist() for i, n in enumerate(LENGTHS)}
    positions = {IMAGE_REQUEST: plain.prompt_positions(len(reqs[IMAGE_REQUEST]), [IMAGE_SPAN])[0]}
    cfg, w = plain.load_model_dir(folder, np.float64)
    want = {rid: plain.forward_logits(cfg, w, ids, positions.get(rid)).astype(np.float32) for rid, ids in reqs.items()}
    del w
    return folder, reqs, positions, want


def _with_positions(steps, positions):
    """Gives the entries of requests with explicit positions their slice of them."""
    at = {}
    for s in steps:
        for e in s["entries"]:
            n = len(e["tokens"])
            a = at.get(e["id"], 0)
            if e["id"] in positions:
                e["positions"] = positions[e["id"]][:, a:a + n].tolist()
            at[e["id"]] = a + n
    return steps


def _check(got, want, what):
    for rid, ref in want.items():
        err = float(np.abs(got[rid] - ref).max())
        assert err < 1e-4, f"{what}: request {rid} differs from the plain decoder by {err:.3e}"


@pytest.mark.parametrize("mode", ["whole", "last_32_one_by_one", "portions", "mixed"])
def test_float32_at_3b_layer_sizes(full_size, mode):
    folder, reqs, positions, want = full_size
    if mode == "whole":
        steps = ru.whole(reqs)
    elif mode == "last_32_one_by_one":
        steps = ru.prefill_then_decode(reqs, 32)
    elif mode == "portions":
        steps = ru.portions(reqs, (7, 2, 40, 3, 2, 21, 5))
    else:
        steps = ru.mixed(reqs, seed=7, max_live=4)
        assert max(len(s["entries"]) for s in steps) >= 3
    steps = _with_positions(steps, positions)
    got, runner = ru.run_in_process(folder, "float32", steps, ru.max_live_tokens(steps), 16)
    _check(got, want, mode)
    runner.cache.check([])


def test_whole_3b_model_in_float32_fits_and_does_not_depend_on_the_cut():
    """All 36 layers in 32-bit (12.3 GB of weights): a prompt fed whole and the same prompt in
    portions of changing size give the same logits at its last position, and a few greedy tokens
    come out of the entry point."""
    import torch
    from qwen25vl_lite import LLM, SamplingParams
    from qwen25vl_lite.engine.runner import StepEntry
    config = {**CONFIG_3B, "text_config": {**CONFIG_3B["text_config"], "num_hidden_layers": 36}}
    llm = LLM(random_config=config, weights_seed=0, dtype="float32", num_blocks=64, block_size=16, max_num_seqs=4,
              max_num_batched_tokens=256, max_model_len=512)
    assert llm.model.weight_bytes() > 12.3e9
    ids = np.random.default_rng(32).integers(0, VOCAB, size=150).tolist()
    runner = llm.runner
    a, b = runner.open_request("whole"), runner.open_request("cut")
    whole = runner.step([StepEntry(a, ids, [len(ids) - 1])]).cpu().numpy()
    at = 0
    for n in (7, 2, 64, 3, 40, 34):
        out = runner.step([StepEntry(b, ids[at:at + n], [n - 1] if at + n == len(ids) else [])])
        at += n
    cut = out.cpu().numpy()
    assert np.isfinite(whole).all() and np.abs(whole).max() > 1e-3
    assert np.abs(whole - cut).max() < 2e-5
    runner.close_request(a)
    runner.close_request(b)
    outs = llm.generate([ids[:40]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert len(outs[0].output_token_ids) == 4 and int(np.argmax(whole[0])) < VOCAB
    del llm, runner
    torch.cuda.empty_cache()
