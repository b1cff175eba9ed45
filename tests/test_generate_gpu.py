"""Generation through the Python entry point and the command line, against the plain
implementation run without a cache."""

import subprocess
import sys
import os

import numpy as np
import pytest

from plain import decoder as plain
from tiny_models import TINY

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prompts(name, lengths, seed):
    vocab = TINY[name][0]["text_config"]["vocab_size"]
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


def test_greedy_tiny_a(model_dirs):
    """3 prompts of 5, 11 and 17 tokens, 8 greedy tokens each, pages of 4 tokens."""
    from qwen25vl_lite import LLM, SamplingParams
    prompts = _prompts("A", (5, 11, 17), 21)
    llm = LLM(model_dirs["A"], dtype="float32", num_blocks=64, block_size=4, max_num_seqs=4)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    cfg, w = plain.load_model_dir(model_dirs["A"], np.float64)
    for p, o in zip(prompts, outs):
        assert o.prompt_token_ids == p and o.finish_reason == "length"
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 8)
    assert llm.runner.cache.pages_in_use() == [0]


def test_temperature_chunked_mixed_tiny_b(model_dirs):
    """4 prompts of 1, 9, 23 and 40 tokens (the last with a 12-token image run, grid
    t1 x h3 x w4), portions of 7 mixed with decoding, temperature 0.8 seed 2, pages of 8."""
    from qwen25vl_lite import LLM, SamplingParams
    prompts = _prompts("B", (1, 9, 23, 40), 22)
    llm = LLM(model_dirs["B"], dtype="float32", num_blocks=32, block_size=8, max_num_seqs=4, max_num_batched_tokens=7)
    params = SamplingParams(temperature=0.8, seed=2, max_tokens=6, ignore_eos=True)
    ids = [llm.engine.add_request(p, params, image_spans=[(9, 1, 3, 4)] if len(p) == 40 else None) for p in prompts]
    outs = {o.seq_id: o for o in llm.engine.run_until_complete()}
    assert llm.engine.stats()["steps"] > 12                      # the prompts really were cut
    cfg, w = plain.load_model_dir(model_dirs["B"], np.float64)
    for i, p in zip(ids, prompts):
        pos, delta = plain.prompt_positions(len(p), [(9, 1, 3, 4)] if len(p) == 40 else [])
        want = plain.greedy_generate(cfg, w, p, 6, pos, delta, temperature=0.8, seed=2)
        assert outs[i].output_token_ids == want, f"prompt of {len(p)} tokens"


def test_preemption_on_the_device_changes_nothing(model_dirs):
    from qwen25vl_lite import LLM, SamplingParams
    prompts = _prompts("C", (30, 30, 30, 30), 23)
    params = SamplingParams(max_tokens=40, ignore_eos=True)
    roomy = LLM(model_dirs["C"], dtype="float32", num_blocks=64, block_size=16, max_num_seqs=4)
    want = [o.output_token_ids for o in roomy.generate(prompts, params)]
    tight = LLM(model_dirs["C"], dtype="float32", num_blocks=11, block_size=16, max_num_seqs=4)
    got = tight.generate(prompts, params)
    assert tight.engine.stats()["preemptions"] > 0
    assert [o.output_token_ids for o in got] == want
    assert tight.runner.cache.pages_in_use() == [0, 0]


def test_bfloat16_generation_runs(model_dirs, tmp_path):
    from qwen25vl_lite import LLM, SamplingParams
    from tiny_models import make_model_dir
    llm = LLM(make_model_dir(tmp_path, "B", "bfloat16"), dtype="bfloat16", num_blocks=32, block_size=16)
    outs = llm.generate(_prompts("B", (12, 33), 24), SamplingParams(max_tokens=10, temperature=0.7, seed=5, ignore_eos=True))
    assert [len(o.output_token_ids) for o in outs] == [10, 10]
    again = llm.generate(_prompts("B", (12, 33), 24), SamplingParams(max_tokens=10, temperature=0.7, seed=5, ignore_eos=True))
    assert [o.output_token_ids for o in again] == [o.output_token_ids for o in outs]     # seeded: reproducible


def test_command_line(model_dirs):
    prompt = _prompts("A", (9,), 25)[0]
    cmd = [sys.executable, "-m", "qwen25vl_lite.cli", "generate", "--model", model_dirs["A"], "--dtype", "float32",
           "--block-size", "4", "--num-blocks", "32", "--max-tokens", "5", "--ignore-eos",
           "--prompt-token-ids", ",".join(map(str, prompt))]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    cfg, w = plain.load_model_dir(model_dirs["A"], np.float64)
    assert res.stdout.strip().splitlines()[-1] == str(plain.greedy_generate(cfg, w, prompt, 5))
    res = subprocess.run(cmd[:-2], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert res.returncode == 2 and "--prompt-token-ids is required" in res.stderr
