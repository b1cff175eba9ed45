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


@pytest.mark.parametrize("hidden,heads,kv_heads,inter,batch", [(3584, 28, 4, 18944, 8), (5120, 40, 8, 27648, 13), (2048, 16, 2, 11008, 3)])
def test_captured_decode_steps_agree_with_kernel_by_kernel_steps_at_full_layer_sizes(hidden, heads, kv_heads, inter, batch):
    """Layer sizes of the 7B, 32B and 3B models (one layer, small vocabulary, random weights): decode
    steps replayed from CUDA graphs, where the products run as chains of one persistent kernel with K
    cut into slices, against the same steps launched kernel by kernel.  Query groups of 7, 5 and 8
    heads, widths that are no power of two, 8, 13 and 3 rows."""
    import torch
    from qwen25vl_lite import LLM
    from qwen25vl_lite.engine.runner import StepEntry
    from qwen25vl_lite.ops import kernels
    config = {"architectures": ["Qwen2_5_VLForConditionalGeneration"], "tie_word_embeddings": False,
              "text_config": {"hidden_size": hidden, "num_hidden_layers": 1, "num_attention_heads": heads,
                              "num_key_value_heads": kv_heads, "intermediate_size": inter, "vocab_size": 3000,
                              "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
                              "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
                              "sliding_window": 32768, "use_sliding_window": False}}
    outs = []
    for graphs in (True, False):
        llm = LLM(random_config=config, weights_seed=2, dtype="bfloat16", num_blocks=16 * 24, block_size=16, max_num_seqs=16,
                  max_num_batched_tokens=4096, max_model_len=384, cuda_graph=graphs)
        runner = llm.runner
        rng = np.random.default_rng(8)
        reqs = [runner.open_request(i) for i in range(batch)]
        runner.step([StepEntry(r, rng.integers(0, 3000, size=int(rng.integers(5, 200))).tolist(), []) for r in reqs])
        got = [runner.step([StepEntry(r, [int(rng.integers(0, 3000))], [0]) for r in reqs]).float().cpu().numpy() for _ in range(3)]
        assert runner.graph_replays == (3 if graphs else 0)
        assert int(kernels.error_flag("cuda:0")[0]) == 0
        outs.append(np.stack(got))
        del llm, runner
        torch.cuda.empty_cache()
    graph, eager = outs
    assert np.abs(graph - eager).max() <= 2e-2 * np.abs(eager).max()
