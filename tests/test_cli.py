"""The command line without a GPU: option names and defaults (the reference's where it has them,
src/qwen25vl_lite/cli.py:634-673: --model, --prompt-token-ids, --temperature, --top-p, --top-k,
--min-p, --max-tokens, --seed, --ignore-eos, --dtype, engine sizes), and ``random-model``, which
writes a model folder that loads back."""

import json

import pytest

from qwen25vl_lite import cli
from tiny_models import TINY_A


def test_generate_options_and_defaults():
    p = cli.build_parser()
    a = p.parse_args(["generate", "--model", "m", "--prompt-token-ids", "1,2,3"])
    assert (a.temperature, a.top_p, a.top_k, a.min_p, a.max_tokens, a.seed, a.ignore_eos) == (0.0, 1.0, -1, 0.0, 64, None, False)
    assert (a.dtype, a.block_size, a.max_num_seqs, a.no_chunked_prefill, a.random_weights, a.weights_seed) == \
           ("float32", 16, 8, False, False, 0)
    a = p.parse_args(["generate", "--model", "m", "--prompt-token-ids", "5", "--temperature", "0.7", "--top-k", "40", "--top-p",
                      "0.9", "--min-p", "0.05", "--max-tokens", "7", "--seed", "3", "--ignore-eos", "--dtype", "bfloat16",
                      "--num-blocks", "64", "--max-num-batched-tokens", "256", "--max-model-len", "512", "--no-chunked-prefill"])
    assert (a.temperature, a.top_k, a.top_p, a.min_p, a.max_tokens, a.seed, a.ignore_eos, a.dtype) == \
           (0.7, 40, 0.9, 0.05, 7, 3, True, "bfloat16")
    assert (a.num_blocks, a.max_num_batched_tokens, a.max_model_len, a.no_chunked_prefill) == (64, 256, 512, True)
    with pytest.raises(SystemExit):
        p.parse_args(["generate", "--prompt-token-ids", "1"])                 # --model is required
    with pytest.raises(SystemExit):
        p.parse_args(["generate", "--model", "m", "--dtype", "float16"])       # only the two engine dtypes


def test_the_other_subcommands_parse():
    p = cli.build_parser()
    a = p.parse_args(["replay", "--model", "m", "--out", "o"])
    assert (a.trace, a.dtype, a.max_tokens, a.page_size) == ("-", "float32", 4096, 16)
    a = p.parse_args(["bench", "--model", "m", "--batch", "4", "--prompt-len", "128", "--steps", "9"])
    assert (a.batch, a.prompt_len, a.steps) == (4, 128, 9)
    a = p.parse_args(["random-model", "--config", "c.json", "--out", "o", "--seed", "5", "--storage-dtype", "float32"])
    assert (a.seed, a.storage_dtype) == (5, "float32")


def test_random_model_writes_a_folder_that_loads_back(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert cli.main(["random-model", "--config", str(cfg), "--out", str(out), "--seed", "4"]) == 0
    assert json.loads((out / "config.json").read_text())["architectures"] == TINY_A["architectures"]
    assert (out / "model.safetensors").stat().st_size > 0
    # the same seed writes the same bytes, another seed other bytes
    out2, out3 = tmp_path / "model2", tmp_path / "model3"
    cli.main(["random-model", "--config", str(cfg), "--out", str(out2), "--seed", "4"])
    cli.main(["random-model", "--config", str(cfg), "--out", str(out3), "--seed", "5"])
    same = (out / "model.safetensors").read_bytes() == (out2 / "model.safetensors").read_bytes()
    other = (out / "model.safetensors").read_bytes() != (out3 / "model.safetensors").read_bytes()
    assert same and other
