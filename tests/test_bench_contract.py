"""What ``bench.py`` promises that needs no GPU: one line and exit code 2 for more than one GPU, the
reference arm's ``unavailable`` line where the reference is not installed or the workload is not the
one it measures, peaks read from the driver's file with the stated fallback, and byte / flop counts
that follow from the sizes alone."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    res = run_bench("--gpus", "2")
    assert res.returncode == 2
    assert len(res.stdout.strip().splitlines()) == 1 and "one GPU" in res.stdout


def test_the_reference_arm_measures_the_headline_workload_only():
    res = run_bench("--impl", "reference", "--config", "32b")
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_peaks_come_from_the_measured_file_or_the_stated_fallback(tmp_path, monkeypatch):
    import bench
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.load_peaks() == dict(bench.FALLBACK_PEAKS, source="fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6000.5, "bf16_tflops": 1600, "other": "x"}))
    peaks = bench.load_peaks()
    assert peaks["source"] == "measured" and peaks["hbm_gbs"] == 6000.5 and peaks["bf16_tflops"] == 1600.0
    assert peaks["bf16_tflops_sustained"] == bench.FALLBACK_PEAKS["bf16_tflops_sustained"]      # absent from the file
    (tmp_path / "MEASURED_PEAKS.json").write_text("{ not json")
    assert bench.load_peaks()["source"] == "fallback"


def test_byte_and_flop_counts_follow_from_the_sizes():
    import bench
    from qwen25vl_lite.engine import benchmark as B
    t = bench.CONFIG_3B["text_config"]
    layers = t["num_hidden_layers"]
    h, i, v = t["hidden_size"], t["intermediate_size"], t["vocab_size"]
    qkv = (t["num_attention_heads"] + 2 * t["num_key_value_heads"]) * 128
    per_layer = h * qkv + h * h + 3 * h * i
    assert B.layer_matrix_params(t) == per_layer
    assert B.weight_bytes(t, layers) == 2 * (layers * per_layer + v * h)        # tied: the table is read once, as the head
    assert B.kv_bytes_per_token(t, layers) == layers * 2 * t["num_key_value_heads"] * 128 * 2 == 36864
    flops = B.prefill_flops(t, layers, 2048)
    assert flops > 2 * 2048 * layers * per_layer and flops < 2.2 * 2048 * (layers * per_layer + v * h)
