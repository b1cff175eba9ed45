#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-VL-3B sizes, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  The headline ``value`` is decoded tokens
a second at batch 8 after 2,048-token prompts (context capacity 4,096), timed on the device
over exactly K steps that are fed back-to-back; ``e2e`` is the same through the public
entry point (scheduler, host tokens in and out every step).  The same line carries the
2,048-token prefill, the decode step's HBM roofline, decode at batch 1 and 64, the clocks
seen while timing, and the number of this engine's kernel launches in the timed region.
The engine is single-GPU: for --gpus N > 1 one line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-VL-3B text decoder sizes (BASELINE.json configs[2])
CONFIG_3B = {
    "architectures": ["Qwen2_5_VLForConditionalGeneration"],
    "model_type": "qwen2_5_vl",
    "tie_word_embeddings": True,
    "text_config": {
        "hidden_size": 2048, "num_hidden_layers": 36, "num_attention_heads": 16, "num_key_value_heads": 2,
        "intermediate_size": 11008, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
        "sliding_window": 32768, "use_sliding_window": False,
    },
}
FULL_LAYERS = 36
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            mhz.append(int(parts[0]))
            mx = int(parts[1]) if parts[1].isdigit() else mx
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def matmul_flops_per_token(t, layers):
    h, d = t["hidden_size"], t["hidden_size"] // t["num_attention_heads"]
    nq, nkv, inter = t["num_attention_heads"], t["num_key_value_heads"], t["intermediate_size"]
    return layers * 2 * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter)


def weight_bytes(t, layers):
    h, d = t["hidden_size"], t["hidden_size"] // t["num_attention_heads"]
    nq, nkv, inter = t["num_attention_heads"], t["num_key_value_heads"], t["intermediate_size"]
    per_layer = h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter
    return 2 * (layers * per_layer + t["vocab_size"] * h)      # bf16; the head is the embedding table (tied)


def kv_bytes_per_token(t, layers):
    d = t["hidden_size"] // t["num_attention_heads"]
    return layers * 2 * t["num_key_value_heads"] * d * 2


def run_reference(args):
    """The unmodified reference (installed under baseline/_ref) on the same metric: 3B sizes,
    random bfloat16 weights, batch 8, 2,048-token prompts, through its own public API and stock
    settings (LLMEngine.add_request / step; no opt-in kernels, no CUDA graphs).  None of this
    repository's models, kernels or engine is imported on this path."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "qwen25vl_lite")):
        print(json.dumps({"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}))
        return 0
    sys.path.insert(0, ref)
    try:
        import numpy as np
        import torch

        import qwen25vl_lite as reference
        if os.path.realpath(os.path.dirname(reference.__file__)) != os.path.realpath(os.path.join(ref, "qwen25vl_lite")):
            raise RuntimeError("the reference package did not come first on sys.path")
        from qwen25vl_lite import EngineConfig, LLMEngine, ModelRunner, Qwen25VLConfig, SamplingParams
        from qwen25vl_lite.model import Qwen25VLLite

        t = dict(CONFIG_3B["text_config"])
        layers = args.layers or FULL_LAYERS
        t["num_hidden_layers"] = layers
        t["mrope_section"] = t.pop("rope_scaling")["mrope_section"]
        # the vision tower is built by the reference's model class but never run here; keep it tiny
        raw = {"text_config": t, "tie_word_embeddings": True,
               "vision_config": {"depth": 1, "hidden_size": 64, "intermediate_size": 64, "num_heads": 2,
                                 "out_hidden_size": t["hidden_size"], "fullatt_block_indexes": [0]}}
        cfg = Qwen25VLConfig.from_dict(raw)
        torch.manual_seed(0)
        with torch.device("cuda:0"):
            model = Qwen25VLLite(cfg)
        with torch.no_grad():
            for name, p in model.named_parameters():
                p.normal_(0.0, 0.02)
                if name.endswith("norm.weight") or "layernorm" in name:
                    p.add_(1.0)
        model = model.to(torch.bfloat16).eval()
        ecfg = EngineConfig(num_blocks=8 * CONTEXT_LEN // PAGE + 64, block_size=PAGE, max_num_seqs=8,
                            max_num_batched_tokens=8192, max_model_len=CONTEXT_LEN, enable_prefix_cache=False,
                            device="cuda:0", dtype=torch.bfloat16)
        engine = LLMEngine(ModelRunner(model, ecfg, device="cuda:0"), ecfg)
        rng = np.random.default_rng(0)
        params = SamplingParams(temperature=0.0, max_tokens=args.warmup + args.steps + 8, ignore_eos=True)
        for _ in range(8):
            engine.add_request(rng.integers(0, 150000, size=PROMPT_LEN).tolist(), params)
        with torch.no_grad():
            while engine.waiting or any(s.num_computed_tokens < len(s.prompt_token_ids) for s in engine.running):
                engine.step()
            for _ in range(args.warmup):
                engine.step()
            clocks = ClockSampler()
            clocks.start()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                engine.step()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
            clock_record = clocks.stop()
        value = 8 * args.steps / (ms / 1e3)
        d = t["hidden_size"] // t["num_attention_heads"]
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s, Qwen2.5-VL-3B dims, batch 8, 2048-token prompts",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (seeded uniform-random token ids, random-init weights N(0, 0.02))",
            "config": {"model": "Qwen2.5-VL-3B text dims", "layers": layers, "layers_full": FULL_LAYERS,
                       "hidden": t["hidden_size"], "q_heads": t["num_attention_heads"], "kv_heads": t["num_key_value_heads"],
                       "head_dim": d, "intermediate": t["intermediate_size"], "vocab": t["vocab_size"], "global_batch": 8,
                       "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "kv_page": PAGE, "parallelism": "single GPU"},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
            "clocks": clock_record}))
    except Exception as exc:  # the reference could not run here: say why, in one line
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200]}"}))
    return 0


def run_ours(args):
    import numpy as np
    import torch

    from qwen25vl_lite import LLM, SamplingParams
    from qwen25vl_lite.engine.runner import StepEntry
    from qwen25vl_lite.ops import kernels

    peaks = load_peaks()
    cfg = json.loads(json.dumps(CONFIG_3B))
    layers = args.layers or FULL_LAYERS
    cfg["text_config"]["num_hidden_layers"] = layers
    t = cfg["text_config"]
    max_batch = 64
    llm = LLM(random_config=cfg, weights_seed=0, dtype="bfloat16", num_blocks=max_batch * CONTEXT_LEN // PAGE,
              block_size=PAGE, max_num_seqs=max_batch, max_num_batched_tokens=8192, max_model_len=CONTEXT_LEN,
              cuda_graph=not args.no_cuda_graph)
    runner, engine = llm.runner, llm.engine
    rng = np.random.default_rng(0)
    vocab = t["vocab_size"]
    dev = torch.device("cuda:0")

    def prompts(n):
        return [rng.integers(0, vocab, size=PROMPT_LEN).tolist() for _ in range(n)]

    # ---- prefill: one prompt of 2,048 tokens, one step -------------------------------------
    def prefill_once():
        req = runner.open_request("prefill")
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ids = prompts(1)[0]
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry(req, ids, [PROMPT_LEN - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.close_request(req)
        return a.elapsed_time(b)

    for _ in range(3):
        prefill_once()
    prefill_ms = statistics.median(prefill_once() for _ in range(5))
    d = t["hidden_size"] // t["num_attention_heads"]
    prefill_flops = (PROMPT_LEN * matmul_flops_per_token(t, layers) + 2 * vocab * t["hidden_size"]
                     + layers * 4 * t["num_attention_heads"] * d * PROMPT_LEN * (PROMPT_LEN + 1) // 2)
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)}

    # ---- decode, device-timed: K steps fed back-to-back with given tokens -------------------
    def decode_device(batch, steps, warmup, sample=True):
        reqs = [runner.open_request(f"d{i}") for i in range(batch)]
        ps = prompts(batch)
        for i in range(0, batch, 4):
            runner.step([StepEntry(r, p, []) for r, p in zip(reqs[i:i + 4], ps[i:i + 4])])
        feed = rng.integers(0, vocab, size=(steps + warmup, batch))
        out = torch.empty(batch, dtype=torch.int32, device=dev)

        def one(k):
            logits = runner.step([StepEntry(r, [int(feed[k, i])], [0]) for i, r in enumerate(reqs)])
            kernels.sample_rows(logits, None, None, None, out)

        for k in range(warmup):
            one(k)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        launches0 = kernels.launch_count()
        a.record()
        for k in range(warmup, warmup + steps):
            one(k)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = kernels.launch_count() - launches0
        ctx = PROMPT_LEN + warmup + steps // 2
        for r in reqs:
            runner.close_request(r)
        return batch * steps / (ms / 1e3), ms / steps, launches, ctx

    # ---- decode, end to end: the public entry point, host tokens in and out -----------------
    def decode_e2e(batch, steps, warmup):
        params = SamplingParams(max_tokens=warmup + steps + 8, ignore_eos=True)
        for p in prompts(batch):
            engine.add_request(p, params)
        while engine.waiting or any(s.pending > 1 for s in engine.running):
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        for s in list(engine.running):
            engine.abort(s.seq_id)
        return batch * steps / dt

    if args.only_batch:             # for profiler runs at another batch size: that decode loop alone, a short line
        tok_s, ms, launches, ctx = decode_device(args.only_batch, args.steps, args.warmup)
        print(json.dumps({"decode_batch": args.only_batch, "tokens_per_s": tok_s, "ms_per_step": ms, "layers": layers,
                          "context": ctx, "gpu_launches": launches}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    value, ms_per_step, launches, ctx = decode_device(8, args.steps, args.warmup)
    clock_record = clocks.stop()
    if args.headline_only:          # for profiler runs: the headline loop and the prefill alone
        e2e_value = b1 = b64 = None
    else:
        e2e_value = decode_e2e(8, args.steps, args.warmup)
        small = max(8, args.steps // 4)
        b1, _, _, _ = decode_device(1, small, args.warmup)
        b64, _, _, _ = decode_device(64, small, args.warmup)

    step_bytes = weight_bytes(t, layers) + 8 * ctx * kv_bytes_per_token(t, layers)
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    n_groups = len(runner.cache.groups)
    h2d = 4 * (8 * (2 + 3 + n_groups) + 9 + 16 + 8 + 8 * n_groups * (-(-(ctx + 1) // PAGE)))
    line = {
        "metric": "decode tokens/s, Qwen2.5-VL-3B dims, batch 8, 2048-token prompts", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform-random token ids, "
        "random-init weights N(0, 0.02))",
        "config": {"model": "Qwen2.5-VL-3B text dims", "layers": layers, "layers_full": FULL_LAYERS, "hidden": t["hidden_size"],
                   "q_heads": t["num_attention_heads"], "kv_heads": t["num_key_value_heads"], "head_dim": d,
                   "intermediate": t["intermediate_size"], "vocab": vocab, "global_batch": 8, "seq_len": CONTEXT_LEN,
                   "prompt_len": PROMPT_LEN, "kv_page": PAGE, "parallelism": "single GPU",
                   "l2": "weights read per step (6.2 GB) exceed L2 (126 MB)", "peaks": peaks["source"]},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * 4},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": {"decode_b1": b1, "decode_b64": b64},
        "clocks": clock_record,
    }
    print(json.dumps(line))
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--headline-only", action="store_true", help="skip e2e and the batch 1 / 64 points")
    ap.add_argument("--no-cuda-graph", action="store_true", help="launch decode steps kernel by kernel (for profilers)")
    ap.add_argument("--only-batch", type=int, default=0, help="time decode steps at this batch size only (for profilers)")
    args = ap.parse_args(argv)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
