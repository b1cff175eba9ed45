#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-VL sizes, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 3b|7b-trace|32b]

One "step" is one decode step of the whole batch.  The default run (``--config 3b``) has the 3B
layer sizes: the headline ``value`` is decoded tokens a second at batch 8 after 2,048-token
prompts (context capacity 4,096), timed on the device over exactly K steps that are fed
back-to-back; ``e2e`` is the same through the public entry point (scheduler, host tokens in and
out every step).  The same line carries the 2,048-token prefill, the decode step's HBM roofline,
decode at batch 1 and 64, the clocks seen while timing, and the number of this engine's kernel
launches in the timed region.  ``--config 7b-trace`` runs a continuous-batching trace of 128
requests at the 7B sizes, ``--config 32b`` decode at batch 1 / 8 / 32 after 8,192-token prompts and
a 2,048-token prefill at the 32B sizes; each prints one line of its own.
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


def _sizes(hidden, layers, heads, kv_heads, inter, vocab, tied):
    return {
        "architectures": ["Qwen2_5_VLForConditionalGeneration"],
        "model_type": "qwen2_5_vl",
        "tie_word_embeddings": tied,
        "text_config": {
            "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": kv_heads, "intermediate_size": inter, "vocab_size": vocab, "rms_norm_eps": 1e-6,
            "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
            "sliding_window": 32768, "use_sliding_window": False,
        },
    }


# the text decoder sizes of the Qwen2.5-VL releases (3B: the headline configuration)
CONFIG_3B = _sizes(2048, 36, 16, 2, 11008, 151936, True)
CONFIG_7B = _sizes(3584, 28, 28, 4, 18944, 152064, False)
CONFIG_32B = _sizes(5120, 64, 40, 8, 27648, 152064, False)
FULL_LAYERS = 36
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE = 16
# Seconds of rest between a timed decode loop's prompts and its warm-up steps: the prompts' products run
# at the power cap and leave the SM clock lowered for some tens of milliseconds, which 20 timed
# steps of 2 ms would spend at 1.6 to 1.9 GHz instead of the 1.965 GHz decode steps run at by
# themselves (2.18 to 2.45 ms a step without the rest, 2.05 ms with it or over 256 steps).
SETTLE_S = 0.25
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
    """Samples SM clocks and throttle reasons while a region is timed: through NVML in a thread of this
    process (what ``nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons...`` reads,
    without the tool).  ``nvidia-smi -lms`` beside the run held the GPU for 2 to 4 ms at each of its
    polls: over 20 timed steps of 2 ms that was 4 to 10 % of the figure; a poll through NVML takes
    tens of microseconds.  Falls back to ``nvidia-smi`` where the NVML binding is missing."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    INTERVAL_S = 0.05

    def __init__(self):
        self.proc = None
        self.lines = []
        self.samples = []          # (sm MHz, max MHz, reason bits) from NVML
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    # ---- NVML ----
    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(0)

    def _sample(self):
        nv, h = self._nvml
        reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
        self.samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM),
                             int(reasons)))

    def _poll(self):
        while not self._stop.wait(self.INTERVAL_S):
            try:
                self._sample()
            except Exception:
                return

    def start(self):
        """Returns when the sampler runs (NVML loaded and a first sample taken, which is dropped)."""
        try:
            self._nvml = self._nvml_handle()
            self._sample()
            del self.samples[:]
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._nvml = None
        self._start_tool()

    def stop(self):
        if self._nvml is not None:
            try:
                self._sample()                        # at least one sample, taken under load: the region has just ended
            except Exception:
                pass
            self._stop.set()
            if self._thread is not None:
                self._thread.join(timeout=2.0)
            nv = self._nvml[0]
            bits = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            mhz = [m for m, _, _ in self.samples]
            reasons = sorted(n for n, bit in bits.items() if any(r & bit for _, _, r in self.samples))
            return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": self.samples[0][1] if self.samples else None,
                    "reasons": reasons, "samples": len(mhz), "source": "nvml"}
        return self._stop_tool()

    # ---- nvidia-smi, where there is no NVML binding ----
    def _start_tool(self):
        """Returns when the first sample has come (or after five seconds): nvidia-smi's own start
        can hold the driver for up to a second, which must not fall into what is timed."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
            return
        deadline = time.time() + 5.0
        while not self.lines and time.time() < deadline and self.proc.poll() is None:
            time.sleep(0.02)
        del self.lines[:]

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def _stop_tool(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            mhz.append(int(parts[0]))
            mx = int(parts[1]) if parts[1].isdigit() else mx
            for n, v in zip(self.NAMES, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz), "source": "nvidia-smi"}


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
            torch.cuda.synchronize()
            time.sleep(SETTLE_S)                           # the same rest as our own arm gets
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
                       "seq_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "kv_page": PAGE, "parallelism": "single GPU",
                       "l2": "weights read per step exceed L2 (126 MB)", "peaks": load_peaks()["source"],
                       "settle_ms": int(SETTLE_S * 1e3)},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
            "clocks": clock_record}))
    except Exception as exc:  # the reference could not run here: say why, in one line
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc).splitlines()[0][:200]}"}))
    return 0


def _base_line(metric, value, args, ms_per_step, cfg, layers, batch, seq_len, prompt_len, peaks, extra_config=None):
    t = cfg["text_config"]
    config = {"model": metric.split(",")[1].strip() if "," in metric else metric, "layers": layers,
              "layers_full": t["num_hidden_layers"], "hidden": t["hidden_size"], "q_heads": t["num_attention_heads"],
              "kv_heads": t["num_key_value_heads"], "head_dim": t["hidden_size"] // t["num_attention_heads"],
              "intermediate": t["intermediate_size"], "vocab": t["vocab_size"], "global_batch": batch, "seq_len": seq_len,
              "prompt_len": prompt_len, "kv_page": PAGE, "parallelism": "single GPU",
              "l2": "weights read per step exceed L2 (126 MB)", "peaks": peaks["source"], "settle_ms": int(SETTLE_S * 1e3)}
    config.update(extra_config or {})
    return {"metric": metric, "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform-random token ids, random-init weights N(0, 0.02))", "config": config}


def run_ours(args):
    import numpy as np
    import torch

    from qwen25vl_lite import LLM
    from qwen25vl_lite.engine import benchmark as B

    peaks = load_peaks()
    cfg = json.loads(json.dumps(CONFIG_3B))
    layers = args.layers or FULL_LAYERS
    t = cfg["text_config"]
    full_layers, t["num_hidden_layers"] = t["num_hidden_layers"], layers
    max_batch = 64
    llm = LLM(random_config=cfg, weights_seed=0, dtype=args.dtype, num_blocks=max_batch * CONTEXT_LEN // PAGE,
              block_size=PAGE, max_num_seqs=max_batch, max_num_batched_tokens=8192, max_model_len=CONTEXT_LEN,
              cuda_graph=not args.no_cuda_graph)
    element = 2 if args.dtype == "bfloat16" else 4
    runner, engine = llm.runner, llm.engine
    rng = np.random.default_rng(0)
    vocab = t["vocab_size"]

    # ---- prefill: one prompt of 2,048 tokens, one step -------------------------------------
    prefill_ms = B.time_prefill(runner, PROMPT_LEN, vocab, rng)
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": B.prefill_flops(t, layers, PROMPT_LEN) / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
               # the same against the library's throughput in a seconds-long loop under the power cap, which is the
               # state eight prompts in a row leave the GPU in
               "frac_sustained": B.prefill_flops(t, layers, PROMPT_LEN) / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)}

    if args.only_batch:             # for profiler runs at another batch size: that decode loop alone, a short line
        r = B.time_decode_steps(runner, args.only_batch, PROMPT_LEN, args.steps, args.warmup, vocab, rng, settle_s=SETTLE_S)
        print(json.dumps({"decode_batch": args.only_batch, "tokens_per_s": r["tokens_per_s"], "ms_per_step": r["ms_per_step"],
                          "layers": layers, "context": r["context"], "gpu_launches": r["launches"]}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    head = B.time_decode_steps(runner, 8, PROMPT_LEN, args.steps, args.warmup, vocab, rng, settle_s=SETTLE_S)
    clock_record = clocks.stop()
    points = {}
    if args.headline_only:          # for profiler runs: the headline loop and the prefill alone
        e2e_value = None
    else:
        e2e_value = B.time_decode_e2e(engine, 8, PROMPT_LEN, args.steps, args.warmup, vocab, rng, settle_s=SETTLE_S)
        for b in (1, 16, 17, 32, 64):      # every point over as many steps as the headline
            points[f"decode_b{b}"] = B.time_decode_steps(runner, b, PROMPT_LEN, args.steps, args.warmup, vocab, rng, settle_s=SETTLE_S)["tokens_per_s"]

    ctx = head["context"]
    step_bytes = B.weight_bytes(t, layers, element) + 8 * ctx * B.kv_bytes_per_token(t, layers, element)
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    n_groups = len(runner.cache.groups)
    h2d = 4 * (8 * (2 + 3 + n_groups) + 9 + 16 + 8 + 8 * n_groups * (-(-(ctx + 1) // PAGE)))
    t["num_hidden_layers"] = full_layers
    line = _base_line("decode tokens/s, Qwen2.5-VL-3B dims, batch 8, 2048-token prompts", head["tokens_per_s"], args,
                      head["ms_per_step"], cfg, layers, 8, CONTEXT_LEN, PROMPT_LEN, peaks)
    line["config"]["model"] = "Qwen2.5-VL-3B text dims"
    if args.dtype == "float32":      # the true 32-bit path: plain FMA products, no tensor cores, so no tensor-peak fraction
        line["dtype"] = "fp32"
        prefill["frac"] = None
    line.update({
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * 4},
        "gpu_launches": head["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": points,
        "clocks": clock_record,
    })
    print(json.dumps(line))
    return 0


def run_32b(args):
    """Decode at batch 1, 8 and 32 after 8,192-token prompts and one 2,048-token prefill at the 32B
    sizes (65.5 GB of bfloat16 weights, up to 70 GB of cache)."""
    import numpy as np

    from qwen25vl_lite import LLM
    from qwen25vl_lite.engine import benchmark as B

    peaks = load_peaks()
    cfg = json.loads(json.dumps(CONFIG_32B))
    t = cfg["text_config"]
    layers = args.layers or t["num_hidden_layers"]
    full_layers, t["num_hidden_layers"] = t["num_hidden_layers"], layers
    prompt_len = 8192
    context = prompt_len + args.steps + args.warmup + 64              # every timed and warm-up step adds a token
    llm = LLM(random_config=cfg, weights_seed=0, dtype="bfloat16", num_blocks=32 * (-(-context // PAGE)), block_size=PAGE,
              max_num_seqs=32, max_num_batched_tokens=8192, max_model_len=context, cuda_graph=not args.no_cuda_graph)
    rng = np.random.default_rng(0)
    vocab = t["vocab_size"]
    prefill_ms = B.time_prefill(llm.runner, PROMPT_LEN, vocab, rng, warmup=2, repeats=3)
    prefill = {"value": PROMPT_LEN / (prefill_ms / 1e3), "tokens": PROMPT_LEN, "ms": prefill_ms,
               "frac": B.prefill_flops(t, layers, PROMPT_LEN) / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
               # the same against the library's throughput in a seconds-long loop under the power cap, which is the
               # state eight prompts in a row leave the GPU in
               "frac_sustained": B.prefill_flops(t, layers, PROMPT_LEN) / (prefill_ms / 1e3) / (peaks["bf16_tflops_sustained"] * 1e12)}
    clocks = ClockSampler()
    clocks.start()
    points, roofs, launches = {}, {}, 0
    for b in (8, 1, 32):
        r = B.time_decode_steps(llm.runner, b, prompt_len, args.steps, args.warmup, vocab, rng, prefill_group=1, settle_s=SETTLE_S)
        points[f"decode_b{b}"] = r["tokens_per_s"]
        step_bytes = B.weight_bytes(t, layers) + b * r["context"] * B.kv_bytes_per_token(t, layers)
        roofs[f"decode_b{b}"] = step_bytes / (r["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"]
        if b == 8:
            head, launches = r, r["launches"]
    clock_record = clocks.stop()
    t["num_hidden_layers"] = full_layers
    line = _base_line("decode tokens/s, Qwen2.5-VL-32B dims, batch 8, 8192-token prompts", head["tokens_per_s"], args,
                      head["ms_per_step"], cfg, layers, 8, context, prompt_len, peaks)
    line["config"]["model"] = "Qwen2.5-VL-32B text dims"
    line.update({"gpu_launches": launches, "prefill": prefill, "points": points,
                 "roofline": {"bound": "hbm", "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": roofs["decode_b8"],
                              "frac_b1": roofs["decode_b1"], "frac_b32": roofs["decode_b32"]},
                 "clocks": clock_record})
    print(json.dumps(line))
    return 0


def run_7b_trace(args):
    """A continuous-batching trace at the 7B sizes: 128 requests arrive at once, prompt lengths
    uniform in [128, 4096], output lengths uniform in [32, 512] (seed 3), at most 8,192 tokens a
    request, steps of at most 2,048 tokens.  The ideal time it is compared with: the prompts'
    flops at the sustained tensor peak plus, for every decode step, the weights once and the
    live requests' cache at the measured copy bandwidth.  The trace runs twice: the first pass is the
    warm-up (a server that has run for a while has captured its decode steps and grown its buffers;
    its wall time goes into ``trace.first_pass_wall_s``), the second is timed."""
    import numpy as np

    from qwen25vl_lite import LLM
    from qwen25vl_lite.engine import benchmark as B

    peaks = load_peaks()
    cfg = json.loads(json.dumps(CONFIG_7B))
    t = cfg["text_config"]
    layers = args.layers or t["num_hidden_layers"]
    full_layers, t["num_hidden_layers"] = t["num_hidden_layers"], layers
    n_requests, context = 128, 8192
    rng = np.random.default_rng(3)
    prompt_lens = rng.integers(128, 4097, size=n_requests)
    output_lens = rng.integers(32, 513, size=n_requests)
    pages = int(sum(-(-(p + o) // PAGE) for p, o in zip(prompt_lens, output_lens))) + n_requests
    llm = LLM(random_config=cfg, weights_seed=0, dtype="bfloat16", num_blocks=pages, block_size=PAGE, max_num_seqs=n_requests,
              max_num_batched_tokens=2048, max_model_len=context, cuda_graph=not args.no_cuda_graph)
    vocab = t["vocab_size"]
    warm = B.random_prompts(rng, vocab, [300] * 4)
    B.run_trace(llm.engine, warm, [8] * 4)                       # compile, allocate, touch every path once
    prompts = B.random_prompts(rng, vocab, prompt_lens)
    first = B.run_trace(llm.engine, prompts, output_lens)        # warm-up: the same trace once, untimed
    clocks = ClockSampler()
    clocks.start()
    launches0 = __import__("qwen25vl_lite.ops.kernels", fromlist=["x"]).launch_count()
    r = B.run_trace(llm.engine, prompts, output_lens)
    r["first_pass_wall_s"] = first["wall_s"]
    launches = __import__("qwen25vl_lite.ops.kernels", fromlist=["x"]).launch_count() - launches0
    clock_record = clocks.stop()
    flops = sum(B.prefill_flops(t, layers, int(p)) for p in prompt_lens)
    kvb = B.kv_bytes_per_token(t, layers)
    cache_bytes = sum(kvb * (int(p) * int(o) + int(o) * (int(o) - 1) // 2) for p, o in zip(prompt_lens, output_lens))
    decode_steps = int(output_lens.max())                        # at least this many steps read the weights
    ideal = flops / (peaks["bf16_tflops_sustained"] * 1e12) + (decode_steps * B.weight_bytes(t, layers) + cache_bytes) / (peaks["hbm_gbs"] * 1e9)
    t["num_hidden_layers"] = full_layers
    line = _base_line("generated tokens/s, Qwen2.5-VL-7B dims, continuous-batching trace of 128 requests",
                      r["generated_tokens_per_s"], args, 1e3 * r["wall_s"] / max(r["steps"], 1), cfg, layers, n_requests,
                      context, int(prompt_lens.mean()), peaks, {"chunk_budget": 2048})
    line["config"]["model"] = "Qwen2.5-VL-7B text dims"
    line["steps"], line["warmup"] = int(r["steps"]), int(first["steps"])
    line.update({"gpu_launches": launches, "trace": r,
                 "roofline": {"bound": "tensor (prompts) + hbm (decode steps)", "ideal_s": ideal, "wall_s": r["wall_s"],
                              "frac": ideal / r["wall_s"]},
                 "clocks": clock_record})
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
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32 times the true 32-bit path of the 3b configuration (fewer --layers advised)")
    ap.add_argument("--config", default="3b", choices=["3b", "7b-trace", "32b"],
                    help="3b: the headline line (default); 7b-trace, 32b: the other workloads, one line each")
    args = ap.parse_args(argv)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.config != "3b":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm measures the 3b configuration only"}))
            return 0
        return run_reference(args)
    return {"3b": run_ours, "7b-trace": run_7b_trace, "32b": run_32b}[args.config](args)


if __name__ == "__main__":
    sys.exit(main())
