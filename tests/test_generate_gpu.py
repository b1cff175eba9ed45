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


def test_preemption_recomputes_a_request_with_an_image_run_exactly(model_dirs):
    """tiny-B, pages of 8, a pool too small for both requests: the newer one, whose prompt carries
    a 12-token image run (grid t1 x h3 x w4, so its text resumes at a position offset of its own),
    is preempted after it has generated tokens and comes back with prompt + generated to
    recompute.  Its tokens must be those of the plain decoder run without any cache: positions of
    the recomputed generated tokens continue from the image run's offset
    (src/qwen25vl_lite/rope.py:235-247), and its sampling keys go on where they stopped."""
    from qwen25vl_lite import LLM, SamplingParams
    text, image = _prompts("B", (23, 40), 26)
    spans = [(9, 1, 3, 4)]
    params = SamplingParams(temperature=0.8, seed=3, max_tokens=30, ignore_eos=True)
    llm = LLM(model_dirs["B"], dtype="float32", num_blocks=13, block_size=8, max_num_seqs=2)
    first = llm.engine.add_request(text, params)
    second = llm.engine.add_request(image, params, image_spans=spans)
    generated_when_preempted = None
    while llm.engine.has_work():
        llm.engine.step()
        for seq in llm.engine.waiting:
            if seq.seq_id == second and seq.preemptions and generated_when_preempted is None:
                generated_when_preempted = len(seq.output_token_ids)
    outs = {o.seq_id: o for o in llm.engine.finished}
    assert outs[second].metrics["preemptions"] >= 1 and generated_when_preempted and generated_when_preempted >= 2
    cfg, w = plain.load_model_dir(model_dirs["B"], np.float64)
    pos, delta = plain.prompt_positions(len(image), spans)
    assert delta != 0
    assert outs[second].output_token_ids == plain.greedy_generate(cfg, w, image, 30, pos, delta, temperature=0.8, seed=3)
    assert outs[first].output_token_ids == plain.greedy_generate(cfg, w, text, 30, temperature=0.8, seed=3)
    assert llm.runner.cache.pages_in_use() == [0]


def test_abort_while_the_next_step_is_already_on_the_device(model_dirs):
    """The engine launches the next decode step before it returns from ``step``; a request
    aborted at that moment draws nothing from that step, its pages go back at once (the step's
    writes into them are ordered before any later use), and the others go on exactly."""
    from qwen25vl_lite import LLM, SamplingParams
    prompts = _prompts("A", (5, 11, 17), 27)
    llm = LLM(model_dirs["A"], dtype="float32", num_blocks=64, block_size=4, max_num_seqs=4)
    ids = [llm.engine.add_request(p, SamplingParams(max_tokens=12, ignore_eos=True)) for p in prompts]
    aborted_with = None
    for _ in range(200):
        if not llm.engine.has_work():
            break
        llm.engine.step()
        if aborted_with is None and llm.engine._launched is not None and len(llm.engine.running) == 3 \
                and len(llm.engine.running[1].output_token_ids) >= 3:
            victim = next(s for s in llm.engine.running if s.seq_id == ids[1])
            aborted_with = list(victim.output_token_ids)
            assert llm.engine.abort(ids[1])
    assert aborted_with is not None, "no step was ever launched ahead"
    assert not llm.engine.has_work()
    outs = {o.seq_id: o for o in llm.engine.finished}
    assert ids[1] not in outs
    cfg, w = plain.load_model_dir(model_dirs["A"], np.float64)
    for i in (0, 2):
        assert outs[ids[i]].output_token_ids == plain.greedy_generate(cfg, w, prompts[i], 12)
    assert aborted_with == plain.greedy_generate(cfg, w, prompts[1], 12)[:len(aborted_with)]
    assert llm.runner.cache.pages_in_use() == [0]
    llm.runner.cache.check([])


def test_without_chunked_prefill_on_the_device(model_dirs):
    """``enable_chunked_prefill=False`` (the reference's --no-chunked-prefill,
    src/qwen25vl_lite/engine.py:649-654,673-678): a prompt runs whole or waits for a step with
    room for all of it; the tokens are the plain decoder's."""
    from qwen25vl_lite import LLM, SamplingParams
    prompts = _prompts("B", (9, 30, 17, 26), 28)
    llm = LLM(model_dirs["B"], dtype="float32", num_blocks=64, block_size=8, max_num_seqs=4, max_num_batched_tokens=32,
              enable_chunked_prefill=False)
    fed = []
    step = llm.runner.step
    llm.runner.step = lambda entries: (fed.append([len(e.tokens) for e in entries]), step(entries))[1]
    outs = llm.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))
    whole = {9, 30, 17, 26}
    assert all(n == 1 or n in whole for f in fed for n in f) and all(sum(f) <= 32 for f in fed)
    cfg, w = plain.load_model_dir(model_dirs["B"], np.float64)
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 5)


@pytest.mark.parametrize("name,temperature", [("B", 0.7), ("D", 0.0), ("D", 0.9), ("E", 0.0)])
def test_bfloat16_generation_agrees_with_the_plain_decoder(name, temperature, tmp_path):
    """bfloat16 generation (prompt portions, then decode steps replayed from CUDA graphs) against
    the plain decoder on the same bfloat16-rounded weights: every generated token must be the plain
    decoder's own choice at its place, or score within bfloat16 rounding of it; and a second run
    with the same seed repeats the tokens."""
    from qwen25vl_lite import LLM, SamplingParams
    from tiny_models import BF16_TOLERANCE, make_model_dir
    folder = make_model_dir(tmp_path, name, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", num_blocks=48, block_size=16, max_num_batched_tokens=24)
    prompts = _prompts(name, (12, 33, 70), 24)
    params = SamplingParams(max_tokens=24, temperature=temperature, seed=5, ignore_eos=True)
    outs = llm.generate(prompts, params)
    assert [len(o.output_token_ids) for o in outs] == [24, 24, 24]
    assert llm.runner.graph_replays > 0
    cfg, w = plain.load_model_dir(folder, np.float64)
    tol = BF16_TOLERANCE[name]
    for p, o in zip(prompts, outs):
        margins = plain.generation_margins(cfg, w, p, o.output_token_ids, temperature=temperature, seed=5)
        bound = 2 * tol / temperature if temperature > 0 else 2 * tol       # both scores may be off by tol (/ T)
        assert max(margins) <= bound, f"prompt of {len(p)} tokens: margins {margins}"
        assert sum(m == 0.0 for m in margins) >= 16, f"prompt of {len(p)} tokens: margins {margins}"
    again = llm.generate(prompts, params)
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
        got = [runner.step([StepEntry(r, [int(rng.integers(0, 3000))], [0]) for r in reqs]).float().cpu().numpy() for _ in range(5)]
        assert runner.graph_replays == (3 if graphs else 0)          # a shape is captured when it comes for the third time
        assert int(kernels.error_flag("cuda:0")[0]) == 0
        outs.append(np.stack(got))
        del llm, runner
        torch.cuda.empty_cache()
    graph, eager = outs
    assert np.abs(graph - eager).max() <= 2e-2 * np.abs(eager).max()


def test_a_kernel_that_gave_up_a_wait_fails_the_step_and_only_that_step(model_dirs):
    """Kernels with bounded waits report a wait that ran out through a flag on the device.  The flag
    is set here by hand (no kernel is made to hang): the generation whose step carried it must
    raise before any token of that step is accepted, the trace session likewise before it hands
    logits out, and the next call works, because raising clears the flag."""
    from qwen25vl_lite import LLM, SamplingParams
    from qwen25vl_lite.engine.trace import TraceSession
    from qwen25vl_lite.ops import kernels
    llm = LLM(model_dirs["A"], dtype="float32", num_blocks=32, block_size=4, max_num_seqs=2)
    prompt = _prompts("A", (9,), 29)
    params = SamplingParams(max_tokens=3, ignore_eos=True)
    want = llm.generate(prompt, params)[0].output_token_ids
    kernels.error_flag("cuda:0").fill_(14)
    with pytest.raises(kernels.KernelError, match="code 14"):
        llm.generate(prompt, params)
    for seq in list(llm.engine.running) + list(llm.engine.waiting):
        llm.engine.abort(seq.seq_id)
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    assert llm.generate(prompt, params)[0].output_token_ids == want
    session = TraceSession(llm.runner, None)
    kernels.error_flag("cuda:0").fill_(3)
    with pytest.raises(kernels.KernelError, match="code 3"):
        session.run_step({"step": 0, "entries": [{"id": "x", "tokens": prompt[0], "want": [8]}], "end": ["x"]})
    assert int(kernels.error_flag("cuda:0")[0]) == 0


def test_generate_with_random_weights_from_the_command_line(model_dirs):
    """``generate --random-weights --weights-seed S``: --model only has to hold a config.json."""
    cmd = [sys.executable, "-m", "qwen25vl_lite.cli", "generate", "--model", os.path.join(model_dirs["A"], "config.json"),
           "--random-weights", "--weights-seed", "7", "--dtype", "float32", "--block-size", "4", "--num-blocks", "32",
           "--max-tokens", "4", "--ignore-eos", "--prompt-token-ids", "5,6,7"]
    runs = [subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300) for _ in range(2)]
    assert all(r.returncode == 0 for r in runs), runs[0].stderr
    ids = [eval(r.stdout.strip().splitlines()[-1]) for r in runs]
    assert ids[0] == ids[1] and len(ids[0]) == 4 and all(0 <= t < 256 for t in ids[0])
    cmd[cmd.index("7")] = "8"
    other = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert other.returncode == 0 and len(eval(other.stdout.strip().splitlines()[-1])) == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padded_batches_and_requests_that_end_by_their_token(model_dirs, tmp_path, dtype):
    """11 requests decode together: captured steps run them as 16 rows, the five added rows on a
    page and slot of their own.  One token in 16 ends a request, so requests end by their
    token while the next step is packed ahead, and that step (with its page) is dropped; the batch
    shrinks through 10 and 9 rows (still 16) into the chained products' 8.  Every page and slot
    comes back; in 32-bit, whose sums do not depend on the batch, every request's tokens are those
    of the same request generated alone."""
    from qwen25vl_lite import LLM, SamplingParams
    from tiny_models import make_model_dir
    folder = model_dirs["B"] if dtype == "float32" else make_model_dir(tmp_path, "B", "bfloat16")
    prompts = _prompts("B", (9, 23, 5, 40, 17, 3, 31, 12, 26, 7, 19), 31)
    stops = tuple(range(0, 512, 16))
    params = SamplingParams(max_tokens=40, temperature=0.9, seed=5, stop_token_ids=stops)
    llm = LLM(folder, dtype=dtype, num_blocks=96, block_size=8, max_num_seqs=12)
    outs = llm.generate(prompts, params)
    assert llm.runner.graph_replays > 0
    assert "stop" in [o.finish_reason for o in outs]
    assert llm.runner.cache.pages_in_use() == [0] and llm.runner.cache.free_slots == 12
    llm.runner.cache.check([])
    if dtype == "float32":
        alone = LLM(folder, dtype=dtype, num_blocks=96, block_size=8, max_num_seqs=12, cuda_graph=False)
        for p, o in zip(prompts, outs):
            ref = alone.generate([p], params)[0]
            assert ref.output_token_ids == o.output_token_ids and ref.finish_reason == o.finish_reason
