"""Replay on the GPU against the plain implementation: every way of cutting and batching,
in 32-bit and in bfloat16, on the tiny configurations."""

import numpy as np
import pytest

import replay_util as ru
from tiny_models import BF16_TOLERANCE, TINY

pytestmark = pytest.mark.gpu

# float32: the logits of the tiny models are O(0.1-1); the engine's float32 path agrees with the
# float64 oracle to a few 1e-6.
# bfloat16: weights, activations and the cache are rounded to 8 bits of mantissa; the tolerance is
# three times the largest difference measured per configuration (``tiny_models.MEASURED_BF16_ERROR``).
# Set Q25VL_ERR_LOG=<file> to log the largest difference of every comparison.
TOL = {("float32", name): 1e-4 for name in TINY}
TOL.update({("bfloat16", name): tol for name, tol in BF16_TOLERANCE.items()})
LENGTHS = {"A": (5, 11, 17, 70), "B": (1, 9, 23, 40, 97), "C": (3, 31, 64, 130), "D": (3, 70, 150, 300),
           "E": (5, 40, 97, 200)}
# every pattern has a portion of 128 tokens or more: from there the tcgen05 product and (at head
# size 128) the tcgen05 attention run
PORTIONS = (7, 2, 160, 13, 3, 2, 21, 5)
# tiny-D, prompts of 2,000 tokens: the largest difference of any logit between attention with cut
# keys and with whole tiles was 1.4e-2 on a B200, as large as either's difference from the plain
# decoder: the two differ by the order of float sums, which moves some attention outputs by one
# bfloat16 step, and the layers behind amplify that like any other rounding.  Three times that is
# allowed; that no part of the keys is lost is what the kernel tests show, with one dominant key.
CUT_AGAINST_WHOLE = 4.2e-2


def _requests(name, seed=0):
    vocab = TINY[name][0]["text_config"]["vocab_size"]
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(LENGTHS[name])}


def _bf16_dir(tmp_path_factory, name):
    from tiny_models import make_model_dir

    return make_model_dir(tmp_path_factory.mktemp("bf16"), name, "bfloat16")


def _check(got, want, tol, what):
    import os
    worst = 0.0
    for rid, ref in want.items():
        err = np.abs(got[rid] - ref).max()
        worst = max(worst, float(err))
        assert err < tol, f"{what}: request {rid} differs from the plain decoder by {err:.3e} (tolerance {tol:.1e})"
    if os.environ.get("Q25VL_ERR_LOG"):
        with open(os.environ["Q25VL_ERR_LOG"], "a") as fh:
            fh.write(f"{what} tol={tol:.1e} worst={worst:.3e}\n")


@pytest.fixture(scope="module")
def cases(model_dirs, tmp_path_factory):
    """(name, dtype) -> (model folder, requests, oracle).  The bfloat16 oracle reads the
    bfloat16-rounded weights, so only the engine's own rounding is measured."""
    out = {}
    for name in TINY:
        reqs = _requests(name)
        out[name, "float32"] = (model_dirs[name], reqs, ru.oracle(model_dirs[name], reqs))
        d = _bf16_dir(tmp_path_factory, name)
        out[name, "bfloat16"] = (d, reqs, ru.oracle(d, reqs))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_whole(cases, name, dtype):
    folder, reqs, want = cases[name, dtype]
    steps = ru.whole(reqs)
    got, runner = ru.run_in_process(folder, dtype, steps, ru.max_live_tokens(steps), TINY[name][2])
    _check(got, want, TOL[dtype, name], f"whole {name} {dtype}")
    runner.cache.check([])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_last_32_one_by_one(cases, name, dtype):
    folder, reqs, want = cases[name, dtype]
    steps = ru.prefill_then_decode(reqs, 32)
    got, runner = ru.run_in_process(folder, dtype, steps, ru.max_live_tokens(steps), TINY[name][2])
    _check(got, want, TOL[dtype, name], f"decode {name} {dtype}")
    runner.cache.check([])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_portions_of_changing_size(cases, name, dtype):
    folder, reqs, want = cases[name, dtype]
    steps = ru.portions(reqs, PORTIONS)
    got, runner = ru.run_in_process(folder, dtype, steps, ru.max_live_tokens(steps), TINY[name][2])
    _check(got, want, TOL[dtype, name], f"portions {name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_mixed_with_page_reuse(cases, name, dtype):
    folder, _, _ = cases[name, dtype]
    vocab = TINY[name][0]["text_config"]["vocab_size"]
    rng = np.random.default_rng(11)
    reqs = {f"m{i}": rng.integers(0, vocab, size=int(n)).tolist() for i, n in enumerate(rng.integers(20, 120, size=9))}
    want = ru.oracle(folder, reqs)
    steps = ru.mixed(reqs, seed=3)
    assert max(len(s["entries"]) for s in steps) >= 3
    budget = ru.max_live_tokens(steps)
    got, runner = ru.run_in_process(folder, dtype, steps, budget, TINY[name][2])
    _check(got, want, TOL[dtype, name], f"mixed {name} {dtype}")
    # so few pages that they were used again: more pages were handed out than the pool has
    assert sum(-(-len(v) // 64) * 64 for v in reqs.values()) > budget
    runner.cache.check([])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["D", "B"])
def test_mixed_with_many_live_requests(cases, name, dtype):
    """Up to 40 live requests, so that steps decode 17 to 40 tokens at once beside portions of
    prompts (more rows than the weight-streaming products of a small decode step take), with
    pages used again."""
    folder, _, _ = cases[name, dtype]
    vocab = TINY[name][0]["text_config"]["vocab_size"]
    rng = np.random.default_rng(12)
    reqs = {f"n{i}": rng.integers(0, vocab, size=int(n)).tolist() for i, n in enumerate(rng.integers(40, 140, size=56))}
    want = ru.oracle(folder, reqs)
    steps = ru.mixed(reqs, seed=6, max_live=40, decode_tail=30, chosen_share=0.9, longest=40)
    decode_rows = [sum(1 for e in s["entries"] if len(e["tokens"]) == 1) for s in steps]
    assert max(decode_rows) >= 24 and any(17 <= n and len(s["entries"]) > n for n, s in zip(decode_rows, steps))
    budget = ru.max_live_tokens(steps)
    got, runner = ru.run_in_process(folder, dtype, steps, budget, TINY[name][2], max_requests=40)
    _check(got, want, TOL[dtype, name], f"many live {name} {dtype}")
    assert sum(-(-len(v) // 64) * 64 for v in reqs.values()) > budget
    runner.cache.check([])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_only_steps_of_17_to_40_requests(cases, dtype):
    """40 requests prefilled four at a time, then decoded together one token a step (steps of 40,
    then fewer as requests end): the decode step of a large batch as generation runs it, captured
    into CUDA graphs in bfloat16."""
    folder, _, _ = cases["D", dtype]
    rng = np.random.default_rng(13)
    reqs = {f"q{i}": rng.integers(0, 640, size=int(n)).tolist() for i, n in enumerate(rng.integers(30, 90, size=40))}
    want = ru.oracle(folder, reqs)
    ids = list(reqs)
    steps = []
    tail = {rid: int(rng.integers(4, 24)) for rid in ids}
    for i in range(0, len(ids), 4):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": reqs[rid][:len(reqs[rid]) - tail[rid]], "want": list(range(len(reqs[rid]) - tail[rid]))}
            for rid in ids[i:i + 4]]})
    at = {rid: len(reqs[rid]) - tail[rid] for rid in ids}
    while at:
        entries, end = [], []
        for rid in list(at):
            entries.append({"id": rid, "tokens": [reqs[rid][at[rid]]], "want": [0]})
            at[rid] += 1
            if at[rid] == len(reqs[rid]):
                end.append(rid)
                del at[rid]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    got, runner = ru.run_in_process(folder, dtype, steps, ru.max_live_tokens(steps), 16, max_requests=40)
    _check(got, want, TOL[dtype, "D"], f"decode-only 40 D {dtype}")
    if dtype == "bfloat16":
        assert runner.graph_replays > 0
    runner.cache.check([])


def test_float32_cut_independence(cases):
    """The 32-bit path sums in an order that depends only on a token's own position, so
    whole and cut replays agree far below the tolerance (bit for bit in the matrix
    products; attention and norms within a few ulp)."""
    folder, reqs, _ = cases["B", "float32"]
    a, _ = ru.run_in_process(folder, "float32", ru.whole(reqs), 512, 8)
    b, _ = ru.run_in_process(folder, "float32", ru.portions(reqs, (3, 2, 9)), 512, 8)
    for rid in reqs:
        assert np.abs(a[rid] - b[rid]).max() < 2e-6


def test_image_positions_through_replay(cases):
    """tiny-B's prompt with a 12-token image run (t1 x h3 x w4): explicit positions in the
    prompt portions, then plain tokens that resume at max + 1 through the stored offset."""
    from plain import decoder as plain

    folder, _, _ = cases["B", "float32"]
    rng = np.random.default_rng(4)
    ids = rng.integers(0, 512, size=46).tolist()
    pos40, delta = plain.prompt_positions(40, [(9, 1, 3, 4)])
    pos = np.concatenate([pos40] + [plain.decode_positions(n, delta) for n in range(40, 46)], axis=1)
    want = ru.oracle(folder, {"img": ids}, {"img": pos})
    steps, at = [], 0
    for n in (7, 7, 7, 7, 7, 5):                       # the prompt in portions of 7, positions given
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": "img", "tokens": ids[at:at + n], "want": list(range(n)), "positions": pos40[:, at:at + n].tolist()}]})
        at += n
    for i in range(40, 46):                            # then decoded tokens without positions
        steps.append({"step": len(steps), "end": [], "entries": [{"id": "img", "tokens": [ids[i]], "want": [0]}]})
    got, _ = ru.run_in_process(folder, "float32", steps, 64, 8)
    _check(got, want, 1e-4, "image positions")


def test_trace_run_program(cases, tmp_path):
    """The program itself: protocol lines, files, exit code."""
    folder, reqs, want = cases["A", "float32"]
    steps = ru.mixed(reqs, seed=5, max_live=3)
    got = ru.run_program(folder, "float32", steps, ru.max_live_tokens(steps), str(tmp_path / "out"))
    _check(got, want, 1e-4, "program")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(cases, dtype):
    """Two tokens in one step, then 254 tokens one by one; the logits of the first
    positions (sequences of length 1, 2, 3) are checked like all others."""
    folder, _, _ = cases["B", dtype]
    ids = np.random.default_rng(8).integers(0, 512, size=256).tolist()
    want = ru.oracle(folder, {"long": ids})
    steps = ru.prefill_then_decode({"long": ids}, tail=254)
    assert len(steps) == 255 and len(steps[0]["entries"][0]["tokens"]) == 2
    got, _ = ru.run_in_process(folder, dtype, steps, 256, 8)
    _check(got, want, TOL[dtype, "B"], f"long decoding B {dtype}")
    assert np.abs(got["long"][:3] - want["long"][:3]).max() < TOL[dtype, "B"]


@pytest.mark.parametrize("name", ["D", "E"])
def test_long_decoding_through_graphs_at_large_head_sizes(cases, name):
    """bfloat16, head size 128 (tiny-D) and 64 with a window shorter than two pages (tiny-E): 40
    tokens in one step, then 260 one by one, which the engine replays from CUDA graphs through the
    fused decode attention and the chained products; with the window, pages are given back and
    their block-table entries read as page 0 while the request goes on."""
    folder, _, _ = cases[name, "bfloat16"]
    vocab = TINY[name][0]["text_config"]["vocab_size"]
    ids = np.random.default_rng(9).integers(0, vocab, size=300).tolist()
    want = ru.oracle(folder, {"long": ids})
    steps = ru.prefill_then_decode({"long": ids}, tail=260)
    got, runner = ru.run_in_process(folder, "bfloat16", steps, 320, 16)
    assert runner.graph_replays >= 250
    _check(got, want, TOL["bfloat16", name], f"long decoding {name} bfloat16")
    runner.cache.check([])


def test_long_prompts_whose_keys_the_attention_plan_cuts(cases, monkeypatch):
    """bfloat16, head size 128: a prompt of 2,000 tokens in portions of 1,000, 600, 398 and 2, the
    third beside the whole prompt of a second request and the last beside its first decoded token.
    The steps have few row tiles with long walks, so the attention plan halves the keys between
    pairs of CTAs (first portion) and cuts them into parts for a merge kernel (the others); every
    logit against the plain decoder, and against the same replay with whole tiles."""
    import qwen25vl_lite.ops.attention as attention_ops

    folder, _, _ = cases["D", "bfloat16"]
    rng = np.random.default_rng(12)
    reqs = {"long": rng.integers(0, 640, size=2000).tolist(), "short": rng.integers(0, 640, size=301).tolist()}
    want = ru.oracle(folder, reqs)
    cuts = (0, 1000, 1600, 1998, 2000)
    steps = []
    for k in range(4):
        part = reqs["long"][cuts[k]:cuts[k + 1]]
        entries = [{"id": "long", "tokens": part, "want": list(range(len(part)))}]
        if k == 2:
            entries.append({"id": "short", "tokens": reqs["short"][:300], "want": list(range(300))})
        if k == 3:
            entries.insert(0, {"id": "short", "tokens": reqs["short"][300:], "want": [0]})
        steps.append({"step": k, "entries": entries, "end": ["long", "short"] if k == 3 else []})
    chosen = []
    planner = attention_ops.cut_keys

    def spy(tiles, windowed, places):
        work, merges, pairs = planner(tiles, windowed, places)
        chosen.append("pairs" if pairs else "parts" if merges else "whole")
        return work, merges, pairs

    monkeypatch.setattr(attention_ops, "cut_keys", spy)
    got, runner = ru.run_in_process(folder, "bfloat16", steps, 2432, 16)
    assert chosen == ["pairs", "parts", "parts", "parts"]
    _check(got, want, TOL["bfloat16", "D"], "long prompts with cut keys D bfloat16")
    runner.cache.check([])
    monkeypatch.setattr(attention_ops, "cut_keys", lambda tiles, windowed, places: planner(tiles, True, places))
    whole, _ = ru.run_in_process(folder, "bfloat16", steps, 2432, 16)
    worst = max(float(np.abs(got[r] - whole[r]).max()) for r in got)
    import os
    if os.environ.get("Q25VL_ERR_LOG"):
        with open(os.environ["Q25VL_ERR_LOG"], "a") as fh:
            fh.write(f"cut keys against whole tiles worst={worst:.3e}\n")
    assert worst < CUT_AGAINST_WHOLE
