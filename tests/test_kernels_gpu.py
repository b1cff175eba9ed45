"""Each CUDA kernel alone against a plain float64 computation of the same operation, at sizes
other than the engine's (odd widths, head sizes in steps of 16, odd head counts)."""

import numpy as np
import pytest
import torch

from plain import decoder as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def dev(a, dtype=None):
    t = torch.as_tensor(np.asarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def f64(t):
    return t.detach().to("cpu", torch.float64).numpy()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(dtype):
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(0)
    table = dev(rng.standard_normal((1000, 72)), dtype)
    ids = rng.integers(0, 1000, size=37)
    out = torch.empty((37, 72), dtype=torch.float32, device="cuda")
    kernels.embed_gather(table, dev(ids.astype(np.int32)), out)
    assert np.array_equal(f64(out), f64(table)[ids])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 2048 + 16])
def test_add_rmsnorm(dtype, hidden):
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(1)
    x0 = rng.standard_normal((9, hidden)) * 3
    delta = dev(rng.standard_normal((9, hidden)), dtype)
    w = dev(1 + 0.1 * rng.standard_normal(hidden), torch.float32)
    x = dev(x0, torch.float32)
    out = torch.empty((9, hidden), dtype=dtype, device="cuda")
    kernels.add_rmsnorm(x, delta, w, 1e-5, out)
    xs = f64(dev(x0, torch.float32)) + f64(delta)
    assert np.abs(f64(x) - xs).max() < 1e-6                  # the residual stream took the update
    ref = plain.rms_norm(xs, f64(w), 1e-5)
    assert np.abs(f64(out) - ref).max() < tol(dtype) * 4
    # rows: only some rows, x untouched, update still applied to the normalised value
    rows = np.asarray([7, 0, 3], dtype=np.int32)
    x2 = dev(x0, torch.float32)
    out2 = torch.empty((3, hidden), dtype=dtype, device="cuda")
    kernels.add_rmsnorm(x2, delta, w, 1e-5, out2, dev(rows))
    assert np.array_equal(f64(x2), f64(dev(x0, torch.float32)))
    assert np.abs(f64(out2) - ref[rows]).max() < tol(dtype) * 4
    # no update
    out3 = torch.empty((9, hidden), dtype=dtype, device="cuda")
    kernels.add_rmsnorm(x2, None, w, 1e-5, out3)
    assert np.abs(f64(out3) - plain.rms_norm(f64(x2), f64(w), 1e-5)).max() < tol(dtype) * 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    from qwen25vl_lite.ops import kernels
    gu = dev(np.random.default_rng(2).standard_normal((13, 2 * 136)) * 2, dtype)
    out = torch.empty((13, 136), dtype=dtype, device="cuda")
    kernels.silu_mul(gu, out)
    g, u = f64(gu)[:, :136], f64(gu)[:, 136:]
    assert np.abs(f64(out) - plain.silu(g) * u).max() < tol(dtype) * 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,section", [(5, 5, 48, (8, 8, 8)), (16, 2, 128, (16, 24, 24)), (3, 1, 16, (2, 3, 3))])
def test_rope_store(dtype, nq, nkv, d, section):
    from qwen25vl_lite.ops import kernels
    from qwen25vl_lite.parts.position import MRope
    rng = np.random.default_rng(3)
    n, page_size, pages = 21, 8, 7
    qkv0 = dev(rng.standard_normal((n, (nq + 2 * nkv) * d)), dtype)
    pos = rng.integers(0, 3000, size=(3, n))
    rope = MRope(d, 50000.0, section)
    rope.load({}, "cuda", dtype)
    slots = rng.permutation(pages * page_size)[:n].astype(np.int32)
    k_pages = torch.zeros((pages, nkv, page_size, d), dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    qkv = qkv0.clone()
    kernels.rope_store(qkv, dev(pos.astype(np.int32)), rope.inv_freq, rope.axis, k_pages, v_pages, dev(slots),
                       nq, nkv, d, page_size)
    cos, sin = plain.mrope_cos_sin(pos, d, 50000.0, section, np.float64)
    x = f64(qkv0).reshape(n, nq + 2 * nkv, d)
    q_ref = plain.apply_mrope(x[:, :nq], cos, sin)
    k_ref = plain.apply_mrope(x[:, nq:nq + nkv], cos, sin)
    # float32 angles at positions up to 3000 carry up to ~2e-4 rad of rounding
    t = 2e-3 if dtype == torch.float32 else 4e-2
    assert np.abs(f64(qkv).reshape(n, -1, d)[:, :nq] - q_ref).max() < t
    kp, vp = f64(k_pages), f64(v_pages)
    for i, s in enumerate(slots):
        assert np.abs(kp[s // page_size, :, s % page_size] - k_ref[i]).max() < t
        assert np.array_equal(vp[s // page_size, :, s % page_size], x[i, nq + nkv:])
    if dtype == torch.bfloat16:
        # the same with the step's angles handed in (what every layer after the first does): bit for bit
        angles = kernels.rope_angles(dev(pos.astype(np.int32)), rope.inv_freq, rope.axis)
        qkv_b, k_b, v_b = qkv0.clone(), torch.zeros_like(k_pages), torch.zeros_like(k_pages)
        kernels.rope_store(qkv_b, dev(pos.astype(np.int32)), rope.inv_freq, rope.axis, k_b, v_b, dev(slots),
                           nq, nkv, d, page_size, angles)
        assert torch.equal(qkv_b, qkv) and torch.equal(k_b, k_pages) and torch.equal(v_b, v_pages)
        with pytest.raises(kernels.KernelError):
            kernels.rope_store(qkv_b, dev(pos.astype(np.int32)), rope.inv_freq, rope.axis, k_b, v_b, dev(slots),
                               nq, nkv, d, page_size, angles[:, :-1])
    # slot -1 stores nothing; no positions = no rotation
    k2 = torch.zeros_like(k_pages)
    qkv = qkv0.clone()
    kernels.rope_store(qkv, None, None, None, k2, torch.zeros_like(k2), dev(np.full(n, -1, np.int32)), nq, nkv, d, page_size)
    assert float(k2.abs().max()) == 0 and torch.equal(qkv, qkv0)


def paged_case(rng, lens, q_lens, nq, nkv, d, page_size, dtype, n_pages=None, key_gain=None):
    """Random requests laid out in shuffled pages.  Returns tensors for the kernel and the
    dense per-request q, k, v for the oracle.  key_gain(L) gives a factor for the key at each position."""
    total_pages = sum(-(-L // page_size) for L in lens)
    n_pages = n_pages or total_pages + 3
    order = rng.permutation(n_pages)
    k_pages = torch.zeros((n_pages, nkv, page_size, d), dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    width = max(-(-L // page_size) for L in lens)
    table = np.zeros((len(lens), width), dtype=np.int32)
    dense, qs, token_seq, cu, start = [], [], [], [0], []
    at = 0
    for s, (L, ql) in enumerate(zip(lens, q_lens)):
        k = rng.standard_normal((L, nkv, d))
        if key_gain is not None:
            k = k * np.asarray(key_gain(L))[:, None, None]
        k = torch.as_tensor(k).to(dtype)
        v = torch.as_tensor(rng.standard_normal((L, nkv, d))).to(dtype)
        q = torch.as_tensor(rng.standard_normal((ql, nq, d))).to(dtype)
        npg = -(-L // page_size)
        table[s, :npg] = order[at:at + npg]
        at += npg
        pad = npg * page_size - L
        pages_of = torch.as_tensor(table[s, :npg].astype(np.int64), device="cuda")
        for src, dst in ((k, k_pages), (v, v_pages)):
            whole = torch.cat([src, torch.zeros((pad, nkv, d), dtype=dtype)]).cuda()
            dst[pages_of] = whole.view(npg, page_size, nkv, d).permute(0, 2, 1, 3)
        dense.append((q, k, v))
        qs.append(q)
        token_seq += [s] * ql
        cu.append(cu[-1] + ql)
        start.append(L - ql)
    n = cu[-1]
    qkv = torch.zeros((n, (nq + 2 * nkv) * d), dtype=dtype, device="cuda")
    qkv[:, :nq * d] = torch.cat(qs).reshape(n, nq * d).cuda()
    return dict(qkv=qkv, k_pages=k_pages, v_pages=v_pages, table=dev(table), token_seq=dev(np.asarray(token_seq, np.int32)),
                cu=dev(np.asarray(cu, np.int32)), start=dev(np.asarray(start, np.int32)), dense=dense)


def attention_oracle(dense, window):
    outs = []
    for q, k, v in dense:
        L, ql = k.shape[0], q.shape[0]
        qf = np.zeros((L, q.shape[1], q.shape[2]))
        qf[L - ql:] = f64(q)
        outs.append(plain.causal_attention(qf, f64(k), f64(v), window)[L - ql:])
    return np.concatenate(outs).reshape(sum(o.shape[0] for o in outs), -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [
    (4, 2, 16, 4, None), (6, 1, 32, 8, None), (5, 5, 48, 16, 24), (16, 2, 128, 16, None), (3, 3, 256, 16, 40),
    (8, 2, 64, 16, 33), (7, 7, 80, 32, None)])
def test_paged_attention_generic(dtype, nq, nkv, d, page_size, window):
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(5)
    lens, q_lens = [1, 37, 130, 64, 200], [1, 37, 2, 1, 45]     # a first token, a whole prompt, portions, a decode
    c = paged_case(rng, lens, q_lens, nq, nkv, d, page_size, dtype)
    out = torch.empty((c["qkv"].shape[0], nq * d), dtype=dtype, device="cuda")
    kernels.paged_attention_generic(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["token_seq"], c["cu"],
                                    c["start"], nq, nkv, d, page_size, window or 0, d ** -0.5)
    ref = attention_oracle(c["dense"], window)
    assert np.abs(f64(out) - ref).max() < tol(dtype) * 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_the_window_edge(dtype):
    """One key among hundreds gets a score that dominates the softmax: the output must be
    that key's value.  The key sits on the first slot of a page, on the last one, and just
    inside / just outside the window."""
    from qwen25vl_lite.ops import kernels
    nq, nkv, d, ps, L = 2, 1, 32, 16, 300
    for key, window, visible in [(0, None, True), (143, None, True), (144, None, True), (299, None, True),
                                 (300 - 50, 50, True), (300 - 51, 50, False)]:
        rng = np.random.default_rng(key)
        c = paged_case(rng, [L], [1], nq, nkv, d, ps, dtype)
        q, k, v = c["dense"][0]
        k = k.clone()
        k[key] = (q[0, 0] * 6).to(dtype)            # q . k ~ 6 |q|^2: e^(6*32/sqrt(32)) beats 299 others
        pg = int(c["table"][0, key // ps])
        c["k_pages"][pg, :, key % ps] = k[key].cuda()
        out = torch.empty((1, nq * d), dtype=dtype, device="cuda")
        kernels.paged_attention_generic(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["token_seq"], c["cu"],
                                        c["start"], nq, nkv, d, ps, window or 0, d ** -0.5)
        hit = np.abs(f64(out)[0, :d] - f64(v)[key, 0]).max() < 5e-2
        assert hit == visible, f"key {key} window {window}: found={hit}"
        ref = attention_oracle([(q, k, v)], window)
        assert np.abs(f64(out) - ref).max() < tol(dtype) * 2


@pytest.mark.parametrize("m,n,k", [(1, 100, 70), (37, 130, 257), (200, 64, 16), (16, 300, 2048)])
def test_gemm_f32(m, n, k):
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(6)
    a, w, b = dev(rng.standard_normal((m, k)), torch.float32), dev(rng.standard_normal((n, k)), torch.float32), \
        dev(rng.standard_normal(n), torch.float32)
    out = torch.empty((m, n), dtype=torch.float32, device="cuda")
    kernels.gemm_f32(a, w, b, out)
    ref = f64(a) @ f64(w).T + f64(b)
    assert np.abs(f64(out) - ref).max() < 1e-5 * np.sqrt(k) * 4
    # a row's result does not depend on the batch it is in: bit for bit
    out1 = torch.empty((1, n), dtype=torch.float32, device="cuda")
    kernels.gemm_f32(a[m // 2:m // 2 + 1].contiguous(), w, b, out1)
    assert torch.equal(out1[0], out[m // 2])
    out_nb = torch.empty((m, n), dtype=torch.float32, device="cuda")
    kernels.gemm_f32(a, w, None, out_nb)
    assert np.abs(f64(out_nb) - f64(a) @ f64(w).T).max() < 1e-5 * np.sqrt(k) * 4


def test_sample_rows_greedy_and_temperature():
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(7)
    logits = rng.standard_normal((6, 1031)).astype(np.float32)
    logits[1, 500] = logits[1, 77] = 9.0                     # a tie: the lower index wins
    lg = dev(logits)
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    kernels.sample_rows(lg, None, None, None, out)
    assert out.tolist() == [int(np.argmax(r)) for r in logits] and out[1].item() == 77
    temps = np.asarray([0.0, 0.8, 1.3, 0.0, 0.05, 2.0], dtype=np.float32)
    seeds = np.asarray([1, 2, 2**63 + 5, 4, 5, 6], dtype=np.uint64)
    index = np.asarray([0, 3, 1, 2, 9, 100], dtype=np.int32)
    kernels.sample_rows(lg, dev(temps), dev(seeds.view(np.int64)), dev(index), out)
    want = [plain.sample(logits[r], float(temps[r]), int(seeds[r]), int(index[r])) for r in range(6)]
    assert out.tolist() == want
    # the draws follow softmax(logits / T)
    small = np.tile(np.asarray([[2.0, 1.0, 0.0, -1.0]], dtype=np.float32), (4000, 1))
    o = torch.empty(4000, dtype=torch.int32, device="cuda")
    kernels.sample_rows(dev(small), dev(np.full(4000, 1.0, np.float32)), dev(np.full(4000, 7, np.int64)),
                        dev(np.arange(4000, dtype=np.int32)), o)
    freq = np.bincount(o.cpu().numpy(), minlength=4) / 4000
    p = np.exp(small[0]) / np.exp(small[0]).sum()
    assert np.abs(freq - p).max() < 0.03


def test_penalties_and_filters():
    from qwen25vl_lite.sampling import Sampler, SamplingParams, filter_scores
    rng = np.random.default_rng(8)
    logits = rng.standard_normal((3, 300)).astype(np.float32)
    prev = [[5, 5, 9], [], [1, 2, 3, 3, 3]]
    params = [SamplingParams(repetition_penalty=1.5, presence_penalty=0.2, frequency_penalty=0.1),
              SamplingParams(), SamplingParams(temperature=0.7, seed=3, frequency_penalty=0.5)]
    got = Sampler("cuda").sample(dev(logits), params, [0, 0, 3], [3, 0, 5], prev)
    want = []
    for r, p in enumerate(params):
        lg = plain.apply_penalties(logits[r], prev[r], p.repetition_penalty, p.presence_penalty, p.frequency_penalty)
        want.append(plain.sample(lg, p.temperature, 3, [3, 0, 5][r]))
    assert got == want
    for kw in (dict(top_k=5), dict(top_p=0.6), dict(min_p=0.1), dict(top_k=20, min_p=0.05, top_p=0.8)):
        full = {**dict(top_k=-1, min_p=0.0, top_p=1.0), **kw}
        s = filter_scores(dev(logits[0] / 0.7), full["top_k"], full["min_p"], full["top_p"]).cpu().numpy()
        ref = plain.filter_scores(logits[0] / np.float32(0.7), **full)
        assert np.array_equal(np.isinf(s), np.isinf(ref)), kw
        p = SamplingParams(temperature=0.7, seed=11, **kw)
        tok = Sampler("cuda").sample(dev(logits[:1]), [p], [11], [2], [[]])[0]
        assert tok == plain.sample(logits[0], 0.7, 11, 2, full["top_k"], full["min_p"], full["top_p"])


def run_mma_attention(c, lens, q_lens, nq, nkv, d, page_size, window, splits):
    """The tensor-core kernels as the engine calls them: one-token entries through the decode
    kernel, runs through the prefill kernel."""
    from qwen25vl_lite.ops import kernels
    G = nq // nkv
    out = torch.zeros((c["qkv"].shape[0], nq * d), dtype=torch.bfloat16, device="cuda")
    dec = [i for i, n in enumerate(q_lens) if n == 1 and G <= 16]
    tiles = [(i, t) for i, n in enumerate(q_lens) if i not in dec for t in range(-(-n * G // 64))]
    if dec:
        scratch = torch.full((len(dec) * nq * splits * (d + 2) + 7,), float("nan"), device="cuda") if splits > 1 else None
        kernels.attention_decode(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["cu"], c["start"],
                                 dev(np.asarray(dec, np.int32)), nq, nkv, d, page_size, window or 0, d ** -0.5, splits, scratch)
    if tiles:
        kernels.attention_prefill(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["cu"], c["start"],
                                  dev(np.asarray(tiles, np.int32)), nq, nkv, d, page_size, window or 0, d ** -0.5)
    return out


@pytest.mark.parametrize("splits", [1, 3, 16, 70])
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [
    (4, 2, 16, 4, None), (6, 1, 32, 8, None), (5, 5, 48, 16, 24), (16, 2, 128, 16, None), (8, 2, 64, 16, 33),
    (7, 7, 80, 32, None), (12, 4, 96, 16, 100), (4, 1, 112, 8, None), (32, 1, 64, 16, None)])
def test_attention_tensor_core_kernels(nq, nkv, d, page_size, window, splits):
    rng = np.random.default_rng(9)
    lens, q_lens = [1, 37, 130, 64, 200, 333, 31], [1, 37, 2, 1, 45, 1, 1]
    c = paged_case(rng, lens, q_lens, nq, nkv, d, page_size, torch.bfloat16)
    out = run_mma_attention(c, lens, q_lens, nq, nkv, d, page_size, window, splits)
    ref = attention_oracle(c["dense"], window)
    assert np.abs(f64(out) - ref).max() < 3e-2


def run_tcgen05_prefill(c, lens, q_lens, nq, nkv, d, page_size, window, shortest=None, fill=0.0):
    """The tcgen05 prefill kernel over every run of the case: whole row tiles, or (``shortest``: key
    tiles per part at least) with the keys of the long tiles cut into parts and merged, as the
    engine's plan cuts them, or (``shortest`` = "pairs") by clusters of two CTAs that halve the keys of
    the longer tiles."""
    from qwen25vl_lite.ops import kernels
    from qwen25vl_lite.ops.attention import pair_split, split_keys
    G = nq // nkv
    tiles = []
    for i, n in enumerate(q_lens):
        for t in range(-(-n * G // 128)):
            last = min((t * 128 + 127) // G, n - 1)
            tiles.append((i, t, (lens[i] - n + last) // 64 + 1))
    pairs = shortest == "pairs"
    if pairs:
        work, merges = pair_split(tiles), []
        assert window is None and any(code == 2 for _, _, code in work) and any(code == 1 for _, _, code in work)
    elif shortest is None:
        work, merges = sorted(tiles, key=lambda w: -w[2]), []
        work = [(i, t, 1) for i, t, _ in work]
    elif window:
        work, merges = [(i, t, 1) for i, t, _ in tiles], []          # keys behind a window are not cut
    else:
        work, merges = split_keys(tiles, shortest)
        assert merges
    out = torch.full((c["qkv"].shape[0], nq * d), fill, dtype=torch.bfloat16, device="cuda")
    scratch = torch.full((len(work) * nkv * 128 * (d + 2),), float("nan"), device="cuda") if merges else None
    kernels.attention_prefill_tcgen05(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["cu"], c["start"],
                                      dev(np.asarray(work, np.int32)), nq, nkv, d, page_size, window or 0, d ** -0.5,
                                      dev(np.asarray(merges, np.int32)) if merges else None, scratch, pairs)
    return out


@pytest.mark.parametrize("shortest", [None, 1, 3, "pairs"])
@pytest.mark.parametrize("nq,nkv,page_size,window", [(16, 2, 16, None), (8, 8, 4, None), (28, 4, 16, 150), (5, 1, 32, None), (40, 8, 8, 64)])
def test_attention_prefill_tcgen05(nq, nkv, page_size, window, shortest):
    """The tcgen05 prefill attention (scores, P and outputs in tensor memory, head size 128) against
    the oracle: runs that start inside a cached prefix, runs shorter and longer than a row tile,
    groups of 8, 1, 7 and 5 query heads, small and large pages, windows that cut the keys; with
    whole row tiles and with their keys cut into parts of one and of three key tiles at least (a
    part of one tile lies wholly behind some rows of its row tile, which then bring nothing)."""
    from qwen25vl_lite.ops import kernels
    if shortest == "pairs" and window:
        pytest.skip("keys behind a window are not cut")
    d = 128
    rng = np.random.default_rng(21)
    lens, q_lens = [300, 37, 130, 64, 517, 333, 9], [300, 37, 2, 17, 200, 70, 9]
    c = paged_case(rng, lens, q_lens, nq, nkv, d, page_size, torch.bfloat16)
    if window:
        # pages wholly behind the window of a run's first query were given back: their places in the
        # block table read as a live page of another request
        table = c["table"].cpu().numpy()
        for i, (L, ql) in enumerate(zip(lens, q_lens)):
            passed = max(0, L - ql + 1 - window) // page_size
            table[i, :passed] = table[(i + 1) % len(lens), 0]
        c["table"] = dev(table)
    assert kernels.attention_tcgen05_supports(torch.bfloat16, d, page_size, c["qkv"])
    out = run_tcgen05_prefill(c, lens, q_lens, nq, nkv, d, page_size, window, shortest)
    torch.cuda.synchronize()
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    ref = attention_oracle(c["dense"], window)
    assert np.abs(f64(out) - ref).max() < 3e-2
    assert not kernels.attention_tcgen05_supports(torch.bfloat16, 64, page_size)


@pytest.mark.parametrize("shortest", [None, 4, "pairs"])
def test_attention_prefill_tcgen05_long_runs_repeat_exactly(shortest):
    """Many key tiles per CTA, more CTAs than the GPU holds at once, and scores that keep growing
    along the keys, so that the rows in tensor memory are rescaled again and again: against the
    oracle, and eight launches give the same bits (the rows of a CTA, the thread that issues the
    products and the copies meet only at barriers; a missed one shows as a difference between runs).
    The same with the keys cut into parts of four key tiles at least, up to eight parts a tile."""
    from qwen25vl_lite.ops import kernels
    nq, nkv, d, page_size = 16, 2, 128, 16
    rng = np.random.default_rng(22)
    lens, q_lens = [1500, 1100, 300], [1000, 1100, 90]
    # keys grow with their position in every run: the running maximum of a row moves by far more
    # than the lazy threshold over its keys
    c = paged_case(rng, lens, q_lens, nq, nkv, d, page_size, torch.bfloat16, key_gain=lambda L: 1.0 + 5.0 * np.arange(L) / L)
    dense = c["dense"]
    outs = [run_tcgen05_prefill(c, lens, q_lens, nq, nkv, d, page_size, None, shortest, fill=3.0) for _ in range(8)]
    torch.cuda.synchronize()
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    ref = attention_oracle(dense, None)
    assert np.abs(f64(outs[0]) - ref).max() < 3e-2


@pytest.mark.parametrize("q_len", [1, 5])
def test_tensor_core_attention_finds_a_far_key_and_the_window_edge(q_len):
    """As for the general kernel: one dominant key on page edges, at both ends, and just inside /
    outside the window; through the decode kernel (one token, several splits) and the prefill
    kernel (a run of 5 whose last query is the one that matches)."""
    nq, nkv, d, ps, L = 8, 2, 128, 16, 700
    for key, window, visible in [(0, None, True), (15, None, True), (16, None, True), (351, None, True),
                                 (699, None, True), (700 - 60, 60, True), (700 - 61, 60, False)]:
        rng = np.random.default_rng(key)
        c = paged_case(rng, [L], [q_len], nq, nkv, d, ps, torch.bfloat16)
        q, k, v = c["dense"][0]
        k = k.clone()
        k[key, 0] = (q[-1, 0] * 3).to(torch.bfloat16)      # the last query's head 0 matches this key
        pg = int(c["table"][0, key // ps])
        c["k_pages"][pg, 0, key % ps] = k[key, 0].cuda()
        out = run_mma_attention(c, [L], [q_len], nq, nkv, d, ps, window, splits=5)
        hit = np.abs(f64(out)[-1, :d] - f64(v)[key, 0]).max() < 6e-2
        assert hit == visible, f"key {key} window {window}: found={hit}"
        ref = attention_oracle([(q, k, v)], window)
        assert np.abs(f64(out) - ref).max() < 3e-2


def test_tcgen05_prefill_attention_finds_a_far_key_and_the_window_edge():
    """The tcgen05 prefill kernel with one dominant key: on the edges of pages and of its 64-key
    tiles, at both ends of the keys, just inside and just outside the window; the matching query
    is the last of a run of 70 (so the key lies many tiles before the diagonal) and, in a second
    run of the batch, a query in the middle of a row tile.  Without a window also with the keys cut
    into parts of two key tiles: the key then lies in the first, a middle or the last part."""
    from qwen25vl_lite.ops import kernels
    nq, nkv, d, ps = 8, 2, 128, 16
    lens, q_lens = [700, 300], [70, 300]
    cases = [(0, None, True), (15, None, True), (16, None, True), (63, None, True), (64, None, True),
             (351, None, True), (629, None, True), (699, None, True), (700 - 60, 60, True), (700 - 61, 60, False)]
    for key, window, visible, shortest in [case + (None,) for case in cases] + [case + (p,) for case in cases if case[1] is None for p in (2, "pairs")]:
        rng = np.random.default_rng(key)
        c = paged_case(rng, lens, q_lens, nq, nkv, d, ps, torch.bfloat16)
        dense = [list(t) for t in c["dense"]]
        q, k, v = dense[0]
        k = k.clone()
        k[key, 0] = (q[-1, 0] * 3).to(torch.bfloat16)      # the last query's head 0 matches this key
        c["k_pages"][int(c["table"][0, key // ps]), 0, key % ps] = k[key, 0].cuda()
        dense[0][1] = k
        # second run: query 150 (of 300, head 5 = kv head 1) matches key 100, which every later query sees too
        q2, k2, v2 = dense[1]
        k2 = k2.clone()
        k2[100, 1] = (q2[150, 5] * 3).to(torch.bfloat16)
        c["k_pages"][int(c["table"][1, 100 // ps]), 1, 100 % ps] = k2[100, 1].cuda()
        dense[1][1] = k2
        out = run_tcgen05_prefill(c, lens, q_lens, nq, nkv, d, ps, window, shortest)
        torch.cuda.synchronize()
        assert int(kernels.error_flag("cuda:0")[0]) == 0
        o = f64(out)
        hit = np.abs(o[69, :d] - f64(v)[key, 0]).max() < 6e-2
        assert hit == visible, f"key {key} window {window} parts of {shortest}: found={hit}"
        in_window = window is None or 150 - 100 < window
        hit2 = np.abs(o[70 + 150, 5 * d:6 * d] - f64(v2)[100, 1]).max() < 6e-2
        assert hit2 == in_window
        ref = attention_oracle([tuple(t) for t in dense], window)
        assert np.abs(o - ref).max() < 3e-2


def test_decode_splits_heuristic():
    from qwen25vl_lite.ops.attention import decode_splits
    assert decode_splits(1, 2, 100) == 1                  # short context: nothing to split
    assert decode_splits(1, 2, 2048) == 8                 # 2048 keys / 256 per split
    assert decode_splits(8, 2, 4096) == 9                 # 144 CTAs: one per SM, no second wave
    assert decode_splits(64, 2, 8192) == 1                # 128 (entry, head) pairs already fill the GPU
    assert decode_splits(1, 1, 100000) == 64


@pytest.mark.parametrize("m", [1, 3, 5, 8])
@pytest.mark.parametrize("n,k", [(100, 64), (2560, 2048), (4752, 256), (2048, 11008), (48, 8192), (600, 3584), (2560, 4096),
                                 (5000, 6400), (512, 2208)])
def test_gemm_skinny(m, n, k):
    """The weight-streaming product (a chain of one) against float64 on the same bfloat16 operands,
    all epilogues, K that fits one slice and K cut into many (slices to different CTAs, slices one
    after the other, x whole with the CTA walking the slices), row counts that do not fill the
    8-wide MMA columns, N that is no multiple of 16."""
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(m * 1000 + n)
    x = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) * 0.05, torch.bfloat16)
    bias = dev(rng.standard_normal(n), torch.float32)
    ref = f64(x) @ f64(w).T
    scale = max(1.0, np.abs(ref).max())
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_skinny(x, w, None, out, kernels.SKINNY_STORE)
    assert np.abs(f64(out) - ref).max() / scale < 1e-2
    kernels.gemm_skinny(x, w, bias, out, kernels.SKINNY_BIAS)
    assert np.abs(f64(out) - (ref + f64(bias))).max() / scale < 1e-2
    out32 = torch.empty((m, n), dtype=torch.float32, device="cuda")
    kernels.gemm_skinny(x, w, None, out32, kernels.SKINNY_F32)
    assert np.abs(f64(out32) - ref).max() / scale < 1e-4          # float accumulation, float out
    if n % 16 == 0:
        act = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        kernels.gemm_skinny(x, w, None, act, kernels.SKINNY_SWIGLU)
        pairs = ref.reshape(m, n // 16, 2, 8)
        want = (plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, n // 2)
        assert np.abs(f64(act) - want).max() / max(1.0, np.abs(want).max()) < 1e-2
        # the activation kernel of the library path reads the same layout
        gu = dev(ref, torch.bfloat16)
        act2 = torch.empty_like(act)
        kernels.silu_mul(gu, act2, paired=True)
        pairs = f64(gu).reshape(m, n // 16, 2, 8)
        want2 = (plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, n // 2)
        assert np.abs(f64(act2) - want2).max() / max(1.0, np.abs(want2).max()) < 1e-2
    assert int(kernels.error_flag("cuda:0")[0]) == 0


def test_gemm_skinny_refuses_what_it_cannot_do():
    from qwen25vl_lite.ops import kernels
    x = torch.zeros((9, 64), dtype=torch.bfloat16, device="cuda")           # more rows than an MMA has batch columns
    w = torch.zeros((32, 64), dtype=torch.bfloat16, device="cuda")
    assert not kernels.gemm_skinny_supports(x, w)
    assert not kernels.gemm_skinny_supports(x[:4, :48], w[:, :48])          # K no multiple of 32
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny(x, w, None, torch.empty((9, 32), dtype=torch.bfloat16, device="cuda"), kernels.SKINNY_STORE)
    with pytest.raises(kernels.KernelError):                                # SwiGLU pairs need whole groups of 16 rows of w
        kernels.gemm_skinny(x[:4], w[:24], None, torch.empty((4, 12), dtype=torch.bfloat16, device="cuda"), kernels.SKINNY_SWIGLU)


def test_sample_rows_large_vocabulary():
    """A vocabulary that is scanned by several blocks per row: same winners as the plain sampler,
    ties across chunk borders still go to the lowest index."""
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(10)
    vocab = 151936
    logits = rng.standard_normal((3, vocab)).astype(np.float32)
    logits[0, 150000] = logits[0, 4095] = logits[0, 4096] = 20.0
    lg = dev(logits)
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    kernels.sample_rows(lg, None, None, None, out)
    assert out.tolist() == [4095, int(np.argmax(logits[1])), int(np.argmax(logits[2]))]
    temps = np.asarray([0.9, 0.0, 1.7], dtype=np.float32)
    kernels.sample_rows(lg, dev(temps), dev(np.asarray([3, 4, 5], dtype=np.int64)), dev(np.asarray([0, 1, 2], np.int32)), out)
    got = out.tolist()
    assert got[1] == int(np.argmax(logits[1]))
    # the plain sampler's per-token Python loop is slow at this size: check the winner is the
    # argmax of the same perturbed scores, computed here in bulk
    for r in (0, 2):
        g = np.asarray([0.0])
        key = plain._mix64((int([3, 4, 5][r]) * 0x9E3779B97F4A7C15 + r) & ((1 << 64) - 1))
        idx = np.arange(vocab, dtype=np.uint64)
        with np.errstate(over="ignore"):
            x = (np.uint64(key) + idx * np.uint64(0xD1342543DE82EF95))
            x ^= x >> np.uint64(30); x *= np.uint64(0xBF58476D1CE4E5B9)
            x ^= x >> np.uint64(27); x *= np.uint64(0x94D049BB133111EB)
            x ^= x >> np.uint64(31)
        u = ((x >> np.uint64(41)).astype(np.float64) + 0.5) / 8388608.0
        g = -np.log(-np.log(u.astype(np.float32), dtype=np.float32), dtype=np.float32)
        assert got[r] == int(np.argmax(logits[r] / temps[r] + g))


@pytest.mark.parametrize("m", [1, 4, 7, 8])
@pytest.mark.parametrize("n,k", [(2560, 2048), (96, 64), (4752, 256), (1024, 2560), (320, 5120), (64, 11008), (2560, 4096),
                                 (96, 6400)])
def test_gemm_skinny_with_norm_inside_and_residual_epilogue(m, n, k):
    """The product that normalises its float32 input inside the kernel, and the epilogue that
    adds into the float32 residual stream.  The shapes take every way of cutting K: one slice; x
    whole and the CTA walking two or four slices (2560, 5120); slices to different CTAs, two of
    them (4096 wide, 160 groups: too few for every CTA to walk), four (6400: x whole would not
    fit) and six (11008), whose shares the owners' warps add."""
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(m * 77 + k)
    x = dev(rng.standard_normal((m, k)) * 3, torch.float32)
    nw = dev(1 + 0.1 * rng.standard_normal(k), torch.float32)
    w = dev(rng.standard_normal((n, k)) * 0.05, torch.bfloat16)
    bias = dev(rng.standard_normal(n), torch.float32)
    assert kernels.gemm_skinny_norm_supports(x, w)
    h = plain.rms_norm(f64(x), f64(nw), 1e-5)
    ref = h @ f64(w).T
    scale = max(1.0, np.abs(ref).max())
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_skinny_norm(x, nw, 1e-5, w, bias, out, kernels.SKINNY_BIAS)
    assert np.abs(f64(out) - (ref + f64(bias))).max() / scale < 1.5e-2       # h is rounded to bfloat16 inside
    if n % 16 == 0:
        act = torch.empty((m, n // 2), dtype=torch.bfloat16, device="cuda")
        kernels.gemm_skinny_norm(x, nw, 1e-5, w, None, act, kernels.SKINNY_SWIGLU)
        pairs = ref.reshape(m, n // 16, 2, 8)
        want = (plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, n // 2)
        assert np.abs(f64(act) - want).max() / max(1.0, np.abs(want).max()) < 2e-2
    # residual epilogue: stream += a . w^T, in float32
    a = dev(rng.standard_normal((m, k)), torch.bfloat16)
    stream0 = rng.standard_normal((m, n)) * 5
    stream = dev(stream0, torch.float32)
    kernels.gemm_skinny(a, w, None, stream, kernels.SKINNY_RESIDUAL)
    want = f64(dev(stream0, torch.float32)) + f64(a) @ f64(w).T
    assert np.abs(f64(stream) - want).max() / max(1.0, np.abs(want).max()) < 1e-5
    assert int(kernels.error_flag("cuda:0")[0]) == 0


@pytest.mark.parametrize("sizes", [(1536, 4480, 2048, 3000), (2304, 5184, 2560, 3016), (3584, 4736, 4608, 2000)])
@pytest.mark.parametrize("m", [1, 3, 8])
def test_gemm_chain_runs_dependent_products_as_one_kernel(m, sizes):
    """A layer's worth of products, each reading what the one before wrote (norm inside, bias,
    SwiGLU pairs, residual additions, a K long enough to be cut into slices, float logits), gathered
    into one persistent kernel: the results of the products launched one by one (up to the order of
    the sums), right against float64, and the same to the bit when run again, with the barrier and
    the counters that the first run left.  The wider sizes have rows longer than a slice under the
    norms too (every CTA normalises its slice of a row whose statistics it reads whole) and a
    ring of more, shorter stages."""
    from qwen25vl_lite.ops import kernels
    if not kernels.chain_available():
        pytest.skip("the device cannot hold the chain kernel's whole grid")
    rng = np.random.default_rng(40 + m)
    hidden, inter, qkv_n, vocab = sizes
    x0 = rng.standard_normal((m, hidden)) * 2
    nw = [dev(1 + 0.1 * rng.standard_normal(hidden), torch.float32) for _ in range(3)]
    w_qkv = dev(rng.standard_normal((qkv_n, hidden)) * 0.03, torch.bfloat16)
    b_qkv = dev(rng.standard_normal(qkv_n), torch.float32)
    w_o = dev(rng.standard_normal((hidden, qkv_n)) * 0.03, torch.bfloat16)
    w_gu = dev(rng.standard_normal((2 * inter, hidden)) * 0.03, torch.bfloat16)
    w_down = dev(rng.standard_normal((hidden, inter)) * 0.03, torch.bfloat16)
    w_head = dev(rng.standard_normal((vocab, hidden)) * 0.03, torch.bfloat16)

    def layer():
        x = dev(x0, torch.float32)
        qkv = torch.empty((m, qkv_n), dtype=torch.bfloat16, device="cuda")
        act = torch.empty((m, inter), dtype=torch.bfloat16, device="cuda")
        logits = torch.empty((m, vocab), dtype=torch.float32, device="cuda")
        kernels.gemm_skinny_norm(x, nw[0], 1e-6, w_qkv, b_qkv, qkv, kernels.SKINNY_BIAS)
        kernels.gemm_skinny(qkv, w_o, None, x, kernels.SKINNY_RESIDUAL)
        kernels.gemm_skinny_norm(x, nw[1], 1e-6, w_gu, None, act, kernels.SKINNY_SWIGLU)
        kernels.gemm_skinny(act, w_down, None, x, kernels.SKINNY_RESIDUAL)
        kernels.gemm_skinny_norm(x, nw[2], 1e-6, w_head, None, logits, kernels.SKINNY_F32)
        return x, qkv, act, logits

    one_by_one = layer()
    launches = kernels.launch_count()
    runs = []
    for _ in range(2):
        assert kernels.chain_begin()
        try:
            runs.append(layer())
        finally:
            kernels.chain_end()
        torch.cuda.synchronize()
    assert kernels.launch_count() - launches == 2              # five products, one kernel, twice (one by one: five kernels)
    chained = runs[1]
    for a, b, c in zip(one_by_one, runs[0], runs[1]):
        assert torch.equal(b, c)
        assert (a.float() - b.float()).abs().max().item() <= 2e-2 * a.float().abs().max().item()
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    # against float64 on the same bfloat16 weights
    bf = lambda a: f64(dev(a, torch.bfloat16))
    h = bf(plain.rms_norm(x0, f64(nw[0]), 1e-6))
    qkv = bf(h @ f64(w_qkv).T + f64(b_qkv))
    x1 = x0 + qkv @ f64(w_o).T
    gu = bf(plain.rms_norm(x1, f64(nw[1]), 1e-6)) @ f64(w_gu).T
    pairs = gu.reshape(m, -1, 2, 8)
    act = bf((plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, inter))
    x2 = x1 + act @ f64(w_down).T
    logits = bf(plain.rms_norm(x2, f64(nw[2]), 1e-6)) @ f64(w_head).T
    assert np.abs(f64(chained[0]) - x2).max() / np.abs(x2).max() < 2e-2
    assert np.abs(f64(chained[3]) - logits).max() / np.abs(logits).max() < 3e-2


@pytest.mark.parametrize("hidden,inter", [(2304, 1152), (4096, 3072)])
@pytest.mark.parametrize("m", [2, 8])
def test_gemm_chain_with_x_whole_in_shared_memory(m, hidden, inter):
    """A layer's chain in the order a decode step runs it (o-projection, gate/up, down, the next qkv)
    at widths between 2048 and about 6000, where the host keeps x whole in shared memory and every
    CTA walks the K slices of its groups (at 2304: o and gate/up; at 4096: all four, the down
    projection over its 3072 too): against the products one by one, against float64, and twice."""
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(m + hidden)
    qkv_n = hidden + 512
    x0 = rng.standard_normal((m, hidden)) * 2
    attn = dev(rng.standard_normal((m, hidden)), torch.bfloat16)
    nw = [dev(1 + 0.1 * rng.standard_normal(hidden), torch.float32) for _ in range(2)]
    w_o = dev(rng.standard_normal((hidden, hidden)) * 0.02, torch.bfloat16)
    w_gu = dev(rng.standard_normal((2 * inter, hidden)) * 0.03, torch.bfloat16)
    w_down = dev(rng.standard_normal((hidden, inter)) * 0.03, torch.bfloat16)
    w_qkv = dev(rng.standard_normal((qkv_n, hidden)) * 0.03, torch.bfloat16)
    b_qkv = dev(rng.standard_normal(qkv_n), torch.float32)

    def layer():
        x = dev(x0, torch.float32)
        act = torch.empty((m, inter), dtype=torch.bfloat16, device="cuda")
        qkv = torch.empty((m, qkv_n), dtype=torch.bfloat16, device="cuda")
        kernels.gemm_skinny(attn, w_o, None, x, kernels.SKINNY_RESIDUAL)
        kernels.gemm_skinny_norm(x, nw[0], 1e-6, w_gu, None, act, kernels.SKINNY_SWIGLU)
        kernels.gemm_skinny(act, w_down, None, x, kernels.SKINNY_RESIDUAL)
        kernels.gemm_skinny_norm(x, nw[1], 1e-6, w_qkv, b_qkv, qkv, kernels.SKINNY_BIAS)
        return x, act, qkv

    one_by_one = layer()
    runs = []
    for _ in range(2):
        assert kernels.chain_begin()
        try:
            runs.append(layer())
        finally:
            kernels.chain_end()
        torch.cuda.synchronize()
    for a, b, c in zip(one_by_one, runs[0], runs[1]):
        assert torch.equal(b, c)
        assert (a.float() - b.float()).abs().max().item() <= 2e-2 * a.float().abs().max().item()
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    bf = lambda a: f64(dev(a, torch.bfloat16))
    x1 = x0 + f64(attn) @ f64(w_o).T
    gu = bf(plain.rms_norm(x1, f64(nw[0]), 1e-6)) @ f64(w_gu).T
    pairs = gu.reshape(m, -1, 2, 8)
    act = bf((plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, inter))
    x2 = x1 + act @ f64(w_down).T
    qkv = bf(plain.rms_norm(x2, f64(nw[1]), 1e-6)) @ f64(w_qkv).T + f64(b_qkv)
    x_got, act_got, qkv_got = runs[1]
    assert np.abs(f64(x_got) - x2).max() / np.abs(x2).max() < 2e-2
    assert np.abs(f64(act_got) - act).max() / max(1.0, np.abs(act).max()) < 2e-2
    assert np.abs(f64(qkv_got) - qkv).max() / np.abs(qkv).max() < 3e-2


def test_gemm_skinny_norm_refuses_more_rows_than_it_has_columns():
    from qwen25vl_lite.ops import kernels
    x = torch.zeros((9, 2048), dtype=torch.float32, device="cuda")
    w = torch.zeros((32, 2048), dtype=torch.bfloat16, device="cuda")
    assert not kernels.gemm_skinny_norm_supports(x, w)
    with pytest.raises(kernels.KernelError):
        kernels.gemm_skinny_norm(x, torch.ones(2048, device="cuda"), 1e-6, w, None,
                                 torch.empty((9, 32), dtype=torch.bfloat16, device="cuda"), kernels.SKINNY_STORE)


@pytest.mark.parametrize("dense", [False, True])
@pytest.mark.parametrize("splits", [1, 2, 5, 19])
@pytest.mark.parametrize("nq,nkv,d,section,page_size,window", [
    (16, 2, 128, (16, 24, 24), 16, None), (6, 1, 32, (4, 6, 6), 8, None), (8, 2, 64, (8, 12, 12), 16, 70),
    (12, 4, 96, (16, 16, 16), 4, None), (3, 3, 64, (10, 11, 11), 32, 33)])
def test_attention_decode_fused(nq, nkv, d, section, page_size, window, splits, dense):
    """The one-kernel decode step of attention: rotary encoding of q and the new k inside the
    kernel, the new k and v written to their page slot, merge of the splits; with the list of items
    and without it (``dense``: the items are 0 .. n-1 here)."""
    from qwen25vl_lite.ops import kernels
    from qwen25vl_lite.parts.position import MRope
    rng = np.random.default_rng(12)
    lens = [1, 33, 130, 64, 290, 31, 600]
    c = paged_case(rng, lens, [1] * len(lens), nq, nkv, d, page_size, torch.bfloat16)
    n = len(lens)
    theta = 10000.0
    rope = MRope(d, theta, section)
    rope.load({}, "cuda", torch.bfloat16)
    positions = rng.integers(0, 2000, size=(3, n))
    cos, sin = plain.mrope_cos_sin(positions, d, theta, section, np.float64)
    k_raw = torch.as_tensor(rng.standard_normal((n, nkv, d))).to(torch.bfloat16)
    v_raw = torch.as_tensor(rng.standard_normal((n, nkv, d))).to(torch.bfloat16)
    qkv = c["qkv"].clone()
    qkv[:, nq * d:(nq + nkv) * d] = k_raw.reshape(n, -1).cuda()
    qkv[:, (nq + nkv) * d:] = v_raw.reshape(n, -1).cuda()
    q_raw = f64(qkv[:, :nq * d]).reshape(n, nq, d)
    q_rot = plain.apply_mrope(q_raw, cos, sin)
    k_rot = plain.apply_mrope(f64(k_raw), cos, sin)
    table = c["table"].cpu().numpy()
    if window:
        # pages that a window has passed are given back while the request goes on, and their places
        # in its block table read as some page or other: here as a live page of another request
        for i, L in enumerate(lens):
            passed = max(0, L - window) // page_size
            table[i, :passed] = table[(i + 1) % len(lens), 0]
        c["table"] = dev(table)
    slots, dense = [], []
    for i, L in enumerate(lens):
        page = int(table[i, (L - 1) // page_size])
        slots.append(page * page_size + (L - 1) % page_size)
        c["k_pages"][page, :, (L - 1) % page_size] = 0          # the new token's slot is still empty
        c["v_pages"][page, :, (L - 1) % page_size] = 0
        _, k, v = c["dense"][i]
        k, v = k.clone(), v.clone()
        k[L - 1] = torch.as_tensor(k_rot[i]).to(torch.bfloat16)
        v[L - 1] = v_raw[i]
        dense.append((torch.as_tensor(q_rot[i:i + 1]).to(torch.bfloat16), k, v))
    out = torch.zeros((n, nq * d), dtype=torch.bfloat16, device="cuda")
    qkv_before = qkv.clone()
    scratch = torch.full((n * nq * splits * (d + 2),), float("nan"), device="cuda")
    for _ in range(2):                                           # twice: the split counters must come back to zero
        out.zero_()
        kernels.attention_decode_fused(qkv, out, c["k_pages"], c["v_pages"], c["table"], c["cu"], c["start"],
                                       dev(np.arange(n, dtype=np.int32)), nq, nkv, d, page_size, window or 0, d ** -0.5,
                                       splits, dev(positions.astype(np.int32)), rope.inv_freq, rope.axis,
                                       dev(np.asarray(slots, np.int32)), scratch if splits > 1 else None, dense=dense)
    assert torch.equal(qkv, qkv_before)                          # the projections are left as they were
    ref = attention_oracle(dense, window)
    assert np.abs(f64(out) - ref).max() < 4e-2
    kp, vp = f64(c["k_pages"]), f64(c["v_pages"])
    for i, s in enumerate(slots):                                # the new key and value are in the pages now
        assert np.abs(kp[s // page_size, :, s % page_size] - k_rot[i]).max() < 4e-2
        assert np.array_equal(vp[s // page_size, :, s % page_size], f64(v_raw[i]))


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (2048, 2560, 2048), (300, 1000, 512), (17, 4752, 256), (1000, 512, 11008),
                                   (129, 272, 72), (40, 2048, 2048), (64, 2560, 2048), (17, 2048, 11008), (100, 22016, 2048),
                                   (33, 144, 4160), (127, 151936, 256), (2048, 9700, 128), (700, 5000, 320),
                                   (32, 55296, 128), (98, 37888, 64), (20, 33000, 96)])
def test_gemm_tcgen05(m, n, k):
    """The tcgen05 / TMA product against float64 on the same bfloat16 operands: whole tiles, ragged
    edges in M, N and K, many K blocks (the ring of stages wraps), every epilogue.  Up to 128 rows
    the width of a feature tile follows from the number of features (64 to 256 in steps of 32:
    160 for 22,016 features, 192 for 55,296, 224 for 33,000)."""
    from qwen25vl_lite.ops import kernels
    rng = np.random.default_rng(m + n + k)
    x = dev(rng.standard_normal((m, k)), torch.bfloat16)
    w = dev(rng.standard_normal((n, k)) * 0.05, torch.bfloat16)
    bias = dev(rng.standard_normal(n), torch.float32)
    ref = f64(x) @ f64(w).T
    scale = max(1.0, np.abs(ref).max())
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05(x, w, None, out, kernels.SKINNY_STORE)
    assert np.abs(f64(out) - ref).max() / scale < 1e-2
    kernels.gemm_tcgen05(x, w, bias, out, kernels.SKINNY_BIAS)
    assert np.abs(f64(out) - (ref + f64(bias))).max() / scale < 1e-2
    out32 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    kernels.gemm_tcgen05(x, w, None, out32, kernels.SKINNY_F32)
    assert np.abs(f64(out32) - ref).max() / scale < 1e-4
    stream0 = rng.standard_normal((m, n)) * 5
    stream = dev(stream0, torch.float32)
    kernels.gemm_tcgen05(x, w, None, stream, kernels.SKINNY_RESIDUAL)
    want = f64(dev(stream0, torch.float32)) + ref
    assert np.abs(f64(stream) - want).max() / max(1.0, np.abs(want).max()) < 1e-4
    if n % 16 == 0:
        act = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        kernels.gemm_tcgen05(x, w, None, act, kernels.SKINNY_SWIGLU)
        pairs = ref.reshape(m, n // 16, 2, 8)
        want = (plain.silu(pairs[:, :, 0]) * pairs[:, :, 1]).reshape(m, n // 2)
        assert np.abs(f64(act) - want).max() / max(1.0, np.abs(want).max()) < 1e-2
    assert int(kernels.error_flag("cuda:0")[0]) == 0
    again = torch.empty_like(out32)
    kernels.gemm_tcgen05(x, w, None, again, kernels.SKINNY_F32)
    assert torch.equal(again, out32)
