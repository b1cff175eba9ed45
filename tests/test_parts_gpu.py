"""Each part alone, built from its own parameters, against the plain function of the same
part.  A shell stands in for the model so that the real step function builds the step's
context (block tables, slots, positions) around the part."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import decoder as plain
from qwen25vl_lite.engine.runner import ModelRunner, StepEntry
from qwen25vl_lite.models.decoder import StopRuntime
from qwen25vl_lite.cache import StopNeeds
from qwen25vl_lite import parts

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def f64(t):
    return t.detach().to("cpu", torch.float64).numpy()


def err(got, ref):
    """Largest difference relative to the size of the values compared."""
    return np.abs(f64(got) - ref).max() / max(1.0, np.abs(ref).max())


def rand(rng, shape, init="matrix", scale=0.3):
    t = rng.standard_normal(shape) * scale
    return torch.as_tensor(t + (1.0 if init == "norm" else 0.0), dtype=torch.float32)


def load_random(part, rng, dtype, **kw):
    tensors = {ts.name: rand(rng, ts.shape, ts.init) for ts in part.tensor_specs()}
    if dtype == torch.bfloat16:      # the oracle must see the weights the part computes with
        tensors = {k: (v.to(torch.bfloat16).float() if v.dim() > 1 else v) for k, v in tensors.items()}
    part.load(tensors, "cuda", dtype, **kw)
    return {k: v.double().numpy() for k, v in tensors.items()}


class Shell:
    """What the step function needs of a model, around one callable."""

    def __init__(self, fn, position, dtype, needs=(), vocab=1 << 20, planning=()):
        self.fn, self.position, self.dtype, self.device = fn, position, dtype, torch.device("cuda")
        self._planning = list(planning)
        self.stops = [StopRuntime(i, 0, n.cache_of, n.cache_of is None) for i, n in enumerate(needs)]
        self._needs = list(needs)
        self.head = SimpleNamespace(vocab_size=vocab)

    def stop_needs(self):
        return self._needs

    def planning_parts(self):
        return self._planning

    def forward(self, ctx):
        return self.fn(ctx)


def mrope(d, section, theta=10000.0, dtype=torch.float32):
    p = parts.POSITION_ENCODINGS["mrope"](head_dim=d, theta=theta, sections=section)
    p.load({}, "cuda", dtype)
    return p


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    rng = np.random.default_rng(0)
    norm = parts.NORMS["rmsnorm"](dim=200, eps=3e-5)
    w = load_random(norm, rng, dtype)
    x0 = rand(rng, (11, 200), scale=2.0)
    x = x0.clone().cuda()
    ctx = SimpleNamespace(dtype=dtype)
    delta = rand(rng, (11, 200)).to(dtype).cuda()
    h = norm.forward(ctx, x, delta)
    assert h.dtype == dtype
    assert np.abs(f64(h) - plain.rms_norm(f64(x0) + f64(delta), w["weight"], 3e-5)).max() < tol(dtype) * 4
    assert np.abs(f64(x) - (f64(x0) + f64(delta))).max() < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    rng = np.random.default_rng(1)
    ffn = parts.FEED_FORWARDS["swiglu"](hidden_size=72, intermediate_size=136)
    w = load_random(ffn, rng, dtype)
    h = rand(rng, (9, 72)).to(dtype)
    out = ffn.forward(SimpleNamespace(dtype=dtype), h.cuda())
    ref = plain.swiglu_mlp(f64(h), {"gate_proj.weight": w["gate_proj.weight"], "up_proj.weight": w["up_proj.weight"],
                                    "down_proj.weight": w["down_proj.weight"]}, "")
    assert err(out, ref) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    rng = np.random.default_rng(2)
    emb = parts.EMBEDDINGS["token_embedding"](vocab_size=301, hidden_size=40)
    we = load_random(emb, rng, dtype)
    ids = rng.integers(0, 301, size=13)
    ctx = SimpleNamespace(dtype=dtype, n_tokens=13, token_ids=torch.as_tensor(ids.astype(np.int32)).cuda())
    x = emb.forward(ctx)
    assert x.dtype == torch.float32 and np.array_equal(f64(x), we["weight"][ids])
    tied = parts.HEADS["linear_head"](vocab_size=301, hidden_size=40, tied=True)
    tied.receive({"embed_tokens.weight": emb.weight})
    tied.load({}, "cuda", dtype)
    h = rand(rng, (5, 40)).to(dtype)
    logits = tied.forward(ctx, h.cuda())
    assert logits.dtype == torch.float32 and np.abs(f64(logits) - f64(h) @ we["weight"].T).max() < tol(dtype)
    own = parts.HEADS["linear_head"](vocab_size=301, hidden_size=40, tied=False)
    wh = load_random(own, rng, dtype)
    assert np.abs(f64(own.forward(ctx, h.cuda())) - f64(h) @ wh["weight"].T).max() < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,section,window", [(4, 2, 16, (2, 3, 3), None), (6, 1, 32, (4, 6, 6), 9), (5, 5, 48, (8, 8, 8), None)])
def test_attention_part_in_portions(dtype, nq, nkv, d, section, window):
    """The mixer alone, a request fed in three portions beside another request; positions
    with three different axes."""
    rng = np.random.default_rng(3)
    hidden = nq * d + 8
    rope = mrope(d, section, 10000.0, dtype)
    attn = parts.MIXERS["gqa_attention"](hidden_size=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=d,
                                         position=rope, window=window)
    w = load_random(attn, rng, dtype)
    inputs = {}
    shell = Shell(lambda ctx: attn.forward(ctx, inputs["h"], shell.stops[0]), rope, dtype, [StopNeeds(attn.cache_need())],
                  planning=[attn])
    runner = ModelRunner(shell, 32, 8, 4)
    n_a, n_b = 45, 20
    h_a, h_b = rand(rng, (n_a, hidden)).to(dtype), rand(rng, (n_b, hidden)).to(dtype)
    pos_a = np.stack([np.arange(n_a), np.arange(n_a) // 2 + 3, (np.arange(n_a) * 3) % 17])
    ra, rb = runner.open_request("a"), runner.open_request("b")
    outs_a, outs_b = [], []
    cuts = [(0, 17, 0, 20), (17, 19, None, None), (19, 45, None, None)]
    for a0, a1, b0, b1 in cuts:
        entries = [StepEntry(ra, [0] * (a1 - a0), [], pos_a[:, a0:a1])]
        hs = [h_a[a0:a1]]
        if b0 is not None:
            entries.append(StepEntry(rb, [0] * (b1 - b0), []))
            hs.append(h_b[b0:b1])
        inputs["h"] = torch.cat(hs).cuda()
        out = runner.step(entries)
        outs_a.append(out[:a1 - a0])
        if b0 is not None:
            outs_b.append(out[a1 - a0:])

    def oracle(h, pos):
        cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "hidden_size": nq * d}
        cos, sin = plain.mrope_cos_sin(pos, d, 10000.0, section, np.float64)
        return plain.attention_block(f64(h), w, "", cfg, cos, sin, window)

    assert err(torch.cat(outs_a), oracle(h_a, pos_a)) < tol(dtype)
    assert err(torch.cat(outs_b), oracle(h_b, plain.text_positions(n_b))) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_part(dtype):
    rng = np.random.default_rng(4)
    hidden, nq, nkv, d, inter = 64, 4, 2, 16, 88
    rope = mrope(d, (2, 3, 3), 10000.0, dtype)
    attn = parts.MIXERS["gqa_attention"](hidden_size=hidden, num_heads=nq, num_kv_heads=nkv, head_dim=d, position=rope)
    ffn = parts.FEED_FORWARDS["swiglu"](hidden_size=hidden, intermediate_size=inter)
    norms = [parts.NORMS["rmsnorm"](dim=hidden, eps=1e-6) for _ in range(2)]
    block = parts.BLOCKS["prenorm_residual"](attn, ffn, norms)
    w = {}
    for prefix, part in (("self_attn.", attn), ("mlp.", ffn), ("input_layernorm.", norms[0]), ("post_attention_layernorm.", norms[1])):
        w.update({"layers.0." + prefix + k: v for k, v in load_random(part, rng, dtype).items()})
    x0 = rand(rng, (23, hidden), scale=1.0)
    box = {}

    def fn(ctx):
        x = x0.clone().cuda()
        pending = block.forward(ctx, x, None, shell.stops[0])
        return x if pending is None else x + pending.float()       # None: the block added it itself

    shell = Shell(fn, rope, dtype, [StopNeeds(attn.cache_need())], planning=[attn])
    runner = ModelRunner(shell, 8, 8, 2)
    out = runner.step([StepEntry(runner.open_request("a"), [0] * 23, [])])
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "hidden_size": hidden, "rms_norm_eps": 1e-6}
    cos, sin = plain.mrope_cos_sin(plain.text_positions(23), d, 10000.0, (2, 3, 3), np.float64)
    ref = plain.decoder_layer(f64(x0), w, 0, cfg, cos, sin, None)
    assert err(out, ref) < tol(dtype) * 2
