"""Toy parts and toy architectures around them are registered from here, built, loaded and stepped
without a change to the engine's files: a mixer with state of its own (its model also runs one layer
twice and lets one stop read another stop's cache), a feed-forward that routes tokens to experts,
and a position encoding with one axis and another pairing of channels."""

import os

import numpy as np
import pytest
import torch

from plain import decoder as plain
from qwen25vl_lite.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
from qwen25vl_lite.engine.runner import ModelRunner, StepEntry
from qwen25vl_lite.parts import MIXERS, Mixer, StateNeed, TensorSpec, register_mixer
from qwen25vl_lite.weights import load_model, write_random_model

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV, D, INTER, VOCAB, EPS, DECAY = 48, 3, 1, 16, 80, 97, 1e-5, 0.9


if "toy_decaying_sum" not in MIXERS:
    @register_mixer("toy_decaying_sum")
    class DecayingSum(Mixer):
        """s_t = decay * s_(t-1) + h_t;  out_t = W s_t.  The state s is the request's
        fixed-size state; it is read at the start of a portion and written at its end."""

        def __init__(self, hidden_size, decay, position=None):
            self.hidden_size, self.decay = hidden_size, decay

        def tensor_specs(self):
            return (TensorSpec("mix.weight", (self.hidden_size, self.hidden_size)),)

        def state_need(self):
            return StateNeed((self.hidden_size,), "float32")

        def load(self, tensors, device, dtype):
            self.w = tensors["mix.weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, stop):
            out = torch.empty_like(h)
            at = 0
            for n, slot in zip(ctx.host_q_lens, ctx.host_slots):
                s = stop.state[slot]
                for t in range(n):
                    s = self.decay * s + h[at + t].float()
                    out[at + t] = (self.w @ s).to(h.dtype)
                stop.state[slot] = s
                at += n
            return out


def toy_spec(cfg):
    norms = lambda: (PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "norm_a."), PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "norm_b."))
    ffn = PartSpec("swiglu", dict(hidden_size=HIDDEN, intermediate_size=INTER), "ffn.")
    layers = (
        LayerSpec("prenorm_residual", PartSpec("toy_decaying_sum", dict(hidden_size=HIDDEN, decay=DECAY), "toy."), ffn, norms(), "blocks.0."),
        LayerSpec("prenorm_residual", PartSpec("gqa_attention", dict(hidden_size=HIDDEN, num_heads=HEADS, num_kv_heads=KV, head_dim=D), "attn."),
                  ffn, norms(), "blocks.1."),
    )
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=VOCAB, hidden_size=HIDDEN), "embed."),
        layers=layers,
        schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)),
        final_norm=PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "final_norm."),
        head=PartSpec("linear_head", dict(vocab_size=VOCAB, hidden_size=HIDDEN, tied=True, tied_to="embed.weight"), "head."),
        position=PartSpec("mrope", dict(head_dim=D, theta=10000.0, sections=(2, 3, 3))),
    )


register_architecture("ToyRecurrentForTest", lambda raw: dict(raw), toy_spec, replace=True)


def oracle(w, ids):
    """The toy model from the plain parts, whole sequence, float64."""
    n = len(ids)
    cfg = {"num_attention_heads": HEADS, "num_key_value_heads": KV, "hidden_size": HEADS * D}
    cos, sin = plain.mrope_cos_sin(plain.text_positions(n), D, 10000.0, (2, 3, 3), np.float64)
    x = w["embed.weight"][np.asarray(ids)]

    def ffn(x, p):
        return plain.swiglu_mlp(plain.rms_norm(x, w[p + "norm_b.weight"], EPS), w, p + "ffn.")

    def toy(x):
        h = plain.rms_norm(x, w["blocks.0.norm_a.weight"], EPS)
        s, out = np.zeros(HIDDEN), np.zeros_like(h)
        for t in range(n):
            s = DECAY * s + h[t]
            out[t] = w["blocks.0.toy.mix.weight"] @ s
        x = x + out
        return x + ffn(x, "blocks.0.")

    def qkv(h):
        p = "blocks.1.attn."
        q = (h @ w[p + "q_proj.weight"].T + w[p + "q_proj.bias"]).reshape(n, HEADS, D)
        k = (h @ w[p + "k_proj.weight"].T + w[p + "k_proj.bias"]).reshape(n, KV, D)
        v = (h @ w[p + "v_proj.weight"].T + w[p + "v_proj.bias"]).reshape(n, KV, D)
        return plain.apply_mrope(q, cos, sin), plain.apply_mrope(k, cos, sin), v

    def attn(x, kv=None):
        q, k, v = qkv(plain.rms_norm(x, w["blocks.1.norm_a.weight"], EPS))
        if kv is not None:
            k, v = kv                                  # this stop reads the other stop's keys and values
        x = x + plain.causal_attention(q, k, v).reshape(n, HEADS * D) @ w["blocks.1.attn.o_proj.weight"].T
        return x + ffn(x, "blocks.1."), (k, v)

    x = toy(x)
    x, kv = attn(x)
    x = toy(x)
    x, _ = attn(x, kv)
    return plain.rms_norm(x, w["final_norm.weight"], EPS) @ w["embed.weight"].T


def test_toy_architecture_builds_loads_and_steps(tmp_path):
    folder = write_random_model(str(tmp_path / "toy"), {"architectures": ["ToyRecurrentForTest"]}, seed=4, prefix="")
    _, model = load_model(folder, "float32", "cuda:0")
    needs = model.stop_needs()
    assert [n.state is not None for n in needs] == [True, False, True, False]
    assert needs[3].cache_of == 1 and needs[0].cache is None
    runner = ModelRunner(model, 16, 8, 2)
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].stops == [1]      # stop 3 keeps no pages
    assert sorted(runner.cache.states) == [0, 2]                                     # one state per stop, not per layer
    w = {k: v.astype(np.float64) for k, v in plain.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    rng = np.random.default_rng(0)
    ids_a, ids_b = rng.integers(0, VOCAB, size=29).tolist(), rng.integers(0, VOCAB, size=18).tolist()
    want_a, want_b = oracle(w, ids_a), oracle(w, ids_b)

    ra = runner.open_request("a")
    whole = runner.step([StepEntry(ra, ids_a, list(range(29)))]).cpu().numpy()
    assert np.abs(whole - want_a).max() < 1e-4
    runner.close_request(ra)

    # the same slots again, in portions, two requests side by side: the state was zeroed at
    # admission, is carried across portions, and the cut does not change the result
    ra, rb = runner.open_request("a2"), runner.open_request("b")
    got_a, got_b = [], []
    cuts_a, cuts_b = [0, 5, 7, 20, 29], [0, 9, 10, 18, 18]
    for i in range(4):
        entries, na, nb = [], cuts_a[i + 1] - cuts_a[i], cuts_b[i + 1] - cuts_b[i]
        entries.append(StepEntry(ra, ids_a[cuts_a[i]:cuts_a[i + 1]], list(range(na))))
        if nb:
            entries.append(StepEntry(rb, ids_b[cuts_b[i]:cuts_b[i + 1]], list(range(nb))))
        out = runner.step(entries).cpu().numpy()
        got_a.append(out[:na])
        got_b.append(out[na:])
    assert np.abs(np.concatenate(got_a) - want_a).max() < 1e-4
    assert np.abs(np.concatenate(got_b) - want_b).max() < 1e-4
    assert np.abs(np.concatenate(got_a) - whole).max() < 1e-5


# ---- a feed-forward with routing and another position encoding, defined here ----------------------
from qwen25vl_lite.parts import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding,  # noqa: E402
                                 register_feed_forward, register_position_encoding)

EXPERTS, EXPERT_INTER, THETA2 = 3, 24, 500.0

if "toy_routed" not in FEED_FORWARDS:
    @register_feed_forward("toy_routed")
    class ToyRouted(FeedForward):
        """Every token goes to the one expert whose router logit is largest (logits in float32);
        an expert is relu(h W1^T) W2^T.  The cache and the scheduler know nothing of it."""

        def __init__(self, hidden_size, num_experts, expert_size):
            self.h, self.e, self.i = hidden_size, num_experts, expert_size

        def tensor_specs(self):
            return (TensorSpec("router.weight", (self.e, self.h)), TensorSpec("w1", (self.e, self.i, self.h)),
                    TensorSpec("w2", (self.e, self.h, self.i)))

        def load(self, tensors, device, dtype):
            self.router = tensors["router.weight"].to(device=device, dtype=torch.float32)
            self.w1 = tensors["w1"].to(device=device, dtype=torch.float32)
            self.w2 = tensors["w2"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h):
            x = h.float()
            choice = (x @ self.router.T).argmax(dim=1)
            out = torch.empty_like(x)
            for e in range(self.e):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    out[rows] = torch.relu(x[rows] @ self.w1[e].T) @ self.w2[e].T
            return out.to(h.dtype)


if "toy_rope_pairs" not in POSITION_ENCODINGS:
    @register_position_encoding("toy_rope_pairs")
    class ToyRopePairs(PositionEncoding):
        """One position axis; channels (2j, 2j+1) are rotated together (not j with j + D/2).  It has
        no tables for the fused decode kernel, so its model runs the general attention path."""

        axes = 1

        def __init__(self, head_dim, theta):
            self.d, self.theta = int(head_dim), float(theta)

        def load(self, tensors, device, dtype):
            self.inv = (1.0 / self.theta ** (torch.arange(0, self.d, 2, dtype=torch.float32) / self.d)).to(device)

        def default_positions(self, start, count, offset):
            return np.arange(start + offset, start + offset + count, dtype=np.int64)[None, :]

        def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
            n = qkv.shape[0]
            ang = ctx.positions[0].float()[:, None] * self.inv[None, :]              # [n, D/2]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            heads = qkv.view(n, nq + 2 * nkv, head_dim)
            x = heads[:, :nq + nkv].float()
            a, b = x[..., 0::2], x[..., 1::2]
            y = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).reshape(n, nq + nkv, head_dim)
            heads[:, :nq + nkv] = y.to(qkv.dtype)
            if kv is not None:
                slot = kv.kv_slot.long()
                ok = slot >= 0
                page, off = slot[ok] // kv.page_size, slot[ok] % kv.page_size
                kv.k_pages[page, :, off] = heads[ok, nq:nq + nkv]
                kv.v_pages[page, :, off] = heads[ok, nq + nkv:]


def toy2_spec(cfg):
    norms = lambda: (PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "norm_a."), PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "norm_b."))
    attn = PartSpec("gqa_attention", dict(hidden_size=HIDDEN, num_heads=HEADS, num_kv_heads=KV, head_dim=D), "attn.")
    layers = (
        LayerSpec("prenorm_residual", attn, PartSpec("toy_routed", dict(hidden_size=HIDDEN, num_experts=EXPERTS, expert_size=EXPERT_INTER), "moe."),
                  norms(), "blocks.0."),
        LayerSpec("prenorm_residual", attn, PartSpec("swiglu", dict(hidden_size=HIDDEN, intermediate_size=INTER), "ffn."), norms(), "blocks.1."),
    )
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=VOCAB, hidden_size=HIDDEN), "embed."),
        layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)),
        final_norm=PartSpec("rmsnorm", dict(dim=HIDDEN, eps=EPS), "final_norm."),
        head=PartSpec("linear_head", dict(vocab_size=VOCAB, hidden_size=HIDDEN, tied=True, tied_to="embed.weight"), "head."),
        position=PartSpec("toy_rope_pairs", dict(head_dim=D, theta=THETA2)),
    )


register_architecture("ToyRoutedForTest", lambda raw: dict(raw), toy2_spec, replace=True)


def oracle2(w, ids):
    n = len(ids)
    pos = np.arange(n, dtype=np.float64)
    inv = 1.0 / THETA2 ** (np.arange(0, D, 2, dtype=np.float64) / D)
    ang = pos[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def rot(x):
        a, b = x[..., 0::2], x[..., 1::2]
        return np.stack([a * cos - b * sin, b * cos + a * sin], axis=-1).reshape(x.shape)

    x = w["embed.weight"][np.asarray(ids)]
    for layer in (0, 1):
        p = f"blocks.{layer}."
        h = plain.rms_norm(x, w[p + "norm_a.weight"], EPS)
        q = (h @ w[p + "attn.q_proj.weight"].T + w[p + "attn.q_proj.bias"]).reshape(n, HEADS, D)
        k = (h @ w[p + "attn.k_proj.weight"].T + w[p + "attn.k_proj.bias"]).reshape(n, KV, D)
        v = (h @ w[p + "attn.v_proj.weight"].T + w[p + "attn.v_proj.bias"]).reshape(n, KV, D)
        x = x + plain.causal_attention(rot(q), rot(k), v).reshape(n, HEADS * D) @ w[p + "attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[p + "norm_b.weight"], EPS)
        if layer == 0:
            choice = (h @ w[p + "moe.router.weight"].T).argmax(axis=1)
            out = np.zeros_like(h)
            for t in range(n):
                e = choice[t]
                out[t] = np.maximum(h[t] @ w[p + "moe.w1"][e].T, 0) @ w[p + "moe.w2"][e].T
            x = x + out
        else:
            x = x + plain.swiglu_mlp(h, w, p + "ffn.")
    return plain.rms_norm(x, w["final_norm.weight"], EPS) @ w["embed.weight"].T


def test_toy_routed_feed_forward_and_other_position_encoding(tmp_path):
    """A feed-forward that routes tokens to experts and a position encoding with one axis and
    another pairing of channels, both defined in this file: registered, built into a model by data,
    loaded from a random model folder, and stepped whole, in portions and token by token."""
    folder = write_random_model(str(tmp_path / "toy2"), {"architectures": ["ToyRoutedForTest"]}, seed=9, prefix="")
    _, model = load_model(folder, "float32", "cuda:0")
    runner = ModelRunner(model, 12, 8, 2)
    assert runner.axes == 1
    w = {k: v.astype(np.float64) for k, v in plain.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    ids = np.random.default_rng(3).integers(0, VOCAB, size=37).tolist()
    want = oracle2(w, ids)
    r = runner.open_request("whole")
    whole = runner.step([StepEntry(r, ids, list(range(37)))]).cpu().numpy()
    runner.close_request(r)
    assert np.abs(whole - want).max() < 1e-4
    r = runner.open_request("cut")
    got = [runner.step([StepEntry(r, ids[:20], list(range(20)))]).cpu().numpy(),
           runner.step([StepEntry(r, ids[20:23], [0, 1, 2])]).cpu().numpy()]
    got += [runner.step([StepEntry(r, [t], [0])]).cpu().numpy() for t in ids[23:]]
    runner.close_request(r)
    assert np.abs(np.concatenate(got) - want).max() < 1e-4
    runner.cache.check(runner.live.values())


# ---- layers that differ in their position encoding ---------------------------------------------------
D3, HEADS3, KV3, HIDDEN3, THETA3 = 64, 4, 2, 256, 3000.0

if "toy_rope_1axis" not in POSITION_ENCODINGS:
    @register_position_encoding("toy_rope_1axis")
    class ToyRope1Axis(PositionEncoding):
        """A rotary encoding with ONE position axis that pairs channel j with j + D/2 and hands out
        its tables, so that one-token steps take the fused decode attention kernel; everything
        else goes through the engine's rotate-and-store kernel with those same tables."""

        axes = 1
        default_is_linear = True
        graph_safe = True

        def __init__(self, head_dim, theta):
            self.d, self.theta = int(head_dim), float(theta)

        def load(self, tensors, device, dtype):
            self.inv = (1.0 / self.theta ** (torch.arange(0, self.d, 2, dtype=torch.float32) / self.d)).to(device)
            self.axis = torch.zeros(self.d // 2, dtype=torch.int32, device=device)

        def default_positions(self, start, count, offset):
            return np.arange(start + offset, start + offset + count, dtype=np.int64)[None, :]

        def rope_tables(self):
            return self.inv, self.axis

        def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
            from qwen25vl_lite.ops import kernels
            if kv is None:
                kernels.rope_store(qkv, ctx.positions, self.inv, self.axis, None, None, None, nq, nkv, head_dim, 1)
            else:
                kernels.rope_store(qkv, ctx.positions, self.inv, self.axis, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv,
                                   head_dim, kv.page_size)

    @register_position_encoding("toy_no_position")
    class ToyNoPosition(PositionEncoding):
        """No encoding at all: keys and values are stored as projected (a layer that relies on the
        causal mask alone).  It defines no positions of its own, so it can only be a layer's
        encoding, never the model's."""

        axes = 0
        graph_safe = True

        def rotate_and_store(self, ctx, qkv, nq, nkv, head_dim, kv):
            from qwen25vl_lite.ops import kernels
            if kv is not None:
                kernels.rope_store(qkv, None, None, None, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv, head_dim, kv.page_size)


def toy3_spec(cfg):
    norms = lambda: (PartSpec("rmsnorm", dict(dim=HIDDEN3, eps=EPS), "norm_a."), PartSpec("rmsnorm", dict(dim=HIDDEN3, eps=EPS), "norm_b."))
    attn = PartSpec("gqa_attention", dict(hidden_size=HIDDEN3, num_heads=HEADS3, num_kv_heads=KV3, head_dim=D3), "attn.")
    ffn = PartSpec("swiglu", dict(hidden_size=HIDDEN3, intermediate_size=96), "ffn.")
    layers = (
        LayerSpec("prenorm_residual", attn, ffn, norms(), "blocks.0."),                               # the model's encoding
        LayerSpec("prenorm_residual", attn, ffn, norms(), "blocks.1.", position=PartSpec("toy_no_position")),
        LayerSpec("prenorm_residual", attn, ffn, norms(), "blocks.2.",
                  position=PartSpec("toy_rope_1axis", dict(head_dim=D3, theta=7.0 * THETA3))),         # another theta
    )
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=VOCAB, hidden_size=HIDDEN3), "embed."),
        layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)),
        final_norm=PartSpec("rmsnorm", dict(dim=HIDDEN3, eps=EPS), "final_norm."),
        head=PartSpec("linear_head", dict(vocab_size=VOCAB, hidden_size=HIDDEN3, tied=True, tied_to="embed.weight"), "head."),
        position=PartSpec("toy_rope_1axis", dict(head_dim=D3, theta=THETA3)),
    )


register_architecture("ToyMixedPositionsForTest", lambda raw: dict(raw), toy3_spec, replace=True)


def oracle3(w, ids):
    n = len(ids)
    pos = np.arange(n, dtype=np.float64)

    def rot(x, theta):
        if theta is None:
            return x
        inv = 1.0 / theta ** (np.arange(0, D3, 2, dtype=np.float64) / D3)
        ang = pos[:, None] * inv[None, :]
        cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        a, b = x[..., :D3 // 2], x[..., D3 // 2:]
        return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)

    x = w["embed.weight"][np.asarray(ids)]
    for layer, theta in enumerate((THETA3, None, 7.0 * THETA3)):
        p = f"blocks.{layer}."
        h = plain.rms_norm(x, w[p + "norm_a.weight"], EPS)
        q = (h @ w[p + "attn.q_proj.weight"].T + w[p + "attn.q_proj.bias"]).reshape(n, HEADS3, D3)
        k = (h @ w[p + "attn.k_proj.weight"].T + w[p + "attn.k_proj.bias"]).reshape(n, KV3, D3)
        v = (h @ w[p + "attn.v_proj.weight"].T + w[p + "attn.v_proj.bias"]).reshape(n, KV3, D3)
        x = x + plain.causal_attention(rot(q, theta), rot(k, theta), v).reshape(n, HEADS3 * D3) @ w[p + "attn.o_proj.weight"].T
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[p + "norm_b.weight"], EPS), w, p + "ffn.")
    return plain.rms_norm(x, w["final_norm.weight"], EPS) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_layers_with_different_position_encodings(tmp_path, dtype, tol):
    """Three layers of one model: the model's one-axis rotary encoding, no encoding at all, and the
    same rotary kind with another base -- all three kinds defined in this file, named layer by
    layer in the model's description.  Stepped whole, in portions and token by token (in bfloat16
    from CUDA graphs: the rotary layers through the fused decode attention with their one-axis
    tables, the layer without encoding through the split-KV decode kernel)."""
    folder = write_random_model(str(tmp_path / "toy3"), {"architectures": ["ToyMixedPositionsForTest"]}, seed=10,
                                storage_dtype=dtype, prefix="")
    _, model = load_model(folder, dtype, "cuda:0")
    assert len(model.position_encodings()) == 3
    runner = ModelRunner(model, 16, 16, 2)
    assert runner.axes == 1 and runner.cuda_graphs
    w = {k: v.astype(np.float64) for k, v in plain.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    ids = np.random.default_rng(4).integers(0, VOCAB, size=90).tolist()
    want = oracle3(w, ids)
    r = runner.open_request("whole")
    whole = runner.step([StepEntry(r, ids, list(range(90)))]).cpu().numpy()
    runner.close_request(r)
    assert np.abs(whole - want).max() < tol
    r = runner.open_request("cut")
    got = [runner.step([StepEntry(r, ids[:40], list(range(40)))]).cpu().numpy(),
           runner.step([StepEntry(r, ids[40:43], [0, 1, 2])]).cpu().numpy()]
    got += [runner.step([StepEntry(r, [t], [0])]).cpu().numpy() for t in ids[43:]]
    runner.close_request(r)
    assert np.abs(np.concatenate(got) - want).max() < tol
    if dtype == "bfloat16":
        assert runner.graph_replays >= 40
    runner.cache.check(runner.live.values())
