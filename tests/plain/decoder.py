"""Plain, slow implementation of the Qwen2.5-VL text decoder (NumPy, whole sequences, no cache).

This is the oracle of the test-suite.  It is written from the formulas of
zhangjianbang-nb/qwen25vl-lite (each function cites the file and lines of that project it
restates) and shares no code with the engine: it has its own weight reading, its own
position ids, its own sampler.  One function for each part; every function works on a whole
sequence at once and keeps nothing between calls.

All arithmetic runs in the dtype of ``weights`` (float32 as stored, or float64 when the
caller converts the dict), so the oracle is at least as exact as the engine's 32-bit path.
"""

from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

# ----------------------------------------------------------------------------------------
# weights: an independent reader of the safetensors container
# ----------------------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) -> float32: bf16 is the upper half of an fp32."""
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """File layout: u64 little-endian header length, JSON header, raw little-endian data."""
    with open(path, "rb") as fh:
        blob = fh.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out: Dict[str, np.ndarray] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = blob[base + lo:base + hi]
        if meta["dtype"] == "BF16":
            arr = _bf16_to_f32(np.frombuffer(buf, dtype=np.uint16))
        else:
            arr = np.frombuffer(buf, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def load_model_dir(model_dir: str, dtype=np.float32) -> Tuple[dict, Dict[str, np.ndarray]]:
    """Returns (text config dict, weights by un-prefixed name).

    Name handling restates model.py:52-73 of the reference: ``model.language_model.``,
    ``language_model.`` and ``model.`` prefixes all name the same decoder tensors, and
    ``lm_head.weight`` stands alone.  Config handling restates config.py:163-178: sizes live
    under ``text_config`` (we also accept them flat), the MRoPE section under
    ``rope_scaling`` or ``rope_parameters``.
    """
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        raw = json.load(fh)
    text = dict(raw.get("text_config") or raw)
    for key in ("rope_scaling", "rope_parameters"):
        block = raw.get(key) or text.get(key)
        if isinstance(block, dict):
            for k in ("mrope_section", "rope_theta"):
                if k in block:
                    text.setdefault(k, block[k])
    for k in ("rope_theta", "mrope_section"):
        if k in raw:
            text.setdefault(k, raw[k])
    text.setdefault("tie_word_embeddings", raw.get("tie_word_embeddings", True))
    weights: Dict[str, np.ndarray] = {}
    for name, arr in read_safetensors(os.path.join(model_dir, "model.safetensors")).items():
        for prefix in ("model.language_model.", "language_model.", "model."):
            if name.startswith(prefix):
                name = name[len(prefix):]
                break
        weights[name] = arr.astype(dtype)
    return text, weights


# ----------------------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------------------


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """layers.py:27-31 -- ``x * rsqrt(mean(x^2) + eps)`` then times the weight (plain form)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * weight


def rope_inv_freq(head_dim: int, theta: float) -> np.ndarray:
    """rope.py:26-33 -- ``1 / theta^(2i/D)`` for i in [0, D/2), computed in float32."""
    idx = np.arange(0, head_dim, 2, dtype=np.float32)
    return (np.float32(1.0) / np.power(np.float32(theta), idx / np.float32(head_dim))).astype(np.float32)


def mrope_axis_of_channel(mrope_section: Sequence[int]) -> np.ndarray:
    """rope.py:88-95 -- the section list is repeated ([s0,s1,s2,s0,s1,s2]) and its six
    chunks take their angles from axes 0,1,2,0,1,2; so channel j of the first half and
    channel j + D/2 use the same axis.  Returns the axis for j in [0, D/2)."""
    axis: List[int] = []
    for a, n in enumerate(mrope_section):
        axis += [a] * int(n)
    return np.asarray(axis, dtype=np.int64)


def mrope_cos_sin(positions: np.ndarray, head_dim: int, theta: float,
                  mrope_section: Sequence[int], dtype) -> Tuple[np.ndarray, np.ndarray]:
    """rope.py:48-68 and 71-96 -- angle = pos[axis(j)] * inv_freq[j] in float32; the table of
    width D repeats the D/2 angles twice.  ``positions`` is [3, N].  Returns cos, sin [N, D]."""
    inv = rope_inv_freq(head_dim, theta)
    if int(sum(mrope_section)) * 2 != head_dim:
        raise ValueError("mrope_section does not cover head_dim")
    axis = mrope_axis_of_channel(mrope_section)
    pos = positions.astype(np.float32)                       # [3, N]
    picked = pos[axis, :].T                                  # [N, D/2]
    ang = (picked * inv[None, :]).astype(np.float32)         # float32 product, as the reference
    ang = np.concatenate([ang, ang], axis=-1)
    return np.cos(ang).astype(dtype), np.sin(ang).astype(dtype)


def rotate_half(x: np.ndarray) -> np.ndarray:
    """rope.py:36-40 -- cat(-x[D/2:], x[:D/2])."""
    half = x.shape[-1] // 2
    return np.concatenate([-x[..., half:], x[..., :half]], axis=-1)


def apply_mrope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """rope.py:96 -- ``x*cos + rotate_half(x)*sin``; x is [N, heads, D], tables are [N, D]."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def text_positions(n: int, start: int = 0) -> np.ndarray:
    """rope.py:238-247 -- pure text: all three axes carry the running index."""
    r = np.arange(start, start + n, dtype=np.int64)
    return np.stack([r, r, r], axis=0)


def prompt_positions(n: int, image_spans: Sequence[Tuple[int, int, int, int]] = ()) -> Tuple[np.ndarray, int]:
    """rope.py:137-235 (get_rope_index) with rope.py:99-126 (vision_position_ids), for a
    prompt of ``n`` tokens whose image spans are given as ``(start, t, h, w)`` in merged grid
    units (the span has t*h*w tokens).

    Text runs advance a cursor by their length and put ``cursor + i`` on all three axes.  An
    image run at cursor c gets t = c + t_idx (interval 1 for images), h = c + row,
    w = c + col in t-major, row-major order, and advances the cursor by max(h, w).
    ``rope_delta = max(pos) + 1 - n``.
    """
    chunks: List[np.ndarray] = []
    cursor = 0
    at = 0
    for (start, t, h, w) in sorted(image_spans):
        if start > at:
            chunks.append(text_positions(start - at, cursor))
            cursor += start - at
        tt, hh, ww = np.meshgrid(np.arange(t), np.arange(h), np.arange(w), indexing="ij")
        chunks.append(np.stack([tt.reshape(-1), hh.reshape(-1), ww.reshape(-1)], axis=0).astype(np.int64) + cursor)
        cursor += max(h, w)
        at = start + t * h * w
    if n > at:
        chunks.append(text_positions(n - at, cursor))
    pos = np.concatenate(chunks, axis=1)
    assert pos.shape == (3, n), (pos.shape, n)
    return pos, int(pos.max()) + 1 - n


def decode_positions(num_computed: int, rope_delta: int) -> np.ndarray:
    """rope.py:238-247, engine.py:447 -- a decoded token: all axes = computed + rope_delta."""
    p = num_computed + rope_delta
    return np.asarray([[p], [p], [p]], dtype=np.int64)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: Optional[int] = None) -> np.ndarray:
    """text.py:78,156-175; attention.py:143-148,366-372 -- scores = q.k^T * D^-1/2, query i
    sees keys j <= i, softmax over keys, out = P.v; query head h reads kv head
    h // (nq / nkv).  ``window`` (not used by the reference's attention, which parses
    sliding_window at config.py:93-94 and never consults it) keeps only i - window < j.
    q: [N, nq, D]; k, v: [N, nkv, D].  Returns [N, nq, D]."""
    n, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = d ** -0.5
    out = np.zeros_like(q)
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    allow = j <= i
    if window is not None:
        allow &= j > i - window
    for h in range(nq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = np.where(allow, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def attention_block(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str, cfg: dict,
                    cos: np.ndarray, sin: np.ndarray, window: Optional[int]) -> np.ndarray:
    """text.py:85-90,116-118,177-178 -- biased q/k/v projections, head-major split, MRoPE on
    q and k, attention, concat heads, unbiased o projection."""
    n = x.shape[0]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg["hidden_size"] // nq
    q = x @ w[prefix + "q_proj.weight"].T + w[prefix + "q_proj.bias"]
    k = x @ w[prefix + "k_proj.weight"].T + w[prefix + "k_proj.bias"]
    v = x @ w[prefix + "v_proj.weight"].T + w[prefix + "v_proj.bias"]
    q = apply_mrope(q.reshape(n, nq, d), cos, sin)
    k = apply_mrope(k.reshape(n, nkv, d), cos, sin)
    o = causal_attention(q, k, v.reshape(n, nkv, d), window)
    return o.reshape(n, nq * d) @ w[prefix + "o_proj.weight"].T


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def swiglu_mlp(x: np.ndarray, w: Dict[str, np.ndarray], prefix: str) -> np.ndarray:
    """text.py:59-66 -- down(silu(gate x) * up x), no biases."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (silu(g) * u) @ w[prefix + "down_proj.weight"].T


def layer_windows(cfg: dict) -> List[Optional[int]]:
    """text.py:156-175 -- the reference's attention sees every key: ``sliding_window`` and
    ``use_sliding_window`` are parsed (config.py:93-94,105-109) and never consulted, so every
    layer's window is None.  A test architecture that does window lists its windows under
    ``layer_windows`` (None = all keys)."""
    n = cfg["num_hidden_layers"]
    if cfg.get("layer_windows") is not None:
        assert len(cfg["layer_windows"]) == n
        return [None if v is None else int(v) for v in cfg["layer_windows"]]
    return [None] * n


def decoder_layer(x: np.ndarray, w: Dict[str, np.ndarray], i: int, cfg: dict,
                  cos: np.ndarray, sin: np.ndarray, window: Optional[int]) -> np.ndarray:
    """text.py:196-206 -- pre-norm residual block."""
    p = f"layers.{i}."
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, cos, sin, window)
    x = x + swiglu_mlp(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return x


def forward_logits(cfg: dict, w: Dict[str, np.ndarray], token_ids: Sequence[int],
                   positions: Optional[np.ndarray] = None, rows: Optional[Sequence[int]] = None) -> np.ndarray:
    """text.py:213,243-279; model.py:84-86,200-202 -- embed, layers, final norm, head (the
    embedding table again when tied and no lm_head.weight is stored).  Logits for every
    position, [N, V], or for the positions ``rows`` only (model.py:200-202 keeps the wanted
    positions before the head; a large vocabulary makes that worth it here too)."""
    ids = np.asarray(token_ids, dtype=np.int64)
    n = ids.shape[0]
    dtype = w["embed_tokens.weight"].dtype
    if positions is None:
        positions = text_positions(n)
    d = cfg["hidden_size"] // cfg["num_attention_heads"]
    cos, sin = mrope_cos_sin(np.asarray(positions), d, cfg["rope_theta"], cfg["mrope_section"], dtype)
    x = w["embed_tokens.weight"][ids]
    for i, window in enumerate(layer_windows(cfg)):
        x = decoder_layer(x, w, i, cfg, cos, sin, window)
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = rms_norm(x, w["norm.weight"], cfg["rms_norm_eps"])
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["embed_tokens.weight"]
    return x @ head.T


# ----------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    """splitmix64 finaliser on Python integers."""
    x &= _MASK64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK64
    x ^= x >> 31
    return x


def gumbel_noise(seed: int, token_index: int, vocab: int) -> np.ndarray:
    """The engine's counter-based noise, restated: key = mix(seed * golden + token_index),
    u_i = (top 23 bits of mix(key + i * odd) + 0.5) / 2^23 (exact in float32, never 0 or 1),
    g_i = -log(-log(u_i)) in float32.

    The reference draws with torch.multinomial from a CPU generator seeded
    ``seed + len(outputs)`` (engine.py:823-829, sampling.py:103-106); the engine keeps that
    keying (one stream per seed and token index) but not the generator, so tokens are
    compared with this restatement and distributions with the softmax."""
    key = _mix64((seed & _MASK64) * 0x9E3779B97F4A7C15 + (token_index & _MASK64))
    g = np.empty(vocab, dtype=np.float32)
    for i in range(vocab):
        bits = _mix64(key + i * 0xD1342543DE82EF95) >> 41
        u = np.float32((bits + 0.5) * (1.0 / 8388608.0))
        g[i] = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
    return g


def apply_penalties(logits: np.ndarray, prev_ids: Sequence[int], repetition: float = 1.0,
                    presence: float = 0.0, frequency: float = 0.0) -> np.ndarray:
    """sampling.py:44-64 -- seen tokens: positive logits divided by the repetition penalty,
    negative ones multiplied; then minus presence for seen tokens and frequency * count."""
    out = logits.astype(np.float32).copy()
    if not len(prev_ids):
        return out
    counts = np.bincount(np.asarray(prev_ids, dtype=np.int64), minlength=out.shape[-1]).astype(np.float32)
    seen = counts > 0
    if repetition != 1.0:
        out[seen] = np.where(out[seen] > 0, out[seen] / np.float32(repetition), out[seen] * np.float32(repetition))
    out = out - np.float32(presence) * seen.astype(np.float32)
    out = out - np.float32(frequency) * counts
    return out


def filter_scores(scores: np.ndarray, top_k: int = -1, min_p: float = 0.0, top_p: float = 1.0) -> np.ndarray:
    """sampling.py:74-101 -- in this order: top-k keeps scores >= the k-th largest; min-p
    keeps probabilities >= min_p * max; top-p keeps the smallest sorted prefix whose
    cumulative probability reaches top_p (the crossing token included).  Dropped = -inf."""
    s = scores.astype(np.float32).copy()

    def softmax(z):
        z = z - z.max()
        e = np.exp(z)
        return e / e.sum()

    if top_k and top_k > 0:
        k = min(int(top_k), s.size)
        kth = np.sort(s)[::-1][k - 1]
        s = np.where(s < kth, -np.inf, s)
    if min_p > 0:
        p = softmax(s)
        s = np.where(p < np.float32(min_p) * p.max(), -np.inf, s)
    if top_p < 1.0:
        order = np.argsort(-s, kind="stable")
        p = softmax(s[order])
        cum = np.cumsum(p)
        crossing = np.nonzero(cum >= np.float32(top_p))[0]
        keep_n = int(crossing[0]) + 1 if crossing.size else s.size
        drop = order[max(keep_n, 1):]
        s[drop] = -np.inf
    return s.astype(np.float32)


def sample(logits: np.ndarray, temperature: float, seed: int = 0, token_index: int = 0,
           top_k: int = -1, min_p: float = 0.0, top_p: float = 1.0) -> int:
    """sampling.py:67-72 -- temperature <= 0 is argmax (first maximum); else the scores are
    ``logits / T`` in float32, filtered, and one token is drawn from their softmax.  The draw
    is Gumbel-max: argmax(score_i + g_i) is a sample of softmax(score)."""
    lg = logits.astype(np.float32)
    if temperature <= 0:
        return int(np.argmax(lg))
    s = filter_scores(lg / np.float32(temperature), top_k, min_p, top_p)
    return int(np.argmax(s + gumbel_noise(seed, token_index, lg.shape[-1])))


def greedy_generate(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], n_new: int,
                    positions: Optional[np.ndarray] = None, rope_delta: int = 0,
                    temperature: float = 0.0, seed: int = 0) -> List[int]:
    """engine.py:741-808 restated without a cache: after each token the whole sequence is
    run again.  Token k (0-based) of the output is drawn with key (seed, k)."""
    ids = list(prompt)
    pos = text_positions(len(ids)) if positions is None else np.asarray(positions)
    out: List[int] = []
    for k in range(n_new):
        logits = forward_logits(cfg, w, ids, pos)[-1]
        tok = sample(logits, temperature, seed, k)
        out.append(tok)
        pos = np.concatenate([pos, decode_positions(len(ids), rope_delta)], axis=1)
        ids.append(tok)
    return out


def generation_margins(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], generated: Sequence[int],
                       positions: Optional[np.ndarray] = None, rope_delta: int = 0,
                       temperature: float = 0.0, seed: int = 0) -> List[float]:
    """How far each generated token is from the one this implementation would have chosen at its
    place, given the tokens before it: ``max(score) - score[token]`` with score = logits for
    greedy, logits / T + the draw's noise otherwise (the choice is an argmax either way,
    sampling.py:67-72 and ``sample`` above).  0 means the same choice; an engine that rounds
    differently (bfloat16) may pick a token whose score is within its rounding of the best, and
    teacher forcing keeps one such pick from derailing the comparison of the later ones."""
    ids = list(prompt) + [int(t) for t in generated]
    n0 = len(prompt)
    pos = text_positions(n0) if positions is None else np.asarray(positions)
    tail = [decode_positions(n, rope_delta) for n in range(n0, len(ids))]
    pos = np.concatenate([pos] + tail, axis=1) if tail else pos
    logits = forward_logits(cfg, w, ids, pos, rows=list(range(n0 - 1, len(ids) - 1)))
    out = []
    for k, tok in enumerate(generated):
        s = logits[k].astype(np.float64)
        if temperature > 0:
            s = s / temperature + gumbel_noise(seed, k, s.shape[-1]).astype(np.float64)
        out.append(float(s.max() - s[int(tok)]))
    return out
