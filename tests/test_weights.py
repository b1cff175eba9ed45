"""Weights: the container, loading by name with every accepted prefix, one error that lists
missing and unexpected tensors and wrong shapes, the random-weights mode."""

import json
import os

import numpy as np
import pytest
import torch

from plain import decoder as plain
from qwen25vl_lite.weights import SafetensorsFile, WeightsError, load_model, write_safetensors
from tiny_models import TINY, TINY_A, TINY_B


def _rewrite(src_dir, dst_dir, edit):
    """Copies a model folder, passing {name: tensor} through ``edit``."""
    os.makedirs(dst_dir, exist_ok=True)
    f = SafetensorsFile(os.path.join(src_dir, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors = edit(tensors) or tensors
    write_safetensors(os.path.join(dst_dir, "model.safetensors"), tensors.items())
    with open(os.path.join(src_dir, "config.json")) as a, open(os.path.join(dst_dir, "config.json"), "w") as b:
        b.write(a.read())
    return dst_dir


def test_container_round_trip_and_independent_reader(tmp_path):
    t = {"a.weight": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t.items(), {"k": "v"})
    f = SafetensorsFile(path)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for n, v in t.items():
        assert torch.equal(f.tensor(n), v) and f.dtype(n) == v.dtype and f.shape(n) == tuple(v.shape)
    other = plain.read_safetensors(path)
    assert np.array_equal(other["a.weight"], t["a.weight"].numpy())
    assert np.array_equal(other["b"], t["b"].float().numpy())
    from safetensors import safe_open       # the library reads what we wrote
    with safe_open(path, framework="pt") as lib:
        assert torch.equal(lib.get_tensor("b"), t["b"])


def test_random_mode_is_seeded_and_distributed_as_stated(model_dirs, tmp_path):
    from qwen25vl_lite.weights import write_random_model
    a = plain.read_safetensors(os.path.join(model_dirs["B"], "model.safetensors"))
    again = write_random_model(str(tmp_path / "again"), TINY_B, TINY["B"][1])
    b = plain.read_safetensors(os.path.join(again, "model.safetensors"))
    assert a.keys() == b.keys() and all(np.array_equal(a[k], b[k]) for k in a)
    other = plain.read_safetensors(os.path.join(write_random_model(str(tmp_path / "other"), TINY_B, 99), "model.safetensors"))
    assert not np.array_equal(a["lm_head.weight"], other["lm_head.weight"])
    emb = a["model.language_model.embed_tokens.weight"]
    assert abs(emb.std() - 0.02) < 1e-3 and abs(emb.mean()) < 1e-3
    norm = a["model.language_model.layers.0.input_layernorm.weight"]
    assert abs(norm.mean() - 1.0) < 0.02
    assert abs(a["model.language_model.layers.1.self_attn.q_proj.bias"].std() - 0.02) < 0.01
    assert "lm_head.weight" in a                                  # untied: a head of its own
    tied = plain.read_safetensors(os.path.join(model_dirs["A"], "model.safetensors"))
    assert "lm_head.weight" not in tied                           # tied: none is stored
    cfg = json.load(open(os.path.join(model_dirs["A"], "config.json")))
    assert cfg == TINY_A


@pytest.mark.parametrize("prefix", ["model.language_model.", "language_model.", "model.", ""])
def test_every_prefix_loads(model_dirs, tmp_path, prefix):
    def edit(t):
        return {(n if n == "lm_head.weight" else prefix + n[len("model.language_model."):]): v for n, v in t.items()}
    folder = _rewrite(model_dirs["B"], str(tmp_path / "p"), edit)
    cfg, model = load_model(folder, "float32", "cpu")
    assert model.embedding.weight.shape == (512, 192)
    assert model.blocks[0].mixer.qkv_proj.weight.shape == ((6 + 2) * 32, 192)
    assert model.blocks[0].mixer.qkv_proj.bias.dtype == torch.float32


def test_vision_tensors_are_ignored_and_tied_head(model_dirs, tmp_path):
    def edit(t):
        t["visual.blocks.0.attn.qkv.weight"] = torch.zeros(4, 4)
        t["model.visual.merger.ln_q.weight"] = torch.zeros(4)
    folder = _rewrite(model_dirs["A"], str(tmp_path / "v"), edit)
    _, model = load_model(folder, "float32", "cpu")
    assert model.head.proj.weight.data_ptr() == model.embedding.weight.data_ptr()     # tied: one table

    def with_head(t):
        t["lm_head.weight"] = torch.full((256, 64), 0.5)
    folder = _rewrite(model_dirs["A"], str(tmp_path / "h"), with_head)
    _, model = load_model(folder, "float32", "cpu")
    assert float(model.head.proj.weight[0, 0]) == 0.5              # an explicit head wins over the tie


def test_one_error_lists_everything(model_dirs, tmp_path):
    def edit(t):
        del t["model.language_model.layers.1.mlp.up_proj.weight"]
        del t["model.language_model.norm.weight"]
        t["model.language_model.layers.0.extra.weight"] = torch.zeros(2)
        t["model.language_model.layers.2.self_attn.k_proj.bias"] = torch.zeros(33)
        t["model.language_model.layers.0.self_attn.o_proj.weight"] = torch.zeros(192, 192).to(torch.int32)
    folder = _rewrite(model_dirs["B"], str(tmp_path / "bad"), edit)
    with pytest.raises(WeightsError) as err:
        load_model(folder, "float32", "cpu")
    e = err.value
    assert e.missing == ["layers.1.mlp.up_proj.weight", "norm.weight"]
    assert e.unexpected == ["model.language_model.layers.0.extra.weight"]
    assert len(e.wrong_shape) == 2 and "k_proj.bias" in str(e) and "[33]" in str(e) and "[32]" in str(e)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "up_proj", "extra.weight"):
        assert word in str(e)


def test_untied_model_needs_its_head(model_dirs, tmp_path):
    def edit(t):
        del t["lm_head.weight"]
    folder = _rewrite(model_dirs["B"], str(tmp_path / "nohead"), edit)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_model(folder, "float32", "cpu")


def test_dtypes_kept(model_dirs, tmp_path):
    from tiny_models import make_model_dir
    bf = make_model_dir(tmp_path, "A", "bfloat16")
    _, m = load_model(bf, "bfloat16", "cpu")
    assert m.embedding.weight.dtype == torch.bfloat16 and m.blocks[0].feed_forward.down_proj.weight.dtype == torch.bfloat16
    assert m.final_norm.weight.dtype == torch.float32             # vectors of float32 arithmetic stay 32-bit
    _, m32 = load_model(model_dirs["A"], "float32", "cpu")
    assert m32.embedding.weight.dtype == torch.float32
    assert m.position.axis.dtype == torch.int32                   # integer tables are int32


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_model(str(tmp_path), "float32", "cpu")
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(str(tmp_path), "float32", "cpu")


def test_sharded_folder_with_an_index(model_dirs, tmp_path):
    """``model.safetensors.index.json`` naming two shards (src/qwen25vl_lite/model.py:312-327): every
    tensor is found in whichever shard holds it, and a tensor in no shard is reported missing."""
    src = SafetensorsFile(os.path.join(model_dirs["B"], "model.safetensors"))
    names = src.names()
    half = len(names) // 2
    folder = tmp_path / "sharded"
    os.makedirs(folder)
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, part in shards.items():
        write_safetensors(str(folder / fname), [(n, src.tensor(n).clone()) for n in part])
    with open(folder / "model.safetensors.index.json", "w") as fh:
        json.dump({"metadata": {}, "weight_map": {n: f for f, part in shards.items() for n in part}}, fh)
    with open(os.path.join(model_dirs["B"], "config.json")) as a, open(folder / "config.json", "w") as b:
        b.write(a.read())
    _, sharded = load_model(str(folder), "float32", "cpu")
    _, single = load_model(model_dirs["B"], "float32", "cpu")
    for a, b in zip(sharded.blocks, single.blocks):
        assert torch.equal(a.mixer.qkv_proj.weight, b.mixer.qkv_proj.weight)
        assert torch.equal(a.feed_forward.down_proj.weight, b.feed_forward.down_proj.weight)
    assert torch.equal(sharded.head.proj.weight, single.head.proj.weight)
    os.remove(folder / "model-00002-of-00002.safetensors")
    write_safetensors(str(folder / "model-00002-of-00002.safetensors"), [(n, src.tensor(n).clone()) for n in names[half:-1]])
    with pytest.raises(WeightsError, match="missing tensors"):
        load_model(str(folder), "float32", "cpu")
