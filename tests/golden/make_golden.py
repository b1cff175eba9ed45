"""Makes tests/golden/*.npz: logits of the reference's own text decoder on the tiny models.

Run once, on a machine that has the reference checkout, from the repository root:

    python tests/golden/make_golden.py /path/to/qwen25vl-lite

It imports ``qwen25vl_lite.text.TextModel`` / ``qwen25vl_lite.rope.get_rope_index`` from
``<checkout>/src`` (CPU, float32), fills the model with the weights that this repository's
random-weights mode writes for tiny-A and tiny-B, runs the dense whole-sequence forward
with explicit position ids and stores, per model: the token ids, the position ids, and the
logits of every position.  tiny-B's prompt holds a 12-token image run (grid t1 x h3 x w4
after the 2x2 merge), whose positions come from the reference's ``get_rope_index``.
``tests/test_plain.py`` checks the plain implementation against these files.
"""

import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_reference(checkout):
    """Imports the reference package under the name ``qwen25vl_lite_reference``."""
    src = os.path.join(checkout, "src", "qwen25vl_lite")
    spec = importlib.util.spec_from_file_location("qwen25vl_lite_reference", os.path.join(src, "__init__.py"),
                                                  submodule_search_locations=[src])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["qwen25vl_lite_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    checkout = sys.argv[1]
    ref = load_reference(checkout)
    from qwen25vl_lite_reference.config import TextConfig
    from qwen25vl_lite_reference.rope import get_rope_index
    from qwen25vl_lite_reference.text import TextModel
    from safetensors import safe_open

    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from tiny_models import TINY, make_model_dir

    tmp = tempfile.mkdtemp()
    for name, n_tokens, image in (("A", 17, None), ("B", 40, (9, 1, 3, 4))):
        cfg_json, seed, _ = TINY[name]
        folder = make_model_dir(tmp, name)
        t = dict(cfg_json["text_config"])
        section = t.pop("rope_scaling")["mrope_section"]
        tcfg = TextConfig.from_dict({**t, "mrope_section": section, "tie_word_embeddings": cfg_json["tie_word_embeddings"]})
        model = TextModel(tcfg)
        state, head = {}, None
        with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key == "lm_head.weight":
                    head = f.get_tensor(key)
                else:
                    state[key[len("model.language_model."):]] = f.get_tensor(key)
        model.load_state_dict(state, strict=True)
        model.eval()
        if head is None:
            head = model.embed_tokens.weight
        rng = np.random.default_rng(100 + seed)
        ids = rng.integers(0, tcfg.vocab_size - 1, size=n_tokens)
        if image is None:
            pos, delta = get_rope_index(torch.tensor([ids.tolist()]), image_token_id=-1, video_token_id=-2,
                                        spatial_merge_size=2)
        else:
            start, gt, gh, gw = image
            image_id = tcfg.vocab_size - 1
            ids[start:start + gt * gh * gw] = image_id
            pos, delta = get_rope_index(torch.tensor([ids.tolist()]),
                                        image_grid_thw=torch.tensor([[gt, gh * 2, gw * 2]]),
                                        image_token_id=image_id, video_token_id=-2, spatial_merge_size=2)
        with torch.no_grad():
            hidden = model(model.embed_tokens(torch.tensor([ids.tolist()])), pos)
            logits = hidden[0] @ head.T
        out = os.path.join(HERE, f"tiny_{name}.npz")
        np.savez_compressed(out, token_ids=ids.astype(np.int64), positions=pos[:, 0].numpy().astype(np.int64),
                            rope_delta=np.int64(delta[0, 0].item()), logits=logits.numpy().astype(np.float32),
                            image=np.asarray(image if image else (-1, 0, 0, 0), dtype=np.int64))
        print(out, logits.shape, "rope_delta", int(delta[0, 0]))


if __name__ == "__main__":
    main()
