"""The work lists the attention kernels walk (``ops/attention.py: plan_step``), on the CPU: every
row of every run of tokens lies in exactly one tile, single tokens are the decode kernel's, and the
tiles that see the most keys come first."""

from types import SimpleNamespace

import numpy as np
import pytest

from qwen25vl_lite.ops.attention import PREFILL_TILE_ROWS, plan_step


def host(q_lens, starts):
    return SimpleNamespace(q_lens=list(q_lens), starts=list(starts), n_tokens=int(sum(q_lens)), n_seqs=len(q_lens))


@pytest.mark.parametrize("group", [1, 2, 7, 8, 16])
def test_every_row_is_in_one_tile_and_single_tokens_are_decode_items(group):
    rng = np.random.default_rng(group)
    for _ in range(50):
        n = int(rng.integers(1, 12))
        q_lens = [int(rng.choice([1, 1, 2, 3, 17, 64, 65, 300])) for _ in range(n)]
        starts = [int(rng.integers(0, 5000)) for _ in range(n)]
        plan = plan_step(host(q_lens, starts), group)
        assert plan["decode_items"].dtype == np.int32
        assert list(plan["decode_items"]) == [i for i, q in enumerate(q_lens) if q == 1]
        for rows in PREFILL_TILE_ROWS:
            pairs = plan[f"tiles{rows}"].reshape(-1, 2)
            want = {(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(-(-q * group // rows))}
            assert len(pairs) == len(want) and {tuple(p) for p in pairs.tolist()} == want
            # heaviest first: the keys a tile's last row sees never grow along the list
            seen = [starts[i] + min((t + 1) * rows // group, q_lens[i]) for i, t in pairs.tolist()]
            reach = [starts[i] + (t + 1) * rows // group for i, t in pairs.tolist()]
            assert reach == sorted(reach, reverse=True) and all(s >= 1 for s in seen)


def test_a_group_wider_than_the_decode_kernels_rows_goes_with_the_runs():
    plan = plan_step(host([1, 1, 5], [10, 700, 0]), 24)                 # 24 query heads per kv head: more than 16 rows
    assert plan["decode_items"].size == 0
    pairs = plan["tiles64"].reshape(-1, 2).tolist()
    assert sorted(pairs) == [[0, 0], [1, 0], [2, 0], [2, 1]]            # 24 rows each, 120 rows for the run of five


def test_a_step_of_single_tokens_has_no_tiles():
    plan = plan_step(host([1] * 9, range(9)), 8)
    assert list(plan["decode_items"]) == list(range(9))
    assert plan["tiles64"].size == 0 and plan["tiles128"].size == 0
