"""The work lists the attention kernels walk (``ops/attention.py: plan_step``), on the CPU: every
row of every run of tokens lies in exactly one tile, single tokens are the decode kernel's, and the
tiles that see the most keys come first."""

from types import SimpleNamespace

import numpy as np
import pytest

from qwen25vl_lite.ops.attention import KEY_TILE, MAX_PARTS, plan_step

PLACES = 148    # CTAs of the tcgen05 kernel at a time for one of two kv heads, on the device the engine is written for


def host(q_lens, starts):
    return SimpleNamespace(q_lens=list(q_lens), starts=list(starts), n_tokens=int(sum(q_lens)), n_seqs=len(q_lens))


@pytest.mark.parametrize("group", [1, 2, 7, 8, 16])
def test_every_row_is_in_one_tile_and_single_tokens_are_decode_items(group):
    rng = np.random.default_rng(group)
    for _ in range(50):
        n = int(rng.integers(1, 12))
        q_lens = [int(rng.choice([1, 1, 2, 3, 17, 64, 65, 300])) for _ in range(n)]
        starts = [int(rng.integers(0, 5000)) for _ in range(n)]
        plan = plan_step(host(q_lens, starts), group, places=PLACES)
        assert plan["decode_items"].dtype == np.int32
        assert list(plan["decode_items"]) == [i for i, q in enumerate(q_lens) if q == 1]
        pairs = plan["tiles64"].reshape(-1, 2)
        want = {(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(-(-q * group // 64))}
        assert len(pairs) == len(want) and {tuple(p) for p in pairs.tolist()} == want
        # heaviest first: the keys a tile's last row sees never grow along the list
        reach = [starts[i] + (t + 1) * 64 // group for i, t in pairs.tolist()]
        assert reach == sorted(reach, reverse=True)
        # tiles of 128 rows: whole, every part of a cut tile once, or (for clusters of two CTAs) codes 1 and 2
        want = {(i, t) for i, q in enumerate(q_lens) if q > 1 for t in range(-(-q * group // 128))}
        if plan["pairs128"].size:
            triples = plan["tiles128"].reshape(-1, 3).tolist()
            assert plan["merge128"].size == 0 and len(triples) == len(want) and {(i, t) for i, t, _ in triples} == want
            assert {code for _, _, code in triples} <= {1, 2}
            continue
        triples = plan["tiles128"].reshape(-1, 3).tolist()
        assert {(i, t) for i, t, _ in triples} == want
        whole = [(i, t) for i, t, code in triples if code == 1]
        cut = {}
        for i, t, code in triples:
            if code != 1:
                cut.setdefault((i, t), []).append(code)
        assert len(whole) == len(set(whole)) and not set(whole) & set(cut)
        merges = plan["merge128"].reshape(-1, 4).tolist()
        assert {(i, t) for i, t, _, _ in merges} == set(cut)
        taken = []
        for i, t, first, parts in merges:
            assert 2 <= parts <= MAX_PARTS
            assert sorted(cut[(i, t)]) == [(first << 8) | (p << 4) | parts for p in range(parts)]
            taken += list(range(first, first + parts))
        assert sorted(taken) == list(range(len(taken))) and len(taken) <= len(triples)      # the scratch has a place for each


def walks_of(plan, q_lens, starts, group):
    """Key tiles each piece of work of the tcgen05 kernel walks, as the kernel derives them."""
    walks = []
    for i, t, code in plan["tiles128"].reshape(-1, 3).tolist():
        n = (starts[i] + min((t * 128 + 127) // group, q_lens[i] - 1)) // KEY_TILE + 1
        parts, part = code & 15, (code >> 4) & 15
        per = -(-n // parts)
        walks.append(min(n, (part + 1) * per) - part * per)
    return walks


def test_few_long_tiles_are_cut_to_fill_the_places_once():
    q_lens, starts = [512], [3000]
    whole = sum((3000 + min(t * 16 + 15, 511)) // KEY_TILE + 1 for t in range(32))
    plan = plan_step(host(q_lens, starts), 8, places=PLACES)
    walks = walks_of(plan, q_lens, starts, 8)
    assert plan["pairs128"].size == 0
    assert len(walks) > 2 * 32 and len(walks) <= PLACES                  # more pieces, one round of CTAs
    assert min(walks) >= 1 and sum(walks) == whole and walks == sorted(walks, reverse=True)
    assert max(walks) <= -(-55 // (len(walks) // 32)) + 1
    # more tiles than three quarters of the places, short walks, a window (a part could hold no key a row sees),
    # no places given: whole tiles
    for q, s, kw in (([2048], [0], {}), ([4096], [0], {}), ([128], [0], {}), ([512], [3000], dict(window=300)), ([512], [3000], dict(places=0))):
        plan = plan_step(host(q, s), 8, **{**dict(places=PLACES), **kw})
        assert plan["merge128"].size == 0 and plan["pairs128"].size == 0
        assert all(code == 1 for code in plan["tiles128"].reshape(-1, 3)[:, 2])


def test_steps_that_fill_up_to_three_quarters_of_the_places_go_to_pairs_of_ctas():
    """1,024 tokens after 1,024 are 64 row tiles of 17 to 32 key tiles: parts that fit the places
    would be as long as half a tile, so clusters of two CTAs halve every tile; 1,500 tokens are 94
    tiles, too many for parts."""
    for q, s in (([1024], [1024]), ([1500], [0]), ([1024], [0])):
        plan = plan_step(host(q, s), 8, places=PLACES)
        assert plan["pairs128"].size == 1 and plan["merge128"].size == 0
        triples = plan["tiles128"].reshape(-1, 3).tolist()
        walk = lambda t: (s[0] + min(t * 16 + 15, q[0] - 1)) // KEY_TILE + 1
        assert all(code == (2 if walk(t) >= 6 else 1) for _, t, code in triples)
        halves = [-(-walk(t) // 2) if code == 2 else walk(t) for _, t, code in triples]
        assert halves == sorted(halves, reverse=True)


def test_a_group_wider_than_the_decode_kernels_rows_goes_with_the_runs():
    plan = plan_step(host([1, 1, 5], [10, 700, 0]), 24, places=PLACES)                 # 24 query heads per kv head: more than 16 rows
    assert plan["decode_items"].size == 0
    pairs = plan["tiles64"].reshape(-1, 2).tolist()
    assert sorted(pairs) == [[0, 0], [1, 0], [2, 0], [2, 1]]            # 24 rows each, 120 rows for the run of five


def test_a_step_of_single_tokens_has_no_tiles():
    plan = plan_step(host([1] * 9, range(9)), 8, places=PLACES)
    assert list(plan["decode_items"]) == list(range(9))
    assert plan["tiles64"].size == 0 and plan["tiles128"].size == 0
