"""The shapes captured decode steps are given (``engine/runner.py``): few enough that a capture is
used again, and never smaller than the step."""

from qwen25vl_lite.engine.runner import GRAPH_WIDTH_STEP, graph_batch, graph_width


def test_graph_widths_grow_by_a_factor():
    widths = sorted({graph_width(p) for p in range(1, 5000)})
    assert widths[0] == GRAPH_WIDTH_STEP and all(w % 8 == 0 for w in widths)
    for a, b in zip(widths, widths[1:]):
        assert 1.3 <= b / a <= 1.5
    for p in range(1, 5000):
        w = graph_width(p)
        assert p <= w and (w == GRAPH_WIDTH_STEP or w < 1.5 * p + 1)
    assert len(widths) <= 20                                  # 80,000 tokens of context in under 20 shapes


def test_graph_batches_are_exact_up_to_8_rows_then_multiples():
    assert [graph_batch(n) for n in range(1, 9)] == list(range(1, 9))       # the chained products take these as they are
    assert [graph_batch(n) for n in (9, 16, 17, 24, 25, 63, 64)] == [16, 16, 24, 24, 32, 64, 64]
    assert [graph_batch(n) for n in (65, 80, 81, 127, 128, 129)] == [80, 80, 96, 128, 128, 144]
    for n in range(1, 600):
        b = graph_batch(n)
        assert n <= b < n + 16
    assert len({graph_batch(n) for n in range(1, 129)}) == 19
