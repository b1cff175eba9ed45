"""The replay program's side of its protocol, with a stand-in for the runner (no GPU): one line
``done <step>`` after every step, a file only for steps that want logits, rows in the order of the
entries and of ``want``, requests opened at their first step and given back at ``end``, and the
kernels' error flag looked at before a step's logits count."""

import io
import json

import numpy as np
import pytest
import torch

from qwen25vl_lite.engine import trace


class FakeRunner:
    device = torch.device("cpu")

    def __init__(self, vocab=7):
        self.vocab, self.opened, self.closed, self.calls, self.checks = vocab, [], [], [], 0
        self.fail_check_at = None

    def open_request(self, rid):
        self.opened.append(rid)
        return rid

    def close_request(self, req):
        self.closed.append(req)

    def step(self, entries):
        self.calls.append([(e.request, list(e.tokens), list(e.want), e.positions) for e in entries])
        rows = [[float(tok)] * self.vocab for e in entries for tok in (e.tokens[w] for w in e.want)]
        return torch.tensor(rows, dtype=torch.float32) if rows else None

    def check_kernel_errors(self):
        self.checks += 1
        if self.fail_check_at == self.checks:
            raise RuntimeError("a kernel gave up a wait")


def lines(*records):
    return [json.dumps(r) for r in records]


def test_steps_files_and_done_lines(tmp_path):
    runner, reply = FakeRunner(), io.StringIO()
    trace.replay(lines(
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [9], "want": []}, {"id": "b", "tokens": [4, 6], "want": [1]}], "end": ["a"]},
        {"step": 2, "entries": [], "end": ["b"]},
    ) + ["", "   "], runner, str(tmp_path), reply)
    assert reply.getvalue() == "done 0\ndone 1\ndone 2\n"
    assert runner.opened == ["a", "b"] and runner.closed == ["a", "b"] and runner.checks == 3
    assert sorted(p.name for p in tmp_path.iterdir()) == ["0.f32", "1.f32"]
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(-1, runner.vocab)
    got1 = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(-1, runner.vocab)
    assert got0[:, 0].tolist() == [5.0, 3.0] and got1[:, 0].tolist() == [6.0]      # entries in order, then ``want`` in order
    assert runner.calls[1][0][:3] == ("a", [9], []) and runner.calls[1][1][:3] == ("b", [4, 6], [1])


def test_positions_travel_and_an_unknown_request_cannot_end(tmp_path):
    runner = FakeRunner()
    session = trace.TraceSession(runner, str(tmp_path))
    session.run_step({"step": 0, "entries": [{"id": "x", "tokens": [1, 2], "want": [1], "positions": [[0, 1], [0, 0], [0, 0]]}]})
    assert runner.calls[0][0][3].tolist() == [[0, 1], [0, 0], [0, 0]]
    with pytest.raises(ValueError, match="not live"):
        session.run_step({"step": 1, "entries": [], "end": ["nobody"]})


def test_logits_of_a_step_whose_kernels_gave_up_are_not_written(tmp_path):
    runner = FakeRunner()
    runner.fail_check_at = 1
    with pytest.raises(RuntimeError):
        trace.replay(lines({"step": 0, "entries": [{"id": "a", "tokens": [1], "want": [0]}], "end": []}), runner, str(tmp_path),
                     io.StringIO())
    assert list(tmp_path.iterdir()) == []


def test_the_pool_size_must_be_whole_pages_of_64():
    with pytest.raises(ValueError, match="multiple of 64"):
        trace.make_runner("nowhere", "float32", 100)
    with pytest.raises(ValueError, match="divide 64"):
        trace.make_runner("nowhere", "float32", 128, page_size=24)
