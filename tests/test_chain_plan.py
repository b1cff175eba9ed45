"""The chain kernel's host-side planner (``csrc/gemm_chain.cu: chain_plan``), without a GPU: the
file is compiled alone into a small library (a few seconds) and asked, through
``q25_gemm_chain_plan``, how it would cut chains of products on a device of 148 SMs.

What must hold for every chain it accepts: the slices of an operation cover its K exactly once in
whole k blocks, no operation asks for more CTAs than the device has SMs (the kernel's grid barrier
needs them all resident), the ring has at least two stages, and everything fits the 227 KB of
shared memory a CTA may take.  And what the measurements behind the planner decided for the sizes
of the released models.
"""

import ctypes
import os
import subprocess

import numpy as np
import pytest

from qwen25vl_lite.ops import build

SMS = 148
SMEM_LIMIT = 227 * 1024
EPI_STORE, EPI_BIAS, EPI_F32, EPI_SWIGLU, EPI_RESIDUAL = range(5)
_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class OpDesc(ctypes.Structure):
    _fields_ = [("W", _P), ("X", _P), ("norm_w", _P), ("bias", _P), ("out", _P), ("ldx", _I), ("ldo", _I), ("M", _I),
                ("N", _I), ("K", _I), ("epi", _I), ("norm", _I), ("eps", _F), ("reserved", _I)]


class PlanOp(ctypes.Structure):
    _fields_ = [(n, _I) for n in ("slices", "slice_k", "ctas", "groups", "seq", "xp")]


@pytest.fixture(scope="module")
def planner(tmp_path_factory):
    try:
        nvcc = build.find_nvcc()
    except build.BuildError:
        pytest.skip("nvcc not found")
    out = tmp_path_factory.mktemp("chain_plan") / "libchain_plan.so"
    cmd = [nvcc, "-O1", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           "-I", build.CSRC, os.path.join(build.CSRC, "gemm_chain.cu"), "-o", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    lib = ctypes.CDLL(str(out))
    assert lib.q25_gemm_chain_desc_bytes() == ctypes.sizeof(OpDesc)
    lib.q25_gemm_chain_plan.argtypes = [_P, _I, _I, _P, _P, _P, _P]

    def plan(ops, sms=SMS):
        """ops: (N, K, norm, epilogue) per operation, rows of x -> None or (smem, stages, pitch, x_off, [PlanOp])."""
        descs = (OpDesc * len(ops))()
        for d, (m, n, k, norm, epi) in zip(descs, ops):
            d.W, d.X, d.norm_w, d.bias, d.out = 256, 256, 256, 256, 256      # aligned, never read by the planner
            d.ldx, d.ldo, d.M, d.N, d.K, d.epi, d.norm, d.eps = k, n, m, n, k, epi, norm, 1e-6
        stages, pitch, x_off = _I(0), _I(0), _I(0)
        out_ops = (PlanOp * len(ops))()
        total = lib.q25_gemm_chain_plan(ctypes.cast(descs, _P), len(ops), sms, ctypes.byref(stages), ctypes.byref(pitch),
                                        ctypes.byref(x_off), ctypes.cast(out_ops, _P))
        return None if total == 0 else (total, stages.value, pitch.value, x_off.value, list(out_ops))

    return plan


def layer(m, hidden, qkv, inter):
    """The products of a decode layer in the order a step chains them."""
    return [(m, hidden, hidden, 0, EPI_RESIDUAL), (m, 2 * inter, hidden, 1, EPI_SWIGLU), (m, hidden, inter, 0, EPI_RESIDUAL),
            (m, qkv, hidden, 1, EPI_BIAS)]


def check(ops, got):
    total, stages, pitch, x_off, plan_ops = got
    assert 2 <= stages <= 24 and total <= SMEM_LIMIT and pitch % 128 == 64          # no bank conflicts between rows
    assert stages * 16 * pitch <= x_off                                             # the ring lies before x
    for (m, n, k, norm, epi), p in zip(ops, plan_ops):
        assert p.groups == -(-n // 16)
        assert p.slice_k % 32 == 0 and p.slice_k * 2 <= pitch
        assert (p.slices - 1) * p.slice_k < k <= p.slices * p.slice_k               # every slice has work, together they cover K
        assert p.seq in (0, 1, 2)
        if p.seq:
            assert 1 <= p.ctas <= min(SMS, p.groups)                                # every CTA walks the slices of its own groups
            assert p.seq == 1 or p.xp >= 2 * k                                      # x whole: a row holds all of K
            assert not (p.seq == 1 and norm)                                        # slices of x by plain copies only
        else:
            assert 1 <= p.ctas and p.ctas * p.slices <= SMS                         # slices x CTAs of a slice, all resident
        assert total >= x_off + 8 * (p.xp if p.seq != 1 else 2 * pitch)             # room for 8 rows of x (two buffers when sliced)


def test_plans_hold_their_invariants_over_many_shapes(planner):
    rng = np.random.default_rng(0)
    seen = set()
    for _ in range(400):
        hidden = int(rng.integers(2, 320)) * 32
        inter = int(rng.integers(2, 900)) * 32
        qkv = hidden + int(rng.integers(1, 64)) * 16
        m = int(rng.integers(1, 9))
        ops = layer(m, hidden, qkv, inter)
        ops = ops[: int(rng.integers(1, 5))] + ([(m, int(rng.integers(1, 10000)) * 16, hidden, 1, EPI_F32)] if rng.random() < 0.3 else [])
        got = planner(ops)
        assert got is not None, ops
        check(ops, got)
        seen.update(p.seq for p in got[4])
    assert seen == {0, 1, 2}                                                        # every way of cutting came up


def test_what_the_planner_does_at_the_released_sizes(planner):
    # 3B: everything but the down projection fits one slice; the down projection's 128 groups go to
    # 128 CTAs that take its six slices one after the other; a ring of two 65 KB stages
    total, stages, pitch, _, ops = planner(layer(8, 2048, 2560, 11008))
    assert (stages, pitch) == (2, 4160)
    assert [(p.slices, p.seq) for p in ops] == [(1, 0), (1, 0), (6, 1), (1, 0)] and ops[2].ctas == 128
    # 7B: the width of 3584 is cut in three and x stays whole (nothing to finish afterwards); the down
    # projection's 224 groups would leave half of the CTAs a second group alone, so its slices go
    # to different CTAs; four stages
    total, stages, pitch, _, ops = planner(layer(8, 3584, 4608, 18944))
    assert stages == 4 and [p.seq for p in ops] == [2, 2, 0, 2] and [p.slices for p in ops] == [3, 3, 16, 3]
    assert ops[2].ctas * ops[2].slices == 144
    # 32B: four stages of 45 KB
    total, stages, pitch, _, ops = planner(layer(8, 5120, 7168, 27648))
    assert stages == 4 and all(p.slice_k >= 1152 for p in ops)


def test_the_planner_refuses_what_the_kernel_cannot_run(planner):
    assert planner([(9, 2048, 2048, 0, EPI_STORE)]) is None             # more rows than an MMA has batch columns
    assert planner([(4, 2048, 2040, 0, EPI_STORE)]) is None             # K no multiple of 32
    assert planner([(4, 2056, 2048, 1, EPI_SWIGLU)]) is None            # SwiGLU pairs need whole groups of 16 rows
    assert planner([(4, 2048, 2048, 0, EPI_STORE)] * 9) is None         # more operations than a chain holds
    assert planner([(4, 2048, 2048, 0, EPI_STORE)], sms=0) is None
    # a device with fewer SMs still gets a plan whose CTAs all fit
    total, stages, pitch, _, ops = planner(layer(8, 2048, 2560, 11008), sms=64)
    assert all((p.ctas if p.seq else p.ctas * p.slices) <= 64 for p in ops)
