"""The decode-attention entry point that allocates nothing (csrc/attention_noalloc.h), called
through its exported C symbol and compared with the entry point that takes a scratch buffer.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
TOO_LARGE = -2
SCRATCH_FLOATS = 4 * 1024 * 1024


def _symbols():
    from qwen25vl_lite.ops import kernels
    lib = kernels.load_library("bf16")
    fn = lib.q25_attention_decode_bf16_noalloc
    fn.argtypes = [P, I, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    msg = lib.q25_attention_decode_noalloc_error
    msg.argtypes = []
    msg.restype = ctypes.c_char_p
    return fn, msg


def _case(seed, lens, nq, nkv, d, page_size):
    from test_kernels_gpu import paged_case
    rng = np.random.default_rng(seed)
    return paged_case(rng, lens, [1] * len(lens), nq, nkv, d, page_size, torch.bfloat16)


def _no_alloc(fn, c, n_items, nq, nkv, d, page_size, window, splits):
    out = torch.zeros((c["qkv"].shape[0], nq * d), dtype=torch.bfloat16, device="cuda")
    items = torch.arange(n_items, dtype=torch.int32, device="cuda")
    code = fn(c["qkv"].data_ptr(), c["qkv"].stride(0), out.data_ptr(), c["k_pages"].data_ptr(), c["v_pages"].data_ptr(),
              c["table"].data_ptr(), c["table"].shape[1], c["cu"].data_ptr(), c["start"].data_ptr(), items.data_ptr(),
              n_items, nq, nkv, d, page_size, window, d ** -0.5, splits, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, out


def _with_scratch(c, n_items, nq, nkv, d, page_size, window, splits):
    from qwen25vl_lite.ops import kernels
    out = torch.zeros((c["qkv"].shape[0], nq * d), dtype=torch.bfloat16, device="cuda")
    items = torch.arange(n_items, dtype=torch.int32, device="cuda")
    scratch = torch.empty(n_items * nq * splits * (d + 2), dtype=torch.float32, device="cuda") if splits > 1 else None
    kernels.attention_decode(c["qkv"], out, c["k_pages"], c["v_pages"], c["table"], c["cu"], c["start"], items,
                             nq, nkv, d, page_size, window, d ** -0.5, splits, scratch)
    torch.cuda.synchronize()
    return out


def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    fn, msg = _symbols()
    # two calls in a row, of different shapes, so that the second finds the first one's leftovers
    # in the shared array: 16 heads of 128 over 6 splits, then 6 heads of 32 over 3 splits, then
    # a call with a single split, which uses no scratch at all
    for seed, lens, nq, nkv, d, ps, window, splits in [
            (1, [700, 33, 1, 260], 16, 2, 128, 16, 0, 6),
            (2, [90, 301, 150], 6, 1, 32, 8, 100, 3),
            (3, [64, 65], 4, 2, 64, 16, 0, 1),
            (5, [2300, 17], 8, 2, 64, 16, 0, 70)]:       # more splits than a warp has lanes, twice over
        c = _case(seed, lens, nq, nkv, d, ps)
        code, got = _no_alloc(fn, c, len(lens), nq, nkv, d, ps, window, splits)
        assert code == 0, msg().decode()
        want = _with_scratch(c, len(lens), nq, nkv, d, ps, window, splits)
        diff = (got.float() - want.float()).abs().max().item()
        assert diff < 3e-2, f"no-alloc entry point differs from the allocating one by {diff}"
        from test_kernels_gpu import attention_oracle, f64
        assert np.abs(f64(got) - attention_oracle(c["dense"], window or None)).max() < 3e-2
        assert msg() == b""


def test_no_alloc_entry_point_refuses_more_scratch_than_it_holds():
    fn, msg = _symbols()
    c = _case(4, [40] * 4, 16, 2, 128, 16)
    # pretend 4096 entries: 4096 * 16 heads * 64 splits * 130 floats is far beyond the array
    need = 4096 * 16 * 64 * 130
    assert need > SCRATCH_FLOATS
    out = torch.zeros((4, 16 * 128), dtype=torch.bfloat16, device="cuda")
    items = torch.zeros(4096, dtype=torch.int32, device="cuda")
    code = fn(c["qkv"].data_ptr(), c["qkv"].stride(0), out.data_ptr(), c["k_pages"].data_ptr(), c["v_pages"].data_ptr(),
              c["table"].data_ptr(), c["table"].shape[1], c["cu"].data_ptr(), c["start"].data_ptr(), items.data_ptr(),
              4096, 16, 2, 128, 16, 0, 128 ** -0.5, 64, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert code == TOO_LARGE
    text = msg().decode()
    assert str(need) in text and str(SCRATCH_FLOATS) in text and "fewer splits" in text
    assert float(out.abs().max()) == 0.0                  # nothing was launched
