"""Python face of the CUDA kernels: each function checks its tensors and launches one kernel
on torch's current stream through ctypes.

There is no fallback: on a machine without the built library, or when a launch fails, the
call raises.  Tensors are torch CUDA tensors used as typed device buffers; nothing here
calls a torch operator on the data.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .build import build_library

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_LL = ctypes.c_longlong

_SIGNATURES = {
    "q25_embed_gather": [_P, _P, _P, _I, _I, _I, _P],
    "q25_add_rmsnorm": [_P, _P, _P, _F, _P, _P, _I, _I, _P],
    "q25_silu_mul": [_P, _P, _I, _I, _I, _P],
    "q25_rope_store": [_P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "q25_paged_attention_generic": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
}
_UNTYPED = {
    "q25_attention_decode_bf16": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "q25_attention_prefill_bf16": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
    "q25_gemm_f32": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "q25_gemm_tcgen05_bf16": [_P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "q25_sample_rows": [_P, _LL, _I, _I, _P, _P, _P, _P, _P, _P],
    "q25_apply_penalties": [_P, _LL, _I, _I, _P, _P, _P, _P, _P, _P, _P],
}

_SUFFIX = {torch.float32: "_f32", torch.bfloat16: "_bf16"}
_libs: Dict[str, ctypes.CDLL] = {}
_fns: Dict[str, object] = {}


class KernelError(RuntimeError):
    pass


def load_library(name: str = "core") -> ctypes.CDLL:
    """Builds (first use) and loads a kernel library; raises if that is not possible."""
    lib = _libs.get(name)
    if lib is None:
        path = build_library(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise KernelError(f"cannot load the CUDA kernel library {path}: {exc}") from exc
        _libs[name] = lib
    return lib


# symbols of the tensor-core kernels, which only the bfloat16 path loads (and so compiles)
_BF16_SYMBOLS = ("q25_attention_decode", "q25_attention_prefill", "q25_gemm_chain", "q25_gemm_tcgen05",
                 "q25_rope_angles")


def _fn(symbol: str, argtypes, library: Optional[str] = None):
    if _chain and symbol not in _CHAIN_SAFE:
        chain_flush()                       # products that wait in the chain come before this kernel
    f = _fns.get(symbol)
    if f is None:
        lib = load_library(library or ("bf16" if symbol.startswith(_BF16_SYMBOLS) else "core"))
        try:
            f = getattr(lib, symbol)
        except AttributeError as exc:
            raise KernelError(f"the kernel library has no symbol {symbol}") from exc
        f.argtypes = argtypes
        f.restype = _I
        _fns[symbol] = f
    return f


def _typed(base: str, dtype: torch.dtype):
    try:
        return _fn(base + _SUFFIX[dtype], _SIGNATURES[base])
    except KeyError:
        raise KernelError(f"{base}: unsupported dtype {dtype}") from None


_launches = 0
_sm_count: Dict[int, int] = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once (148 on the B200 the kernels'
    heuristics were measured on); grids and split counts are derived from it."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    n = _sm_count.get(dev)
    if n is None:
        n = int(_fn("q25_sm_count", [], "core")()) if dev >= 0 else 148
        if n <= 0:
            raise KernelError("cannot read the device's multiprocessor count")
        _sm_count[dev] = n
    return n


def chain_grid() -> int:
    """CTAs of the chain kernel (one per SM); its barrier counter advances by this per barrier."""
    return int(_fn("q25_gemm_chain_grid", [])())


def launch_count() -> int:
    """How many kernels of this engine have been launched by this process."""
    return _launches


def count_replayed(n: int) -> None:
    """Launches that ran from a captured graph (they do not pass through ``_check``)."""
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"CUDA kernel {what} could not be launched: cudaError {code} "
                          f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _dev(t: torch.Tensor, dtype: torch.dtype, what: str) -> torch.Tensor:
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise KernelError(f"{what}: needs a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}, "
                          f"contiguous={t.is_contiguous()}")
    return t


# ---------------------------------------------------------------------------------------------


def embed_gather(table: torch.Tensor, ids: torch.Tensor, x_out: torch.Tensor) -> None:
    """x_out[n, :] (float32) = table[ids[n], :]."""
    n, hidden = x_out.shape
    _dev(ids, torch.int32, "embed_gather ids"); _dev(x_out, torch.float32, "embed_gather out")
    _check(_typed("q25_embed_gather", table.dtype)(table.data_ptr(), ids.data_ptr(), x_out.data_ptr(), n, hidden,
                                                   table.shape[0], _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (when given); out = rmsnorm(x) * weight.  With ``rows`` only those rows are
    normalised into out[0..len(rows)) and x is left as it is."""
    hidden = x.shape[-1]
    n_out = out.shape[0]
    _dev(x, torch.float32, "add_rmsnorm x"); _dev(weight, torch.float32, "add_rmsnorm weight")
    if delta is not None:
        _dev(delta, out.dtype, "add_rmsnorm delta")
    if rows is not None:
        _dev(rows, torch.int32, "add_rmsnorm rows")
    _check(_typed("q25_add_rmsnorm", out.dtype)(x.data_ptr(), _ptr(delta), weight.data_ptr(), float(eps),
                                                out.data_ptr(), _ptr(rows), n_out, hidden, _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False) -> None:
    """out = silu(gate) * up.  ``gate_up`` rows hold gate then up (halves), or with ``paired``
    groups of 8 gate features followed by their 8 up features."""
    n, inter = out.shape
    _dev(gate_up, out.dtype, "silu_mul input")
    if paired and inter % 8:
        raise KernelError(f"silu_mul: the paired layout needs a width that is a multiple of 8, got {inter}")
    _check(_typed("q25_silu_mul", out.dtype)(gate_up.data_ptr(), out.data_ptr(), n, inter, int(paired), _stream()),
           "silu_mul")


def rope_store(qkv: torch.Tensor, positions: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
               axis: Optional[torch.Tensor], k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               kv_slot: Optional[torch.Tensor], nq: int, nkv: int, head_dim: int, page_size: int,
               angles: Optional[torch.Tensor] = None) -> None:
    """Rotates q (in place) and k by the position encoding and writes k, v into the pages at
    ``kv_slot``.  positions None: no rotation; pages None: nothing stored.  ``angles``: what
    ``rope_angles`` made of these positions (float32 [N, D/2, 2]); given, the kernel reads the
    cosines and sines there instead of computing them again in every layer."""
    n = qkv.shape[0]
    rotate = positions is not None
    store = k_pages is not None
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (n, head_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError(f"rope_store: angles must be float32 [{n}, {head_dim // 2}, 2]")
    _check(_typed("q25_rope_store", qkv.dtype)(
        qkv.data_ptr(), _ptr(positions), n, _ptr(inv_freq), _ptr(axis), _ptr(k_pages), _ptr(v_pages), _ptr(kv_slot),
        nq, nkv, head_dim, page_size, int(rotate), int(store), _ptr(angles), _stream()), "rope_store")


def paged_attention_generic(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, token_seq: torch.Tensor, cu_q: torch.Tensor,
                            q_start_pos: torch.Tensor, nq: int, nkv: int, head_dim: int, page_size: int,
                            window: int, scale: float) -> None:
    n = qkv.shape[0]
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    _check(_typed("q25_paged_attention_generic", qkv.dtype)(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), cu_q.data_ptr(), q_start_pos.data_ptr(), n, nq, nkv, head_dim,
        page_size, int(window or 0), float(scale), _stream()), "paged_attention_generic")


def attention_mma_supports(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Sizes the tensor-core attention kernels take; everything else goes to the general kernel."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and page_size > 0 and page_size & (page_size - 1) == 0)


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, items: torch.Tensor,
                     nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float, n_splits: int,
                     scratch: Optional[torch.Tensor]) -> None:
    """Tensor-core attention for the entries listed in ``items`` (int32 entry indices), each
    of which brings exactly one token.  With ``n_splits`` > 1 the keys of an entry are cut
    into that many ranges whose partial results go through ``scratch`` (float32, at least
    ``len(items) * nq * n_splits * (head_dim + 2)`` elements)."""
    n_items = items.shape[0]
    if nq // nkv > 16:
        raise KernelError("attention_decode: more than 16 query heads per kv head; use attention_prefill")
    if n_splits > 1:
        need = n_items * nq * n_splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode: {n_splits} splits need {need} float32 of scratch memory")
    _check(_fn("q25_attention_decode_bf16", _UNTYPED["q25_attention_decode_bf16"])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), items.data_ptr(), n_items, nq, nkv, head_dim,
        page_size, int(window or 0), float(scale), int(n_splits), _ptr(scratch), _stream()), "attention_decode")


def attention_fused_supports(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    return attention_mma_supports(dtype, head_dim, page_size) and head_dim % 32 == 0 and group <= 16


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, items: torch.Tensor,
                           nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float, n_splits: int,
                           positions: torch.Tensor, inv_freq: torch.Tensor, axis: torch.Tensor,
                           kv_slot: torch.Tensor, scratch: Optional[torch.Tensor] = None,
                           angles: Optional[torch.Tensor] = None, dense: bool = False) -> None:
    """One kernel for a step of one-token entries: rotary encoding of q and the new k
    (``positions`` int32 [axes, N], ``inv_freq`` float32 [D/2], ``axis`` int32 [D/2]), the write of
    the new k and v at ``kv_slot``, attention, and the merge of the ``n_splits`` key ranges
    (through ``scratch`` as for ``attention_decode``; the CTA that finishes last merges).
    ``qkv`` is read as projected and left unchanged.  ``angles``: the step's table from
    ``rope_angles`` (the kernel computes the angles itself without it).
    ``dense``: ``items`` is 0 .. n-1 and every entry has exactly one token (the kernel then skips two look-ups)."""
    n_items = items.shape[0]
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (positions.shape[1], head_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError("attention_decode_fused: angles must be float32 [N, D/2, 2]")
    if n_splits > 1:
        need = n_items * nq * n_splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode_fused: {n_splits} splits need {need} float32 of scratch memory")
    if not attention_fused_supports(qkv.dtype, head_dim, page_size, nq // nkv) or n_splits < 1:
        raise KernelError(f"attention_decode_fused: unsupported head size {head_dim}, page size {page_size}, "
                          f"group {nq // nkv} or splits {n_splits}")
    if positions.dtype != torch.int32 or positions.dim() != 2 or (angles is None and positions.shape[0] != 3):
        raise KernelError("attention_decode_fused: positions must be int32 [axes, N]; without an angle table the kernel "
                          "computes the angles itself and reads three axes")
    _check(_fn("q25_attention_decode_fused_bf16",
               [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), items.data_ptr(), items.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), int(n_splits), positions.data_ptr(), positions.shape[1],
        inv_freq.data_ptr(), axis.data_ptr(), kv_slot.data_ptr(), _ptr(scratch),
        _split_counters(qkv.device, n_items * nkv).data_ptr(), _ptr(angles), int(bool(dense)),
        _stream()), "attention_decode_fused")


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, axis: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of every token's rotary angles, float32 [N, D/2, 2]: ``positions`` int32 [axes, N],
    ``inv_freq`` float32 [D/2], ``axis`` int32 [D/2] (which position axis drives each channel)."""
    n, half = positions.shape[1], inv_freq.shape[0]
    _dev(positions, torch.int32, "rope_angles positions"); _dev(inv_freq, torch.float32, "rope_angles inv_freq")
    _dev(axis, torch.int32, "rope_angles axis")
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(_fn("q25_rope_angles", [_P, _I, _P, _P, _I, _P, _P])(
        positions.data_ptr(), n, inv_freq.data_ptr(), axis.data_ptr(), half, out.data_ptr(), _stream()), "rope_angles")
    return out


_counters: Dict[torch.device, torch.Tensor] = {}


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed ints the fused decode attention counts its finished splits in (it leaves them zero)."""
    buf = _counters.get(device)
    if buf is None or buf.numel() < n:
        buf = _counters[device] = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
    return buf


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, tiles: torch.Tensor,
                      nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float) -> None:
    """Tensor-core attention for runs of tokens.  ``tiles`` is int32 [n, 2]: (entry, row
    tile), a row tile being 64 consecutive rows of the entry's (token, head of the kv group)
    pairs, token-major."""
    _check(_fn("q25_attention_prefill_bf16", _UNTYPED["q25_attention_prefill_bf16"])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), _stream()), "attention_prefill")


def attention_tcgen05_supports(dtype: torch.dtype, head_dim: int, page_size: int, qkv: Optional[torch.Tensor] = None) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 128, a page size that is a power
    of two, 16-byte aligned rows."""
    if dtype != torch.bfloat16 or head_dim != 128 or page_size < 1 or page_size & (page_size - 1):
        return False
    return qkv is None or (qkv.data_ptr() % 16 == 0 and qkv.stride(0) % 8 == 0 and qkv.stride(1) == 1)


def attention_prefill_tcgen05(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                              block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor,
                              tiles: torch.Tensor, nq: int, nkv: int, head_dim: int, page_size: int, window: int,
                              scale: float, merges: Optional[torch.Tensor] = None,
                              scratch: Optional[torch.Tensor] = None, pairs: bool = False) -> None:
    """``attention_prefill`` on the tcgen05 tensor cores (scores, P and the outputs in tensor memory).
    ``tiles`` is int32 [n, 3]: (entry, row tile, code) with row tiles of 128 rows; code 1 is a whole
    tile, else first part << 8 | part << 4 | parts: one of the parts its keys are cut into, which
    leaves unnormalised sums in ``scratch`` (float32, room for n * nkv * 128 * (head_dim + 2)).
    ``merges`` is int32 [m, 4]: (entry, row tile, first part, parts) of the cut tiles, which a second
    kernel adds up.  ``pairs``: every piece of work goes to a cluster of two CTAs instead; code 2 then
    means half of the keys for each, added up through the cluster's shared memory, code 1 the whole
    tile for one of them."""
    if not attention_tcgen05_supports(qkv.dtype, head_dim, page_size, qkv):
        raise KernelError(f"attention_prefill_tcgen05: unsupported head size {head_dim}, page size {page_size} or layout")
    if tiles.dim() != 2 or tiles.shape[1] != 3:
        raise KernelError("attention_prefill_tcgen05: the work list is (entry, row tile, code) triples")
    n_merge = 0 if merges is None else merges.shape[0]
    if n_merge and (pairs or scratch is None or scratch.dtype != torch.float32
                    or scratch.numel() < tiles.shape[0] * nkv * 128 * (head_dim + 2)):
        raise KernelError("attention_prefill_tcgen05: cut tiles need float32 scratch for every piece of work, and no pairs")
    if pairs and window:
        raise KernelError("attention_prefill_tcgen05: keys behind a window are not cut")
    _check(_fn("q25_attention_prefill_tcgen05_bf16",
               [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P, _I, _P, _P])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), _ptr(merges), n_merge, _ptr(scratch), int(bool(pairs)),
        error_flag(qkv.device).data_ptr(), _stream()), "attention_prefill_tcgen05")
    if n_merge:
        count_replayed(1)                      # the merge kernel, launched by the same call


def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T + bias, plain float32 FMA."""
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"gemm_f32 {what}: needs a float32 CUDA matrix with unit inner stride")
    _check(_fn("q25_gemm_f32", _UNTYPED["q25_gemm_f32"])(
        a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k, a.stride(0), w.stride(0), out.stride(0),
        _stream()), "gemm_f32")


SKINNY_STORE, SKINNY_BIAS, SKINNY_F32, SKINNY_SWIGLU, SKINNY_RESIDUAL = 0, 1, 2, 3, 4
# Rows the weight-streaming kernel takes: the 8 batch columns of one m16n8k16 MMA.  A variant with two
# column tiles ran 9 to 16 rows; measured against the library path on B200 it lost at every size (a
# decode step of 9 / 12 / 16 requests at the 3B sizes 2.64 / 2.66 / 2.65 ms against 2.43 / 2.55 / 2.59,
# 14 layers of the 7B sizes 2.55 / 2.61 / 2.75 against 1.92 / 2.02 / 2.02 ms) and is gone.
SKINNY_MAX_ROWS = 8
_error_flags: Dict[torch.device, torch.Tensor] = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels with bounded waits set when a wait gave up."""
    device = torch.device(device)
    flag = _error_flags.get(device)
    if flag is None:
        flag = _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return flag


def gemm_skinny_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS
            and w.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = x . w^T for at most 8 rows of x, streaming the weights once (bfloat16).
    ``epilogue``: SKINNY_STORE, SKINNY_BIAS (float32 bias), SKINNY_F32 (float32 out),
    SKINNY_SWIGLU (w rows are groups of 8 gate + 8 up features; out has half as many columns)
    or SKINNY_RESIDUAL (out is float32 and the product is added into it).  Runs as an operation
    of the chain kernel (``csrc/gemm_chain.cu``): at once and alone, or, between ``chain_begin``
    and ``chain_end``, together with the products around it."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_skinny_supports(x, w) or w.shape[1] != k or not w.is_contiguous():
        raise KernelError(f"gemm_skinny: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _skinny_out(out, m, n, epilogue, "gemm_skinny")
    _chain_add(x, None, 0.0, w, bias, out, epilogue)


def _skinny_out(out: torch.Tensor, m: int, n: int, epilogue: int, what: str) -> None:
    cols = n // 2 if epilogue == SKINNY_SWIGLU else n
    want = torch.float32 if epilogue in (SKINNY_F32, SKINNY_RESIDUAL) else torch.bfloat16
    if out.shape != (m, cols) or out.dtype != want or out.stride(1) != 1:
        raise KernelError(f"{what}: output must be [{m}, {cols}] {want}")
    if epilogue == SKINNY_SWIGLU and n % 16:
        raise KernelError(f"{what}: the SwiGLU epilogue needs groups of 8 gate and 8 up rows, got {n} rows")


def gemm_skinny_norm_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_skinny_norm`` takes the float32 rows ``x`` (the residual stream) and ``w``."""
    return (x.dtype == torch.float32 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and 1 <= x.shape[0] <= SKINNY_MAX_ROWS and w.shape[1] % 32 == 0
            and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_skinny_norm(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor,
                     bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = (rmsnorm(x) * norm_weight) . w^T with the normalisation done inside the kernel;
    x is float32 [M <= 8, K], everything else as for ``gemm_skinny``."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_skinny_norm_supports(x, w) or w.shape[1] != k:
        raise KernelError(f"gemm_skinny_norm: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _dev(norm_weight, torch.float32, "gemm_skinny_norm norm weight")
    _skinny_out(out, m, n, epilogue, "gemm_skinny_norm")
    _chain_add(x, norm_weight, eps, w, bias, out, epilogue)


# ---- chains of weight-streaming products -------------------------------------------------------
# Every weight-streaming product is an operation of the chain kernel (``csrc/gemm_chain.cu``).  Outside
# ``chain_begin`` / ``chain_end`` each runs at once as a chain of one.  Between them the products are
# not launched one by one: they wait in a list, and the list runs as ONE persistent kernel as soon
# as any other kernel of this module is asked for, so that the order of all kernels is the order of
# the calls.  Only kernels of this module may be launched meanwhile; whoever runs a library operator
# on the stream in between calls ``chain_flush`` first.


class _ChainOpDesc(ctypes.Structure):
    """One product of a chain as ``csrc/gemm_chain.cu`` reads it (``ChainOpDesc``)."""
    _fields_ = [("W", _P), ("X", _P), ("norm_w", _P), ("bias", _P), ("out", _P), ("ldx", _I), ("ldo", _I), ("M", _I),
                ("N", _I), ("K", _I), ("epi", _I), ("norm", _I), ("eps", _F), ("reserved", _I)]


CHAIN_MAX_OPS = 8
_chain_base = 0                           # value of the barrier counter when the next chain kernel begins
_CHAIN_SAFE = {"q25_gemm_chain_bf16", "q25_gemm_chain_scratch_floats", "q25_gemm_chain_available", "q25_gemm_chain_desc_bytes",
               "q25_gemm_chain_grid", "q25_sm_count"}
_chain: Optional[list] = None             # the waiting products: (description, tensors kept alive)
_chain_state: Dict[torch.device, tuple] = {}
_chain_scratch: Dict[torch.device, list] = {}


_chain_ok: Optional[bool] = None


def chain_available() -> bool:
    """Whether the chain kernel can run here: a CUDA device that holds its whole grid at once."""
    global _chain_ok
    if _chain_ok is None:
        if not torch.cuda.is_available():
            return False
        ok = bool(_fn("q25_gemm_chain_available", [])())
        if ok and _fn("q25_gemm_chain_desc_bytes", [])() != ctypes.sizeof(_ChainOpDesc):
            raise KernelError("gemm_chain: the operation description here and in the library differ in layout")
        _chain_ok = ok
    return _chain_ok


def chain_begin() -> bool:
    """Starts gathering.  The counter of the kernels' barrier starts from zero in every gathering
    (a memset on the stream), so the values that a captured graph carries hold in every replay."""
    global _chain, _chain_base
    if _chain is None and chain_available():
        _chain, _chain_base = [], 0
        device = torch.device("cuda", torch.cuda.current_device())
        _chain_buffers(device)[1].zero_()
    return _chain is not None


def _chain_buffers(device: torch.device):
    state = _chain_state.get(device)
    if state is None:
        state = _chain_state[device] = (torch.zeros(65536, dtype=torch.int32, device=device),
                                        torch.zeros(1, dtype=torch.int32, device=device))
    return state


def chain_end() -> None:
    global _chain
    if _chain is not None:
        chain_flush()
        _chain = None


def _chain_add(x, norm_weight, eps, w, bias, out, epilogue) -> None:
    if not chain_available():
        raise KernelError("the weight-streaming kernel needs a device that holds its whole grid at once (one CTA per SM)")
    desc = _ChainOpDesc(W=w.data_ptr(), X=x.data_ptr(), norm_w=_ptr(norm_weight), bias=_ptr(bias), out=out.data_ptr(),
                        ldx=x.stride(0), ldo=out.stride(0), M=x.shape[0], N=w.shape[0], K=w.shape[1], epi=int(epilogue),
                        norm=0 if norm_weight is None else 1, eps=float(eps))
    entry = (desc, (x, norm_weight, w, bias, out))
    if _chain is None:
        _chain_launch([entry])                # nobody is gathering: a chain of one
        return
    _chain.append(entry)
    if len(_chain) == CHAIN_MAX_OPS:
        chain_flush()


def _chain_launch(waiting) -> None:
    global _chain_base
    device = next(t for t in waiting[0][1] if t is not None).device
    ops = (_ChainOpDesc * len(waiting))(*[w_[0] for w_ in waiting])
    need = _fn("q25_gemm_chain_scratch_floats", [_P, _I])
    need.restype = ctypes.c_longlong
    floats = need(ctypes.cast(ops, _P), len(waiting))
    if floats < 0:
        raise KernelError("gemm_chain: a product of the chain cannot be cut")
    held = _chain_scratch.setdefault(device, [])       # never freed or moved: captured graphs keep the addresses
    if not held or held[-1].numel() < max(floats, 1):
        held.append(torch.empty(max(floats, 1), dtype=torch.float32, device=device))
    counters, barrier = _chain_buffers(device)
    _check(_fn("q25_gemm_chain_bf16", [_P, _I, _P, _P, _P, ctypes.c_uint, _P, _P])(
        ctypes.cast(ops, _P), len(waiting), held[-1].data_ptr(), counters.data_ptr(), barrier.data_ptr(),
        _chain_base, error_flag(device).data_ptr(), _stream()), "gemm_chain")
    _chain_base = (_chain_base + (len(waiting) - 1) * chain_grid()) & 0xFFFFFFFF


def chain_flush() -> None:
    """Runs the products that wait, in order, as one kernel."""
    global _chain
    if not _chain:
        return
    waiting, _chain = _chain, None            # the launch below must not gather again
    try:
        _chain_launch(waiting)
    finally:
        _chain = []


def gemm_tcgen05_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Operands the tcgen05 / TMA product takes: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = x . w^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory), for
    any number of rows; epilogues as for ``gemm_skinny``."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_tcgen05_supports(x, w) or w.shape[1] != k:
        raise KernelError(f"gemm_tcgen05: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _skinny_out(out, m, n, epilogue, "gemm_tcgen05")
    _check(_fn("q25_gemm_tcgen05_bf16", _UNTYPED["q25_gemm_tcgen05_bf16"])(
        w.data_ptr(), x.data_ptr(), x.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), m, n, k, int(epilogue),
        error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05")


def reset_after_error(device) -> None:
    """After a bounded wait gave up: the error flag, and every flag or counter that kernels leave
    zero when they finish normally, back to zero."""
    device = torch.device(device)
    for table in (_error_flags, _counters):
        if device in table:
            table[device].zero_()
    if device in _chain_state:
        for t in _chain_state[device]:
            t.zero_()


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
                token_index: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or temperature is None), else a
    draw from softmax(logits[r] / temperature[r]) keyed by (seed[r], token_index[r])."""
    rows, vocab = logits.shape
    _dev(out, torch.int32, "sample_rows out")
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 rows")
    # a large vocabulary is scanned by several blocks per row; their partial winners need scratch
    chunks = _fn("q25_sample_chunks", [_I, _I])(rows, vocab)
    scratch = torch.empty(2 * rows * chunks, dtype=torch.int32, device=logits.device) if chunks > 1 else None
    _check(_fn("q25_sample_rows", _UNTYPED["q25_sample_rows"])(
        logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _ptr(token_index),
        out.data_ptr(), _ptr(scratch), _stream()), "sample_rows")


def apply_penalties(logits: torch.Tensor, ids: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _check(_fn("q25_apply_penalties", _UNTYPED["q25_apply_penalties"])(
        logits.data_ptr(), logits.stride(0), rows, vocab, ids.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
        repetition.data_ptr(), presence.data_ptr(), frequency.data_ptr(), _stream()), "apply_penalties")
