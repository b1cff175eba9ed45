"""Matrix products of the forward pass: ``y = x . W^T (+ b)``.

* float32: the engine's own FMA kernel (``csrc/gemm_f32.cu``), whose per-element summation
  order is fixed, so results do not depend on the batch.  No library, no TF32.
* bfloat16, at most 8 rows (decode steps): the engine's weight-streaming kernel
  (``csrc/gemm_chain.cu``).  It can normalise its input on the fly (a ``DeferredNorm``)
  and add its result into the float32 residual stream, which removes the norm kernels and
  the separate residual additions from a decode step, and it runs the products of a step
  that follow one another as operations of one launch.
* bfloat16, 128 rows or more (prefill): the engine's tcgen05 product
  (``csrc/gemm_tcgen05.cu``: TMA loads, accumulators in tensor memory) with the same
  epilogues, or the library product (cuBLAS through ``torch.mm`` / ``torch.addmm``), which the
  reference's engine uses for every projection (``nn.Linear``,
  src/qwen25vl_lite/text.py:61-63,80-83; src/qwen25vl_lite/model.py:84); see ``use_tcgen05``.
  Batches of 9 to 127 rows (but for the largest gate/up products) and operands the tcgen05
  kernel refuses (K not a multiple of 8, unaligned rows) go to the library.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import kernels

# The tcgen05 kernel works in tiles of 128 rows; with fewer rows (decode batches of 9 to 127
# requests) the product is a stream of the weights, and it takes only the large ones (see below).
TCGEN05_MIN_ROWS = 128


def use_tcgen05(x: torch.Tensor, w: torch.Tensor, fused_epilogue: bool = False) -> bool:
    """Which kernel takes a product of more than 8 rows.  Measured on B200:

    * 2,048 rows (prefill, 3B sizes): the engine's tcgen05 kernel (pairs of CTAs from 256 rows on)
      reaches 1.22 PFLOP/s on the wide products where cuBLAS reaches 1.46-1.48 (at the 7B sizes
      1.72 on gate/up), and on the narrow ones (qkv, o: 80 and 64 tiles of 256 x 256 for 74 pairs of
      SMs) 0.64-0.79 against 1.2.  So it takes the products where its fused epilogue saves a kernel
      and a round trip through memory (gate_up with SwiGLU: about 150 us against 125 + 75 us), and
      the library the others;
    * 9 to 127 rows (decode steps of that many requests): the products are streams of the weights.
      One CTA per SM takes one tile of all rows x ``bn`` features, ``bn`` picked so that the tiles
      fill the SMs once; the stream then runs at the copy bandwidth, but launch, the first trip to
      memory and the epilogue (about 8 us together) are not hidden behind anything, where the
      library's smaller tiles overlap one another (3 us).  With the SwiGLU epilogue fused, against
      library product + SiLU-mul kernel: 23 against 19 to 23 us at the 3B sizes (45 M weights),
      53 against 51 / 54 / 58 us at 32 / 64 / 98 rows at 7B (136 M), 94 to 98 against 101 to 111 us
      at 32B (283 M).  So it takes gate_up from 64 rows at 2**27 weights and from 9 rows at 2**28.
      A stream-K variant (units of (tile, K block) dealt evenly to all SMs, segment sums handed
      between CTAs in float and added in K order) was built and measured too: 12 / 9 / 26 / 18 us
      for qkv / o / gate_up / down at 17 rows of the 3B sizes against cuBLAS's 5 / 5 / 16 / 17 us.
      What it loses is not the stream but its tail: sums through L2, a counter, a poll, another
      pass, per product.  It is not kept."""
    if not fused_epilogue or not kernels.gemm_tcgen05_supports(x, w):
        return False
    rows, weights = x.shape[0], w.shape[0] * w.shape[1]
    return rows >= TCGEN05_MIN_ROWS or (rows >= 64 and weights >= 1 << 27) or (rows > kernels.SKINNY_MAX_ROWS and weights >= 1 << 28)


class DeferredNorm:
    """``rmsnorm(x) * weight`` that has not been computed yet: a product that can normalise
    inside its kernel takes it as it is, anything else calls ``materialize``."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: torch.dtype):
        self.x, self.weight, self.eps, self.dtype = x, weight, eps, dtype
        self.shape = x.shape
        self.device = x.device

    def materialize(self) -> torch.Tensor:
        out = torch.empty(self.x.shape, dtype=self.dtype, device=self.x.device)
        kernels.add_rmsnorm(self.x, None, self.weight, self.eps, out)
        return out


class Linear:
    """A weight [N, K] (and optional float32 bias [N]) held on the device for ``y = x W^T + b``."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        # the library path adds the bias in the activation dtype
        self._bias_lib = None if bias is None or weight.dtype == torch.float32 else bias.to(weight.dtype)

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None, residual: Optional[torch.Tensor] = None):
        """``x``: activations [M, K] or a ``DeferredNorm``.  With ``residual`` (float32 [M, N])
        the product is added into it and None is returned when the kernel at hand can do
        that; otherwise the product is returned and the caller adds it later."""
        w = self.weight
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear: input width {x.shape[-1]} does not match weight {tuple(w.shape)}")
        deferred = isinstance(x, DeferredNorm)
        if w.dtype == torch.bfloat16 and x.shape[0] <= kernels.SKINNY_MAX_ROWS:
            y = self._skinny(x, deferred, out_dtype, residual)
            if y is not NotImplemented:
                return y
        kernels.chain_flush()           # what follows is no chain product; products that wait come first
        if deferred:
            x = x.materialize()
        if w.dtype == torch.bfloat16 and use_tcgen05(x, w):
            return self._tcgen05(x, out_dtype, residual)
        if w.dtype == torch.float32:
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
            kernels.gemm_f32(x, w, self.bias, out)
            return out
        if out_dtype is not None and out_dtype != w.dtype:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
            if self.bias is not None:
                y += self.bias.to(out_dtype)
            return y
        if self._bias_lib is not None:
            return torch.addmm(self._bias_lib, x, w.t())
        return torch.mm(x, w.t())

    def _tcgen05(self, x, out_dtype, residual):
        w = self.weight
        m = x.shape[0]
        if residual is not None and self.bias is None:
            kernels.gemm_tcgen05(x, w, None, residual, kernels.SKINNY_RESIDUAL)
            return None
        if out_dtype == torch.float32:
            out = torch.empty((m, self.out_features), dtype=torch.float32, device=x.device)
            kernels.gemm_tcgen05(x, w, None, out, kernels.SKINNY_F32)
            if self.bias is not None:
                out += self.bias
            return out
        out = torch.empty((m, self.out_features), dtype=w.dtype, device=x.device)
        kernels.gemm_tcgen05(x, w, self.bias, out, kernels.SKINNY_BIAS if self.bias is not None else kernels.SKINNY_STORE)
        return out

    def _skinny(self, x, deferred: bool, out_dtype, residual):
        """The weight-streaming kernel with the epilogue the call asks for, or NotImplemented."""
        w = self.weight
        if deferred:
            if not kernels.gemm_skinny_norm_supports(x.x, w):
                return NotImplemented
        elif not kernels.gemm_skinny_supports(x, w):
            return NotImplemented
        m = x.shape[0]
        if residual is not None and self.bias is None:
            epilogue, out, result = kernels.SKINNY_RESIDUAL, residual, None
        elif out_dtype == torch.float32:
            if self.bias is not None:
                return NotImplemented
            out = torch.empty((m, self.out_features), dtype=torch.float32, device=x.device)
            epilogue, result = kernels.SKINNY_F32, out
        else:
            out = torch.empty((m, self.out_features), dtype=w.dtype, device=x.device)
            epilogue, result = (kernels.SKINNY_BIAS if self.bias is not None else kernels.SKINNY_STORE), out
        if deferred:
            kernels.gemm_skinny_norm(x.x, x.weight, x.eps, w, self.bias, out, epilogue)
        else:
            kernels.gemm_skinny(x, w, self.bias, out, epilogue)
        return result
