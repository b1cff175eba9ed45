"""Matrix products of the forward pass: ``y = x . W^T (+ b)``.

* float32: the engine's own FMA kernel (``csrc/gemm_f32.cu``), whose per-element summation
  order is fixed, so results do not depend on the batch.  No library, no TF32.
* bfloat16, at most 64 rows (decode steps): the engine's weight-streaming kernel
  (``csrc/gemm_skinny.cu``, mma.sync with the weights on the 16-row side).
* bfloat16, more rows: the library product (cuBLAS through ``torch.mm`` / ``torch.addmm``)
  with float32 accumulation.  The reference's engine uses the same library for every
  projection (``nn.Linear``, src/qwen25vl_lite/text.py:61-63,80-83; src/qwen25vl_lite/model.py:84).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import kernels


class Linear:
    """A weight [N, K] (and optional float32 bias [N]) held on the device for ``y = x W^T + b``."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        # the library path adds the bias in the activation dtype
        self._bias_lib = None if bias is None or weight.dtype == torch.float32 else bias.to(weight.dtype)

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        w = self.weight
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear: input width {x.shape[-1]} does not match weight {tuple(w.shape)}")
        if w.dtype == torch.float32:
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
            kernels.gemm_f32(x, w, self.bias, out)
            return out
        if kernels.gemm_skinny_supports(x, w):
            f32 = out_dtype == torch.float32
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32 if f32 else w.dtype, device=x.device)
            if f32 and self.bias is None:
                kernels.gemm_skinny(x, w, None, out, kernels.SKINNY_F32)
                return out
            if not f32:
                kernels.gemm_skinny(x, w, self.bias, out, kernels.SKINNY_BIAS if self.bias is not None else kernels.SKINNY_STORE)
                return out
        if out_dtype is not None and out_dtype != w.dtype:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
            if self.bias is not None:
                y += self.bias.to(out_dtype)
            return y
        if self._bias_lib is not None:
            return torch.addmm(self._bias_lib, x, w.t())
        return torch.mm(x, w.t())
