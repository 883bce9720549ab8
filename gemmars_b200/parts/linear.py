"""A weight matrix with an optional bias and the product against it; the helper parts build
their projections from.  Not a part itself.

y[t, o] = sum_i W[o, i] x[t, i] (+ b[o])  (src/kernels.rs:54-57).  The product is written in the
activation precision, in float32 (logits), or added into the float32 residual stream.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight.contiguous()
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, x, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x @ W.T (+ b); ``x`` a tensor, or kernels.UnscaledRows (a norm taken into this product)."""
        rows = x.rows if isinstance(x, kernels.UnscaledRows) else x
        if out is None:
            out = torch.empty((rows.shape[0], self.out_features), dtype=out_dtype or rows.dtype, device=rows.device)
        kernels.gemm(x, self.weight, out, self.bias, accumulate=False)
        return out

    def add_into(self, x: torch.Tensor, residual: torch.Tensor, then_norm=None):
        """residual += x @ W.T (+ b); residual is float32.  ``then_norm``: the RMSNorm part that
        reads the residual next, if any; where the kernel can it leaves that norm's input
        (kernels.UnscaledRows), which is returned, else None and the norm runs by itself."""
        link = (then_norm.weight, then_norm.eps) if then_norm is not None else None
        return kernels.gemm(x, self.weight, residual, self.bias, accumulate=True, then_norm=link)

    def bytes(self) -> int:
        b = 0 if self.bias is None else self.bias.numel() * self.bias.element_size()
        return self.weight.numel() * self.weight.element_size() + b
