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

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        kernels.gemm(x, self.weight, out, self.bias, accumulate=False)
        return out

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        """residual += x @ W.T (+ b); residual is float32."""
        kernels.gemm(x, self.weight, residual, self.bias, accumulate=True)

    def bytes(self) -> int:
        b = 0 if self.bias is None else self.bias.numel() * self.bias.element_size()
        return self.weight.numel() * self.weight.element_size() + b
