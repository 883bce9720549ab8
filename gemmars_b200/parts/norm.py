"""RMSNorm: out = x * (mean(x^2) + eps)^-1/2 * w, statistics in float32
(src/kernels.rs:1385-1392; the weight is used as stored, not as 1 + w: src/qwen.rs:343-346 with
src/config.rs:465-469).  Input: rows of the float32 residual stream; output: activations."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part


class RMSNorm(Part):
    category = "norm"
    #: the products around this norm may take it into themselves (kernels.UnscaledRows): its
    #: output is x * rstd(x) * weight with the weight as stored
    linkable = True

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def wants(self):
        return {"weight": TensorWant((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def kernel_units(self):
        return [("elementwise", ())]

    def weight_bytes(self):
        return 0 if self.weight is None else 4 * self.weight.numel()

    def forward(self, ctx, x, rows_index=None):
        rows = x.shape[0] if rows_index is None else rows_index.numel()
        out = torch.empty((rows, self.size), dtype=self.act_dtype, device=x.device)
        kernels.rmsnorm(x, self.weight, out, self.eps, rows_index)
        return out


register_part("norm", "rmsnorm", RMSNorm)
