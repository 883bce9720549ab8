"""Gated feed-forward: down(act(gate(x)) * up(x)), act = SiLU (src/qwen.rs:57-68,
silu(a) = a / (1 + exp(-a)) src/kernels.rs:1416-1426).  The gate and up matrices are stacked at
load into one [2I, H] matrix so one product reads the input once."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part
from .linear import Linear


class GatedMLP(Part):
    category = "ffn"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.hidden_size = int(spec.params["hidden_size"])
        self.intermediate_size = int(spec.params["intermediate_size"])
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation {act!r} has no kernel (known: silu)")
        self.gate_up = self.down = None

    def wants(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate": TensorWant((i, h)), "up": TensorWant((i, h)), "down": TensorWant((h, i))}

    def load(self, tensors):
        self.gate_up = Linear(torch.cat([tensors["gate"], tensors["up"]], dim=0))
        self.down = Linear(tensors["down"])

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("elementwise", ())]

    #: forward takes ``then_norm`` and may be given kernels.UnscaledRows for ``h``
    links_norms = True

    def forward(self, ctx, h, residual, then_norm=None):
        """``h``: the normed activations, or kernels.UnscaledRows.  ``then_norm``: the RMSNorm that
        reads the residual next; returns that norm's input where the down product could leave it."""
        rows = h.rows if isinstance(h, kernels.UnscaledRows) else h
        a = torch.empty((rows.shape[0], self.intermediate_size), dtype=rows.dtype, device=rows.device)
        kernels.gemm_swiglu(h, self.gate_up.weight, a)
        return self.down.add_into(a, residual, then_norm)

    def weight_bytes(self):
        return self.gate_up.bytes() + self.down.bytes()


register_part("ffn", "gated_mlp", GatedMLP)
