"""Token embedding and output head.

Embedding: x[t] = E[token[t]] (* scale when the plan gives one), into the float32 residual
stream (src/qwen.rs:669-672: no scale).  Head: logits = h @ W.T in float32, for the rows that
are asked for only (src/qwen.rs:632-638); its weight may be the embedding's tensor (tied,
src/qwen.rs:472-485)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part
from .linear import Linear


class Embedding(Part):
    category = "embedding"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.scale = spec.params.get("scale") or 1.0
        self.table = None

    def wants(self):
        return {"weight": TensorWant((self.vocab_size, self.hidden_size), "matrix")}

    def load(self, tensors):
        self.table = tensors["weight"].contiguous()

    def kernel_units(self):
        return [("elementwise", ())]

    def forward(self, ctx, tokens, out):
        kernels.embed_gather(self.table, tokens, out, float(self.scale))


class LinearHead(Part):
    category = "head"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.proj = None

    def wants(self):
        return {"weight": TensorWant((self.vocab_size, self.hidden_size), "matrix")}

    def load(self, tensors):
        self.proj = Linear(tensors["weight"])

    def kernel_units(self):
        return kernels.gemm_units(self.compute)

    def forward(self, ctx, h):
        with kernels.profile_category("lm_head"):
            return self.proj(h, out_dtype=torch.float32)

    def weight_bytes(self):
        return self.proj.bytes()


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)
