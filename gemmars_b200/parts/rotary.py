"""Rotary position encoding (rotate-half) over the first ``rotary_dim`` dims of each head.

inv_freq[i] = float32(1 / theta^(2i / rotary_dim)), computed in float64 (src/qwen.rs:529-533);
angle = float32(position) * inv_freq[i] in float32 (src/kernels.rs:1525-1531);
(a, b) = (v[i], v[i + half]) -> (a cos - b sin, b cos + a sin) (src/kernels.rs:1538-1548).

The attention part fuses this rotation into its q/k kernel when its position encoding is this
class; ``apply`` is the stand-alone form with the same kernel."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, register_part


class Rotary(Part):
    category = "position"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary: cannot rotate {self.rotary_dim} of {self.head_dim} dimensions")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self._inv_freq_host = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                               2.0 * i / max(self.rotary_dim, 1))).to(torch.float32)
        self._inv_freq = {}

    def inv_freq(self, device) -> torch.Tensor:
        t = self._inv_freq.get(device)
        if t is None:
            t = self._inv_freq[device] = self._inv_freq_host.to(device)
        return t

    def kernel_units(self):
        return [("elementwise", ())]

    def table(self, ctx) -> torch.Tensor:
        """(cos, sin) of the step's packed tokens' angles, [tokens, rotary_dim / 2, 2] float32,
        computed once a step and shared by every layer with the same rotation."""
        key = ("rope_table", self.rotary_dim, self.theta)
        t = ctx.extras.get(key)
        if t is None:
            t = ctx.extras[key] = kernels.rope_table(ctx.tok_pos, self.inv_freq(ctx.device))
        return t

    def apply(self, ctx, q, k):
        """Rotates q [T, nh, hd] and k [T, nkv, hd] (contiguous views) in place."""
        for x in (q, k):
            t, heads, hd = x.shape
            flat = x.view(t, heads * hd)
            # all heads are treated as "q" heads of one tensor: rotate in place, scale 1
            kernels.head_norm_rope_cache(flat, heads, 0, hd, self.rotary_dim, None, None, 0.0,
                                         self.inv_freq(x.device), 1.0, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                                         None, ctx.page_size, None, None,
                                         kernels.FLAG_ROPE | kernels.FLAG_INPLACE)


register_part("position", "rotary", Rotary)
