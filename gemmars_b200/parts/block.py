"""The arrangement of a layer's parts.

``prenorm`` (src/qwen.rs:682-696): x += mixer(norm(x)); x += ffn(norm(x)), the residual stream
``x`` in float32.  Another arrangement (post-norm, parallel branches, a third norm) is another
class like this one, registered under its own kind and reading its own part names from the
layer's spec."""
from __future__ import annotations

from .base import Block, register_part


class PreNormBlock(Block):
    def __init__(self, layer_spec, compute):
        super().__init__(layer_spec, compute)
        self.mixer_norm = self.need("mixer_norm", "norm")
        self.mixer = self.need("mixer", "mixer")
        self.ffn_norm = self.need("ffn_norm", "norm")
        self.ffn = self.need("ffn", "ffn")

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def forward(self, ctx, x, caches, writes_cache=True):
        mine = self.split_caches(caches)
        self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), x, mine["mixer"], writes_cache)
        self.ffn.forward(ctx, self.ffn_norm.forward(ctx, x), x)


register_part("block", "prenorm", PreNormBlock)
