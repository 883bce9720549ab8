"""The arrangement of a layer's parts.

``prenorm`` (src/qwen.rs:682-696): x += mixer(norm(x)); x += ffn(norm(x)), the residual stream
``x`` in float32.  Another arrangement (post-norm, parallel branches) is another class here."""
from __future__ import annotations

from .base import Part, build_part, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, layer_spec, compute):
        self.compute = compute
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, compute)
        self.mixer = build_part("mixer", layer_spec.mixer, compute)
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm, compute)
        self.ffn = build_part("ffn", layer_spec.ffn, compute)

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def forward(self, ctx, x, cache, writes_cache=True):
        self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), x, cache, writes_cache)
        self.ffn.forward(ctx, self.ffn_norm.forward(ctx, x), x)


register_part("block", "prenorm", PreNormBlock)
