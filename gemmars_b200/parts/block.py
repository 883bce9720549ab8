"""The arrangement of a layer's parts.

``prenorm`` (src/qwen.rs:682-696): x += mixer(norm(x)); x += ffn(norm(x)), the residual stream
``x`` in float32.  Another arrangement (post-norm, parallel branches, a third norm) is another
class like this one, registered under its own kind and reading its own part names from the
layer's spec."""
from __future__ import annotations

from .. import kernels
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

    #: forward takes ``h_in`` / ``next_norm`` and returns what its last product left for the next block's first norm
    chains_norms = True

    def first_norm(self):
        """The norm that reads the residual first: the block before may be asked to feed it."""
        return self.mixer_norm

    def forward(self, ctx, x, caches, writes_cache=True, h_in=None, next_norm=None):
        """Runs the layer on ``x`` in place.  In decode steps the RMSNorms are taken into the
        products around them where the parts can (kernels.UnscaledRows): ``h_in`` is what the block
        before left for this block's first norm (None: the norm runs by itself), ``next_norm`` the
        first norm of the block after; returns what the feed-forward's last product left for it."""
        mine = self.split_caches(caches)
        linking = (kernels.NORM_LINKS and self.compute == "bfloat16" and ctx.n_tokens <= kernels.LINK_MAX_TOKENS)
        h = h_in if h_in is not None else self.mixer_norm.forward(ctx, x)
        left = None
        if getattr(self.mixer, "links_norms", False):
            then = self.ffn_norm if linking and getattr(self.ffn_norm, "linkable", False) else None
            left = self.mixer.forward(ctx, h, x, mine["mixer"], writes_cache, then_norm=then)
        else:
            self.mixer.forward(ctx, _plain(h), x, mine["mixer"], writes_cache)
        h = left if left is not None else self.ffn_norm.forward(ctx, x)
        if getattr(self.ffn, "links_norms", False):
            then = next_norm if linking and getattr(next_norm, "linkable", False) else None
            return self.ffn.forward(ctx, h, x, then_norm=then)
        self.ffn.forward(ctx, _plain(h), x)
        return None


def _plain(h):
    return h.materialize() if isinstance(h, kernels.UnscaledRows) else h


register_part("block", "prenorm", PreNormBlock)
