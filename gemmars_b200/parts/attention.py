"""Causal grouped-query attention over the cache, with an optional RMSNorm per head on q and k,
a position encoding, an optional window and optional biases.

For one step (src/qwen.rs:704-794): q, k, v = h Wq^T, h Wk^T, h Wv^T (one product against the
stacked matrix); per head q = norm(q) -> position encoding -> * scale (the scale after the
rotation, src/qwen.rs:737-761), k = norm(k) -> position encoding; k and v are appended to the
cache (keys normed and rotated, values raw, src/qwen.rs:775-785); each query sees the keys
lo..p of its own sequence (src/model.rs:1187-1226); residual += o Wo^T.

All sizes and constants are parameters: hidden_size, num_heads, num_kv_heads, head_dim,
qk_norm, qk_norm_eps, bias, window, scale (None: head_dim ** -0.5), position (a PartSpec or
None), has_kv (False for a layer that only reads another layer's cache: it has no k and v
matrices and is given the other layer's keys and values).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import PAGE_SIZE, KVNeed
from .base import Part, TensorWant, build_part, register_part
from .linear import Linear
from .rotary import Rotary


class Attention(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("qk_norm_eps", 1e-6))
        self.bias = bool(p.get("bias", False))
        self.window = p.get("window")
        self.has_kv = bool(p.get("has_kv", True))
        scale = p.get("scale")
        self.scale = float(scale) if scale is not None else float(
            torch.tensor(float(self.head_dim), dtype=torch.float32).pow(-0.5))
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"attention: {self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention: head_dim {self.head_dim} is not supported by the kernels "
                             "(a multiple of 16 from 16 to 256)")
        pos = p.get("position")
        self.position = build_part("position", pos, compute) if pos is not None else None
        self.qkv = self.o = self.q_norm = self.k_norm = None

    # ---- weights
    def wants(self):
        h, nh, nkv, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        w = {"q": TensorWant((nh * hd, h)), "o": TensorWant((h, nh * hd))}
        if self.has_kv:
            w.update({"k": TensorWant((nkv * hd, h)), "v": TensorWant((nkv * hd, h))})
        if self.qk_norm:
            w["q_norm"] = TensorWant((hd,), "vector")
            if self.has_kv:
                w["k_norm"] = TensorWant((hd,), "vector")
        if self.bias:
            w.update({"q_bias": TensorWant((nh * hd,), "vector"), "o_bias": TensorWant((h,), "vector")})
            if self.has_kv:
                w.update({"k_bias": TensorWant((nkv * hd,), "vector"), "v_bias": TensorWant((nkv * hd,), "vector")})
        return w

    def load(self, t):
        names = ["q", "k", "v"] if self.has_kv else ["q"]
        bias = torch.cat([t[n + "_bias"] for n in names]) if self.bias else None
        self.qkv = Linear(torch.cat([t[n] for n in names], dim=0), bias)
        self.o = Linear(t["o"], t.get("o_bias") if self.bias else None)
        if self.qk_norm:
            self.q_norm = t["q_norm"].contiguous()
            self.k_norm = t["k_norm"].contiguous() if self.has_kv else self.q_norm

    def kernel_units(self):
        return (kernels.gemm_units(self.compute) + [("elementwise", ())]
                + kernels.attention_units(self.compute, self.head_dim))

    def cache_needs(self):
        return [KVNeed(self.num_kv_heads, self.head_dim, self.window)] if self.has_kv else []

    def weight_bytes(self):
        norms = sum(4 * t.numel() for t in (self.q_norm, self.k_norm if self.has_kv else None) if t is not None)
        return self.qkv.bytes() + self.o.bytes() + norms

    @property
    def capture_depends_on_length(self):
        # the decode kernel that splits the keys over CTAs sizes its split by the longest sequence;
        # the streaming kernel and the float32 kernel launch the same grid at every length
        return self.compute == "bfloat16" and not kernels.attention_decode_stream_usable(
            1, self.num_heads, self.num_kv_heads, self.head_dim, PAGE_SIZE)

    @staticmethod
    def _token_place(ctx, group):
        """(page, position in the page) of the step's tokens in ``group``'s cache, made once a step
        for all the layers of the group."""
        key = ("token_place", id(group))
        t = ctx.extras.get(key)
        if t is None:
            t = ctx.extras[key] = kernels.token_place(ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, group.page_table,
                                                      group.page_size)
        return t

    #: forward takes ``then_norm`` and may be given kernels.UnscaledRows for ``h``
    links_norms = True

    # ---- step
    def forward(self, ctx, h, residual, caches, writes_cache=True, then_norm=None):
        """``h``: the normed activations, or kernels.UnscaledRows (the norm before is taken into
        the q/k/v product).  ``then_norm``: the RMSNorm that reads the residual next; returns that
        norm's input where the o product could leave it, else None."""
        link = h if isinstance(h, kernels.UnscaledRows) else None
        if link is not None:
            h = link.rows
        nh, hd = self.num_heads, self.head_dim
        nkv = self.num_kv_heads if self.has_kv else 0
        group, kc, vc = caches[0]
        writes_cache = writes_cache and self.has_kv
        rotary = self.position is None or isinstance(self.position, Rotary)
        rot = self.position.rotary_dim if isinstance(self.position, Rotary) else 0
        if rotary and ctx.max_new <= 1 and kernels.gemm_qkv_usable(h, self.qkv.weight, nh, nkv, hd, rot):
            # a decode step with heads of 128: norm, rotation, scale and the cache write ride on the
            # q/k/v product's epilogue
            qkv = torch.empty((h.shape[0], self.qkv.out_features), dtype=h.dtype, device=h.device)
            kernels.gemm_qkv(h, self.qkv.weight, self.qkv.bias, qkv, nh, nkv, hd,
                             self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None, self.eps,
                             self.position.inv_freq(h.device) if rot else None, self.scale, ctx.tok_pos, ctx.tok_seq,
                             ctx.seq_slot, group.page_table if writes_cache else None, group.page_size,
                             kc if writes_cache else None, vc if writes_cache else None, link_in=link)
            att = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
            kernels.attention(ctx, qkv[:, :nh * hd], att, nh, kc, vc, group.page_table, group.page_size, self.window)
            return self.o.add_into(att, residual, then_norm)
        if link is not None and h.shape[0] > kernels.LINK_MAX_TOKENS:
            h, link = link.materialize(), None
        if (rotary and writes_cache == self.has_kv
                and kernels.gemm_qkv_prompt_usable(h, self.qkv.weight, nh, nkv, hd, rot, group.page_size)):
            # a prompt step with heads of 128: the same on the prompt product's epilogue; the queries
            # are all that is written out, keys and values go straight into the cache
            q = torch.empty((h.shape[0], nh * hd), dtype=h.dtype, device=h.device)
            kernels.gemm_qkv_prompt(h, self.qkv.weight, self.qkv.bias, q, nh, nkv, hd,
                                    self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None,
                                    self.eps, self.position.table(ctx) if rot else None, self.scale,
                                    self._token_place(ctx, group) if nkv else None, group.page_size,
                                    kc if nkv else None, vc if nkv else None)
            att = torch.empty_like(q)
            kernels.attention(ctx, q, att, nh, kc, vc, group.page_table, group.page_size, self.window)
            return self.o.add_into(att, residual, then_norm)
        qkv = self.qkv(link if link is not None else h)
        norm = kernels.FLAG_NORM if self.qk_norm else 0
        store = kernels.FLAG_CACHE if writes_cache else 0
        if ctx.max_new <= 1:
            store |= kernels.FLAG_SINGLE       # a decode step: one position of each sequence
        common = (ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, group.page_table, group.page_size,
                  kc if writes_cache else None, vc if writes_cache else None)
        if self.position is None or isinstance(self.position, Rotary):
            rope = kernels.FLAG_ROPE if self.position is not None else 0
            rot = self.position.rotary_dim if rope else 0
            inv_freq = self.position.inv_freq(h.device) if rope else None
            kernels.head_norm_rope_cache(qkv, nh, nkv, hd, rot, self.q_norm, self.k_norm, self.eps, inv_freq,
                                         self.scale, *common, norm | rope | store | kernels.FLAG_INPLACE)
        else:
            # another position encoding: norm, then the part's own apply, then scale and cache write
            if norm:
                kernels.head_norm_rope_cache(qkv, nh, nkv, hd, 0, self.q_norm, self.k_norm, self.eps, None, 1.0,
                                             *common[:5], None, None, norm | kernels.FLAG_INPLACE)
            t = qkv.shape[0]
            q_view = qkv[:, :nh * hd].view(t, nh, hd)
            k_view = qkv[:, nh * hd:(nh + nkv) * hd].view(t, nkv, hd)
            self.position.apply(ctx, q_view, k_view)
            kernels.head_norm_rope_cache(qkv, nh, nkv, hd, 0, None, None, self.eps, None, self.scale, *common,
                                         store | kernels.FLAG_INPLACE)
        att = torch.empty((qkv.shape[0], nh * hd), dtype=qkv.dtype, device=qkv.device)
        kernels.attention(ctx, qkv[:, :nh * hd], att, nh, kc, vc, group.page_table, group.page_size, self.window)
        return self.o.add_into(att, residual, then_norm)


register_part("mixer", "attention", Attention)
