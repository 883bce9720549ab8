"""Plain, slow restatement of the Qwen3 dense decoder, for tests only.

Whole sequences, no cache, one function per part, NumPy only.  It shares no code with the
package: it reads ``config.json`` and ``model.safetensors`` with a few lines of its own.

It rests on the formulas of the reference project's Rust sources (cited per function as
``file:line`` within that project).  The reference's model code is Rust and no Rust toolchain
is available where this was written, so it could not be compiled or imported for a golden run;
every function below therefore cites the lines it restates.

Arithmetic is float64 by default (``dtype=np.float64``), except where the reference fixes a
32-bit intermediate that changes the value being computed: the rotation angle is the float32
product ``f32(pos) * f32(inv_freq)`` and ``inv_freq`` is computed in float64 then rounded to
float32, and ``eps`` and the query scale are the float32 values.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# --------------------------------------------------------------------------- model files

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path):
    """name -> float64 / int array.  Format: 8-byte little-endian header length, JSON header
    ``{name: {dtype, shape, data_offsets}}``, offsets relative to the end of the header
    (src/safetensors.rs:228-235, 272-317).  BF16 widens as ``bits << 16`` (src/kernels.rs:16-18)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[base + lo:base + hi]
        if info["dtype"] == "BF16":
            u = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(buf, dtype=_ST_DTYPES[info["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(info["shape"])
    return out


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- parts

def embedding(table, tokens):
    """x[t,:] = E[token[t],:], no scaling (src/qwen.rs:669-672, src/model.rs:103-110)."""
    return table[np.asarray(tokens, dtype=np.int64)].copy()


def rmsnorm(x, w, eps):
    """ss = sum(x^2)/n + eps; out = x * ss^-0.5 * w, with the plain weight (not 1+w) for the
    dense model (src/kernels.rs:1385-1392; src/qwen.rs:343-346; src/config.rs:465-469).
    eps is used as a 32-bit value (src/qwen.rs:663, 718)."""
    eps = float(np.float32(eps))
    ss = (x * x).sum(axis=-1, keepdims=True) / x.shape[-1] + eps
    return x * ss ** -0.5 * w


def linear(x, w, b=None):
    """y[t,o] = sum_i W[o,i] x[t,i] (src/kernels.rs:54-57); the optional bias has no
    counterpart in the reference's Qwen path and follows the checkpoint's ``attention_bias``."""
    y = x @ w.T
    return y if b is None else y + b


def rope_inv_freq(rot, theta):
    """inv_freq[i] = f32(1 / theta^(2i/rot)), computed in float64 then rounded
    (src/qwen.rs:529-533)."""
    i = np.arange(rot // 2, dtype=np.float64)
    return (1.0 / np.power(float(theta), 2.0 * i / rot)).astype(np.float32)


def rope_tables(positions, inv_freq):
    """angle = f32(p) * inv_freq[i] in float32; cos and sin of it (src/kernels.rs:1521-1534)."""
    ang = np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]
    assert ang.dtype == np.float32
    ang = ang.astype(np.float64)
    return np.cos(ang), np.sin(ang)


def apply_rope(v, cos, sin):
    """Rotate-half over the first 2*half dims of each head: a=v[i], b=v[i+half];
    v[i]=a*cos-b*sin, v[i+half]=b*cos+a*sin (src/kernels.rs:1538-1548); dims beyond the
    rotated ones pass through (src/qwen.rs:754-758).  v: [T, heads, hd]; cos, sin: [T, half]."""
    half = cos.shape[-1]
    out = v.copy()
    a = v[..., :half]
    b = v[..., half:2 * half]
    c = cos[:, None, :]
    s = sin[:, None, :]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


def softmax(s):
    """m = max; e = exp(s-m); p = e / sum(e) (src/kernels.rs:1550-1561)."""
    e = np.exp(s - s.max())
    return e / e.sum()


def attention(q, k, v, window=None):
    """Causal grouped-query attention over whole sequences.  The query at position p of head h
    uses kv head h // (nh/nkv) and sees keys lo..p inclusive, lo = max(0, p+1-window) with a
    window, else 0 (src/model.rs:1187-1226).  q: [T, nh, hd] already normed, rotated and
    scaled; k, v: [T, nkv, hd]."""
    t, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    out = np.zeros_like(q)
    for p in range(t):
        lo = 0 if window is None else max(0, p + 1 - window)
        for h in range(nh):
            g = h // rep
            s = k[lo:p + 1, g, :] @ q[p, h, :]
            out[p, h, :] = softmax(s) @ v[lo:p + 1, g, :]
    return out


def attention_block(hn, w, prefix, cfg, positions, window=None):
    """q/k/v projections, per-head RMSNorm on q and k, rotation, the hd^-0.5 scale folded into q
    after the rotation, attention, output projection (src/qwen.rs:704-794)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    t = hn.shape[0]
    bias = (lambda n: w.get(prefix + n + ".bias"))
    q = linear(hn, w[prefix + "q_proj.weight"], bias("q_proj")).reshape(t, nh, hd)
    k = linear(hn, w[prefix + "k_proj.weight"], bias("k_proj")).reshape(t, nkv, hd)
    v = linear(hn, w[prefix + "v_proj.weight"], bias("v_proj")).reshape(t, nkv, hd)
    rot = int(hd * cfg.get("partial_rotary_factor", 1.0))  # src/config.rs:498-506
    cos, sin = rope_tables(positions, rope_inv_freq(rot, cfg["rope_theta"]))
    scale = float(np.float32(hd) ** np.float32(-0.5))  # src/qwen.rs:737
    q = apply_rope(rmsnorm(q, w[prefix + "q_norm.weight"], eps), cos, sin) * scale
    k = apply_rope(rmsnorm(k, w[prefix + "k_norm.weight"], eps), cos, sin)
    att = attention(q, k, v, window).reshape(t, nh * hd)
    return linear(att, w[prefix + "o_proj.weight"], bias("o_proj"))


def silu(a):
    """silu(a) = a / (1 + exp(-a)) (src/kernels.rs:1416-1426)."""
    return a / (1.0 + np.exp(-a))


def mlp_block(hn, w, prefix):
    """down(silu(gate(x)) * up(x)) (src/qwen.rs:57-68)."""
    g = linear(hn, w[prefix + "gate_proj.weight"])
    u = linear(hn, w[prefix + "up_proj.weight"])
    return linear(silu(g) * u, w[prefix + "down_proj.weight"])


def layer_windows(cfg):
    """Per-layer window or None.  The reference's dense Qwen3 path is full attention in every
    layer (src/config.rs:465-469, src/qwen.rs:787); a checkpoint that sets ``use_sliding_window``
    names its windowed layers in ``layer_types`` ("sliding_attention") with ``sliding_window``
    keys each, applied as in src/model.rs:1199-1204."""
    n = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window") or not cfg.get("sliding_window"):
        return [None] * n
    types = cfg.get("layer_types") or ["full_attention"] * n
    return [cfg["sliding_window"] if t == "sliding_attention" else None for t in types]


def tensor_prefix(w):
    """The checkpoint's name prefix, probed on embed_tokens (src/qwen.rs:461-469)."""
    for p in ("model.language_model.", "model.", ""):
        if p + "embed_tokens.weight" in w:
            return p
    raise KeyError("cannot find embed_tokens in checkpoint")


def forward(cfg, w, tokens):
    """Logits [T, vocab] at every position of one whole sequence (src/qwen.rs:658-701, 632-638):
    pre-norm blocks, x += attn(norm(x)); x += mlp(norm(x)); final norm; lm_head, which is the
    embedding when tied or when lm_head.weight is absent (src/qwen.rs:472-485)."""
    p = tensor_prefix(w)
    eps = cfg["rms_norm_eps"]
    x = embedding(w[p + "embed_tokens.weight"], tokens)
    positions = np.arange(len(tokens))
    windows = layer_windows(cfg)
    for l in range(cfg["num_hidden_layers"]):
        lp = f"{p}layers.{l}."
        hn = rmsnorm(x, w[lp + "input_layernorm.weight"], eps)
        x = x + attention_block(hn, w, lp + "self_attn.", cfg, positions, windows[l])
        hn = rmsnorm(x, w[lp + "post_attention_layernorm.weight"], eps)
        x = x + mlp_block(hn, w, lp + "mlp.")
    xf = rmsnorm(x, w[p + "norm.weight"], eps)
    tied = cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in w
    head = w[p + "embed_tokens.weight"] if tied else w["lm_head.weight"]
    return linear(xf, head)


# --------------------------------------------------------------------------- sampling

def argmax(x):
    """First maximum (src/sampler.rs:125-135)."""
    best, bv = 0, -np.inf
    for i, v in enumerate(x):
        if v > bv:
            best, bv = i, v
    return best


class Sampler:
    """Greedy, or temperature + top-k + top-p with an xorshift64* generator
    (src/sampler.rs:3-126).  32-bit arithmetic as in the reference."""

    def __init__(self, temperature, top_k, top_p, seed):
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self.rng = max(int(seed), 1)  # src/sampler.rs:16

    def next_f32(self):
        """src/sampler.rs:20-30."""
        m = (1 << 64) - 1
        x = self.rng
        x ^= x >> 12
        x ^= (x << 25) & m
        x ^= x >> 27
        self.rng = x
        r = (x * 0x2545F4914F6CDD1D) & m
        return np.float32(r >> 40) / np.float32(1 << 24)

    def candidates(self, logits):
        """src/sampler.rs:43-84.  Ties are ordered by index here; the reference leaves their
        order open (unstable selection and sort)."""
        logits = np.asarray(logits, dtype=np.float32)
        k = len(logits) if self.top_k == 0 else min(self.top_k, len(logits))
        order = np.lexsort((np.arange(len(logits)), -logits))[:k]
        inv_t = np.float32(1.0) / np.float32(self.temperature)
        mx = logits[order[0]]
        probs = np.exp(((logits[order] - mx) * inv_t).astype(np.float32)).astype(np.float32)
        total = np.float32(0)
        for p in probs:
            total = np.float32(total + p)
        probs = (probs / total).astype(np.float32)
        cut = len(probs)
        if self.top_p < 1.0:
            acc = np.float32(0)
            for i, p in enumerate(probs):
                acc = np.float32(acc + p)
                if acc >= np.float32(self.top_p):
                    cut = i + 1
                    break
        tot = np.float32(0)
        for p in probs[:cut]:
            tot = np.float32(tot + p)
        return order, probs, cut, tot

    def sample(self, logits):
        """src/sampler.rs:109-122."""
        if self.temperature <= 0:
            return argmax(logits)
        idx, probs, cut, total = self.candidates(logits)
        r = np.float32(self.next_f32() * total)
        for i in range(cut):
            r = np.float32(r - probs[i])
            if r <= 0:
                return int(idx[i])
        return int(idx[cut - 1])


def generate(cfg, w, prompt, max_tokens, stop=(), temperature=0.0, top_k=64, top_p=0.95, seed=42):
    """Sample from the logits after the last token, append, stop after a stop token (kept in
    the output, not run) or max_tokens tokens (src/generate.rs:134-170).  Recomputes the whole
    sequence every step."""
    sampler = Sampler(temperature, top_k, top_p, seed)
    seq = list(prompt)
    out = []
    reason = "length"
    for _ in range(max_tokens):
        logits = forward(cfg, w, seq)[-1]
        tok = sampler.sample(logits.astype(np.float32))
        out.append(tok)
        if tok in stop:
            reason = "stop"
            break
        seq.append(tok)
    return out, reason
