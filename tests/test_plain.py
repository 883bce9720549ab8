"""The plain implementation itself, on the CPU: each part against numbers worked out by hand from
the reference's formulas, and the properties that the whole model must have (a position sees
only what came before it; a window hides what is older; tied and untied heads).  These are what
the engine is compared with on the GPU, so they have to be right on their own."""
import math

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_configs import TINY_A, TINY_B


def _weights(cfg, seed=0):
    """Random float64 weights with the checkpoint's tensor names, made here (no package code)."""
    rng = np.random.default_rng(seed)
    h, nh, nkv, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    inter, v = cfg["intermediate_size"], cfg["vocab_size"]
    w = {"model.embed_tokens.weight": rng.standard_normal((v, h)) * 0.5,
         "model.norm.weight": 1 + 0.1 * rng.standard_normal(h)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = 1 + 0.1 * rng.standard_normal(h)
        w[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.standard_normal(h)
        for name, rows in (("q_proj", nh * hd), ("k_proj", nkv * hd), ("v_proj", nkv * hd)):
            w[p + f"self_attn.{name}.weight"] = rng.standard_normal((rows, h)) * 0.2
            if cfg.get("attention_bias"):
                w[p + f"self_attn.{name}.bias"] = rng.standard_normal(rows) * 0.1
        w[p + "self_attn.o_proj.weight"] = rng.standard_normal((h, nh * hd)) * 0.2
        if cfg.get("attention_bias"):
            w[p + "self_attn.o_proj.bias"] = rng.standard_normal(h) * 0.1
        w[p + "self_attn.q_norm.weight"] = 1 + 0.1 * rng.standard_normal(hd)
        w[p + "self_attn.k_norm.weight"] = 1 + 0.1 * rng.standard_normal(hd)
        w[p + "mlp.gate_proj.weight"] = rng.standard_normal((inter, h)) * 0.2
        w[p + "mlp.up_proj.weight"] = rng.standard_normal((inter, h)) * 0.2
        w[p + "mlp.down_proj.weight"] = rng.standard_normal((h, inter)) * 0.2
    if not cfg.get("tie_word_embeddings"):
        w["lm_head.weight"] = rng.standard_normal((v, h)) * 0.5
    return w


def test_rmsnorm_by_hand():
    # x = (3, 4): mean square 12.5; with eps 0.5: 13 -> x / sqrt(13) * w   (src/kernels.rs:1385-1392)
    out = plain.rmsnorm(np.array([[3.0, 4.0]]), np.array([2.0, 0.5]), 0.5)
    assert np.allclose(out, [[3 / math.sqrt(13) * 2, 4 / math.sqrt(13) * 0.5]], rtol=1e-7)
    # eps is the 32-bit value of what the configuration gives
    tiny = plain.rmsnorm(np.zeros((1, 4)) + 1e-30, np.ones(4), 1e-6)
    assert np.allclose(tiny, 1e-30 / math.sqrt(float(np.float32(1e-6))))


def test_rotation_by_hand_and_its_invariants():
    inv = plain.rope_inv_freq(4, 100.0)              # 1 / 100^(0/4), 1 / 100^(2/4)
    assert inv.dtype == np.float32 and np.allclose(inv, [1.0, 0.1])
    cos, sin = plain.rope_tables([0, 3], inv)
    assert np.allclose(cos[0], 1) and np.allclose(sin[0], 0)                      # position 0 turns nothing
    ang = np.float32(3) * inv                                                     # the angle is a float32 product
    assert np.allclose(cos[1], np.cos(ang.astype(np.float64))) and np.allclose(sin[1], np.sin(ang.astype(np.float64)))
    v = np.array([[[1.0, 2.0, 3.0, 4.0, 9.0]]] * 2)                               # 5 dims, 4 rotated: pairs (0,2), (1,3)
    out = plain.apply_rope(v, cos, sin)
    assert np.allclose(out[0], v[0])
    a0, a1 = ang.astype(np.float64)
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 9.0]
    assert np.allclose(out[1, 0], want)
    # a rotation keeps each pair's length, and q.k depends on the distance of the positions only
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    inv8 = plain.rope_inv_freq(8, 1e4)

    def dot(pq, pk):
        cq, sq = plain.rope_tables([pq], inv8)
        ck, sk = plain.rope_tables([pk], inv8)
        return float((plain.apply_rope(q, cq, sq) * plain.apply_rope(k, ck, sk)).sum())
    assert math.isclose(np.linalg.norm(plain.apply_rope(q, *plain.rope_tables([7], inv8))), np.linalg.norm(q), rel_tol=1e-12)
    assert math.isclose(dot(5, 2), dot(13, 10), rel_tol=1e-5)
    assert not math.isclose(dot(5, 2), dot(5, 3), rel_tol=1e-3)


def test_softmax_silu_and_gated_feed_forward_by_hand():
    p = plain.softmax(np.array([0.0, math.log(3.0)]))
    assert np.allclose(p, [0.25, 0.75]) and math.isclose(p.sum(), 1.0)
    big = plain.softmax(np.array([1000.0, 1000.0]))                               # the maximum is taken out first
    assert np.allclose(big, [0.5, 0.5])
    assert math.isclose(plain.silu(np.array(0.0)), 0.0) and math.isclose(plain.silu(np.array(2.0)), 2 / (1 + math.exp(-2)))
    w = {"m.gate_proj.weight": np.array([[1.0, 0.0], [0.0, 2.0]]), "m.up_proj.weight": np.array([[0.0, 1.0], [1.0, 1.0]]),
         "m.down_proj.weight": np.array([[1.0, -1.0]])}
    x = np.array([[1.0, 0.5]])                       # gate = (1, 1), up = (0.5, 1.5); silu(1) = 0.7310585786
    s1 = 1 / (1 + math.exp(-1))
    assert np.allclose(plain.mlp_block(x, w, "m."), [[s1 * 0.5 - s1 * 1.5]])


def test_attention_by_hand_causal_grouped_and_windowed():
    # two query heads on one kv head, two positions, head size 1
    q = np.array([[[1.0], [2.0]], [[1.0], [0.0]]])           # [T, nh, hd]
    k = np.array([[[0.0]], [[math.log(2.0)]]])
    v = np.array([[[10.0]], [[20.0]]])
    out = plain.attention(q, k, v)
    assert np.allclose(out[0], [[10.0], [10.0]])             # position 0 sees itself only
    # position 1, head 0: scores (0, ln 2) -> (1/3, 2/3); head 1: q = 0 -> (1/2, 1/2)
    assert np.allclose(out[1], [[10 / 3 + 40 / 3], [15.0]])
    assert np.allclose(plain.attention(q, k, v, window=1)[1], [[20.0], [20.0]])   # a window of 1: the position itself
    assert np.allclose(plain.attention(q, k, v, window=2), out)
    # grouped: with 4 query heads and 2 kv heads, heads 0,1 read kv head 0 and heads 2,3 kv head 1
    rng = np.random.default_rng(2)
    q4, k2, v2 = rng.standard_normal((3, 4, 2)), rng.standard_normal((3, 2, 2)), rng.standard_normal((3, 2, 2))
    full = plain.attention(q4, k2, v2)
    assert np.allclose(full[:, :2], plain.attention(q4[:, :2], k2[:, :1], v2[:, :1]))
    assert np.allclose(full[:, 2:], plain.attention(q4[:, 2:], k2[:, 1:], v2[:, 1:]))


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["A", "B"])
def test_a_position_sees_only_what_came_before(cfg):
    w = _weights(cfg, seed=3)
    rng = np.random.default_rng(4)
    toks = rng.integers(0, cfg["vocab_size"], 50).tolist()
    whole = plain.forward(cfg, w, toks)
    assert whole.shape == (50, cfg["vocab_size"])
    assert np.allclose(plain.forward(cfg, w, toks[:17]), whole[:17], rtol=1e-9, atol=1e-9)
    changed = list(toks)
    changed[30] = (changed[30] + 1) % cfg["vocab_size"]
    other = plain.forward(cfg, w, changed)
    assert np.allclose(other[:30], whole[:30], rtol=1e-9, atol=1e-9) and not np.allclose(other[30:], whole[30:])


def test_windowed_layers_forget_and_full_layers_do_not():
    cfg = dict(TINY_B, num_hidden_layers=1, layer_types=["sliding_attention"], sliding_window=8)
    w = _weights(cfg, seed=5)
    toks = np.random.default_rng(6).integers(0, cfg["vocab_size"], 30).tolist()
    base = plain.forward(cfg, w, toks)
    changed = [(toks[0] + 1) % cfg["vocab_size"]] + toks[1:]
    other = plain.forward(cfg, w, changed)
    # one windowed layer: position p sees p-7..p, so token 0 reaches positions 0..7 and no further
    assert not np.allclose(other[7], base[7]) and np.allclose(other[8:], base[8:], rtol=1e-9, atol=1e-9)
    full = dict(cfg, layer_types=["full_attention"])
    assert plain.layer_windows(full) == [None] and plain.layer_windows(cfg) == [8]
    assert not np.allclose(plain.forward(full, w, changed)[29], plain.forward(full, w, toks)[29])
    assert plain.layer_windows(dict(cfg, use_sliding_window=False)) == [None]


def test_tied_and_untied_heads_and_the_name_prefix():
    cfg = dict(TINY_A)
    w = _weights(cfg, seed=7)
    toks = [5, 9, 200]
    tied = plain.forward(cfg, w, toks)
    untied_cfg = dict(cfg, tie_word_embeddings=False)
    assert np.allclose(plain.forward(untied_cfg, w, toks), tied)          # no lm_head tensor: the embedding serves
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"] * 2
    assert np.allclose(plain.forward(untied_cfg, w2, toks), 2 * tied)
    assert np.allclose(plain.forward(cfg, w2, toks), tied)                # tied by configuration: lm_head ignored
    renamed = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v for k, v in w.items()}
    assert plain.tensor_prefix(renamed) == "model.language_model." and np.allclose(plain.forward(cfg, renamed, toks), tied)


def test_sampler_draws_as_the_reference_describes():
    assert plain.argmax(np.array([1.0, 3.0, 3.0, 2.0])) == 1                    # the first maximum
    logits = np.array([0.0, 2.0, 1.0, 2.0, -1.0], dtype=np.float32)
    assert plain.Sampler(0.0, 64, 0.95, 1).sample(logits) == 1                   # greedy when temperature <= 0
    assert plain.Sampler(1.0, 1, 1.0, 1).sample(logits) == 1                     # one candidate: the first of the largest
    s = plain.Sampler(1.0, 3, 1.0, 9)
    idx, probs, cut, total = s.candidates(logits)
    assert list(idx) == [1, 3, 2] and cut == 3                                   # decreasing logit, ties by token id
    e = np.exp(np.array([0.0, 0.0, -1.0]))
    assert np.allclose(probs, e / e.sum(), rtol=1e-6) and math.isclose(total, 1.0, rel_tol=1e-6)
    idx, probs, cut, total = plain.Sampler(1.0, 0, 0.5, 9).candidates(logits)    # top_k 0: all; top_p 0.5: the shortest prefix
    assert len(idx) == 5 and cut == 2 and math.isclose(total, float(probs[0] + probs[1]), rel_tol=1e-6)
    # the generator: xorshift64*, top 24 bits; seed 0 counts as 1; the same seed, the same draws
    a, b, z = plain.Sampler(1.0, 0, 1.0, 42), plain.Sampler(1.0, 0, 1.0, 42), plain.Sampler(1.0, 0, 1.0, 0)
    draws = [float(a.next_f32()) for _ in range(1000)]
    assert draws == [float(b.next_f32()) for _ in range(1000)] and all(0.0 <= u < 1.0 for u in draws)
    assert float(z.next_f32()) == float(plain.Sampler(1.0, 0, 1.0, 1).next_f32())
    x = 42
    x ^= x >> 12; x ^= (x << 25) & ((1 << 64) - 1); x ^= x >> 27
    assert draws[0] == float(np.float32(((x * 0x2545F4914F6CDD1D) & ((1 << 64) - 1)) >> 40) / np.float32(1 << 24))
    assert 0.45 < sum(draws) / len(draws) < 0.55
    # drawing many times follows the distribution
    s = plain.Sampler(1.0, 0, 1.0, 7)
    counts = np.bincount([s.sample(logits) for _ in range(4000)], minlength=5) / 4000
    want = np.exp(logits - logits.max()); want /= want.sum()
    assert np.abs(counts - want).max() < 0.03


def test_generation_stops_and_keeps_the_stop_token():
    cfg = dict(TINY_A)
    w = _weights(cfg, seed=8)
    prompt = [3, 14, 15]
    out, reason = plain.generate(cfg, w, prompt, 6)
    assert len(out) == 6 and reason == "length"
    # greedy generation is the argmax of the whole-sequence logits, token after token
    seq = list(prompt)
    for t in out:
        assert t == plain.argmax(plain.forward(cfg, w, seq)[-1])
        seq.append(t)
    stopped, reason = plain.generate(cfg, w, prompt, 6, stop=(out[2],))
    assert reason == "stop" and stopped == out[:out.index(out[2]) + 1]             # the stop token is kept
