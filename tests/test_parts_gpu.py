"""Each part alone against the plain functions, and that new parts (a mixer with a state of
its own, another position encoding, a feed-forward with routing) can be registered, built and
stepped from a test, without a change to the package's files."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def _ctx(runner_or_cache, lengths_before, news, compute="float32", page_size=64):
    """A StepContext for sequences that hold lengths_before[b] tokens and bring news[b] more;
    slots are 0..B-1 of the given cache (already opened and extended)."""
    from gemmars_b200.parts.base import StepContext
    dev = torch.device("cuda")
    tok_pos = [s + i for s, n in zip(lengths_before, news) for i in range(n)]
    tok_seq = [b for b, n in enumerate(news) for _ in range(n)]
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    return StepContext(compute=compute, act_dtype=torch.float32 if compute == "float32" else torch.bfloat16, device=dev,
                       n_tokens=len(tok_pos), n_seqs=len(news), tok_pos=i32(tok_pos), tok_seq=i32(tok_seq),
                       seq_slot=i32(list(range(len(news)))), seq_start=i32(lengths_before), seq_len=i32(news),
                       cu_seqlens=i32(cu), is_decode=all(n == 1 for n in news), max_new=max(news),
                       max_total=max(s + n for s, n in zip(lengths_before, news)), cache=runner_or_cache,
                       page_size=page_size)


def test_rmsnorm_part():
    from gemmars_b200.parts import PartSpec, build_part
    torch.manual_seed(0)
    for compute, tol in (("float32", 1e-5), ("bfloat16", 2 ** -8)):
        part = build_part("norm", PartSpec("rmsnorm", {"size": 72, "eps": 1e-5}, {"weight": "w"}), compute)
        assert part.wants()["weight"].shape == (72,)
        w = torch.rand(72, device="cuda") + 0.5
        part.load({"weight": w})
        x = torch.randn(9, 72, device="cuda") * 2
        got = part.forward(None, x).float().cpu().numpy()
        want = plain.rmsnorm(x.double().cpu().numpy(), w.double().cpu().numpy(), 1e-5)
        assert np.abs(got - want).max() <= tol * np.abs(want).max()


def test_rotary_part():
    from gemmars_b200.parts import PartSpec, build_part
    torch.manual_seed(1)
    part = build_part("position", PartSpec("rotary", {"head_dim": 48, "rotary_dim": 32, "theta": 5e4}), "float32")
    inv = plain.rope_inv_freq(32, 5e4)
    assert np.array_equal(part.inv_freq(torch.device("cuda")).cpu().numpy(), inv)
    ctx = _ctx(None, [100, 0], [3, 2])
    q = torch.randn(5, 4, 48, device="cuda")
    kk = torch.randn(5, 2, 48, device="cuda")
    q0, k0 = q.double().cpu().numpy(), kk.double().cpu().numpy()
    part.apply(ctx, q, kk)
    cos, sin = plain.rope_tables([100, 101, 102, 0, 1], inv)
    assert np.abs(q.cpu().numpy() - plain.apply_rope(q0, cos, sin)).max() < 1e-5
    assert np.abs(kk.cpu().numpy() - plain.apply_rope(k0, cos, sin)).max() < 1e-5
    assert np.array_equal(q.cpu().numpy()[..., 32:], q0[..., 32:].astype(np.float32))   # dims past the rotated ones


def test_gated_mlp_and_embedding_and_head_parts():
    from gemmars_b200.parts import PartSpec, build_part
    torch.manual_seed(2)
    h, inter, vocab = 80, 112, 301
    g, u, d = (torch.randn(inter, h, device="cuda") * 0.1, torch.randn(inter, h, device="cuda") * 0.1,
               torch.randn(h, inter, device="cuda") * 0.1)
    x = torch.randn(6, h, device="cuda")
    wd = {"p.gate_proj.weight": g.double().cpu().numpy(), "p.up_proj.weight": u.double().cpu().numpy(),
          "p.down_proj.weight": d.double().cpu().numpy()}
    want = plain.mlp_block(x.double().cpu().numpy(), wd, "p.")
    for compute, tol in (("float32", 1e-5), ("bfloat16", 2 ** -6)):
        dt = torch.float32 if compute == "float32" else torch.bfloat16
        mlp = build_part("ffn", PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": inter}), compute)
        assert {k: v.shape for k, v in mlp.wants().items()} == {"gate": (inter, h), "up": (inter, h), "down": (h, inter)}
        mlp.load({"gate": g.to(dt), "up": u.to(dt), "down": d.to(dt)})
        res = torch.ones(6, h, device="cuda")
        mlp.forward(None, x.to(dt), res)
        assert np.abs(res.cpu().numpy() - 1 - want).max() <= tol * max(1.0, np.abs(want).max())
    table = torch.randn(vocab, h, device="cuda")
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": vocab, "hidden_size": h}), "float32")
    emb.load({"weight": table})
    out = torch.empty(3, h, device="cuda")
    emb.forward(None, torch.tensor([300, 0, 7], dtype=torch.int32, device="cuda"), out)
    assert torch.equal(out, table[[300, 0, 7]])
    head = build_part("head", PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": h}), "float32")
    head.load({"weight": table})
    logits = head.forward(None, x)
    assert logits.dtype == torch.float32 and (logits - x @ table.T).abs().max().item() < 1e-4
    with pytest.raises(ValueError, match="unknown ffn kind"):
        build_part("ffn", PartSpec("no_such_ffn"), "float32")


@pytest.mark.parametrize("window,bias", [(None, False), (20, True)])
def test_attention_part(window, bias):
    """The attention part over a cache of its own: a prompt step, then a continuation, against the
    plain attention block on the whole sequence."""
    from gemmars_b200.cache import SequenceCache
    from gemmars_b200.parts import PartSpec, build_part
    torch.manual_seed(3)
    h, nh, nkv, hd = 72, 6, 2, 16
    spec = PartSpec("attention", {"hidden_size": h, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm": True,
                                  "qk_norm_eps": 1e-5, "bias": bias, "window": window,
                                  "position": PartSpec("rotary", {"head_dim": hd, "theta": 1e4})})
    part = build_part("mixer", spec, "float32")
    t = {"q": torch.randn(nh * hd, h) * 0.1, "k": torch.randn(nkv * hd, h) * 0.1, "v": torch.randn(nkv * hd, h) * 0.1,
         "o": torch.randn(h, nh * hd) * 0.1, "q_norm": torch.rand(hd) + 0.5, "k_norm": torch.rand(hd) + 0.5}
    if bias:
        t.update({"q_bias": torch.randn(nh * hd) * 0.1, "k_bias": torch.randn(nkv * hd) * 0.1,
                  "v_bias": torch.randn(nkv * hd) * 0.1, "o_bias": torch.randn(h) * 0.1})
    assert set(part.wants()) == set(t)
    part.load({k: v.cuda() for k, v in t.items()})
    cache = SequenceCache([(0, part.cache_need())], 64 * 4, 2, 0, 64, torch.float32, "cuda")
    assert cache.kv_groups[0].need.window == window
    slot = cache.open()
    x = torch.randn(45, h, device="cuda")
    names = {"q": "a.q_proj.weight", "k": "a.k_proj.weight", "v": "a.v_proj.weight", "o": "a.o_proj.weight",
             "q_norm": "a.q_norm.weight", "k_norm": "a.k_norm.weight", "q_bias": "a.q_proj.bias",
             "k_bias": "a.k_proj.bias", "v_bias": "a.v_proj.bias", "o_bias": "a.o_proj.bias"}
    w = {names[k]: v.double().numpy() for k, v in t.items()}
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": 1e-5, "rope_theta": 1e4}
    want = plain.attention_block(x.double().cpu().numpy(), w, "a.", cfg, np.arange(45), window)
    got = torch.zeros(45, h, device="cuda")
    for start, n in ((0, 30), (30, 14), (44, 1)):
        cache.extend(slot, n)
        cache.sync()
        ctx = _ctx(cache, [start], [n])
        part.forward(ctx, x[start:start + n].contiguous(), got[start:start + n], cache.kv(0), True)
    assert np.abs(got.cpu().numpy() - want).max() < 2e-5


# --------------------------------------------------------------------------- parts defined here

def _register_toy_parts():
    from gemmars_b200.cache import StateNeed
    from gemmars_b200.parts import register_part
    from gemmars_b200.parts.base import Part, TensorWant

    class DecayMixer(Part):
        """A recurrent toy mixer: s <- s * decay + x W_in per token, in order; out = s W_out.
        Its state [width] lives in the cache's per-sequence state area."""
        category = "mixer"

        def __init__(self, spec, compute):
            super().__init__(spec, compute)
            self.h, self.width, self.decay = spec.params["hidden_size"], spec.params["width"], spec.params["decay"]

        def wants(self):
            return {"win": TensorWant((self.width, self.h)), "wout": TensorWant((self.h, self.width))}

        def load(self, t):
            self.win, self.wout = t["win"].float(), t["wout"].float()

        def cache_need(self):
            return StateNeed((self.width,))

        def forward(self, ctx, h, residual, state, writes_cache=True):
            u = h.float() @ self.win.T
            slots, cu = ctx.seq_slot.tolist(), ctx.cu_seqlens.tolist()
            outs = torch.empty_like(u)
            for b, slot in enumerate(slots):                 # every sequence's tokens in order, no padding token
                s = state[slot].clone()
                for i in range(cu[b], cu[b + 1]):
                    s = s * self.decay + u[i]
                    outs[i] = s
                state[slot] = s
            residual += outs @ self.wout.T

    class RoutedFFN(Part):
        """A toy feed-forward with routing: each token goes to the expert with the largest router logit."""
        category = "ffn"

        def __init__(self, spec, compute):
            super().__init__(spec, compute)
            self.h, self.e = spec.params["hidden_size"], spec.params["experts"]

        def wants(self):
            return {"router": TensorWant((self.e, self.h)), "experts": TensorWant((self.e, self.h, self.h))}

        def load(self, t):
            self.router, self.experts = t["router"].float(), t["experts"].float()

        def forward(self, ctx, h, residual):
            pick = (h.float() @ self.router.T).argmax(-1)
            residual += torch.einsum("th,tgh->tg", h.float(), self.experts[pick])

    class ShiftEncoding(Part):
        """A toy position encoding: adds position * step to the first dim of every q and k head."""
        category = "position"

        def apply(self, ctx, q, k):
            pos = ctx.tok_pos.to(q.dtype) * self.spec.params["step"]
            q[:, :, 0] += pos[:, None]
            k[:, :, 0] += pos[:, None]

    register_part("mixer", "toy_decay", DecayMixer)
    register_part("ffn", "toy_routed", RoutedFFN)
    register_part("position", "toy_shift", ShiftEncoding)


def test_toy_parts_register_build_and_step():
    """A model whose layers mix the package's attention (with the toy position encoding) and the toy
    recurrent mixer, with dense and routed feed-forwards, a layer that runs twice and a layer that
    reads another's cache: built from a plan, stepped whole, in pieces and batched, with the same
    result; the recurrent state follows its slot."""
    from gemmars_b200.engine import Runner, StepItem
    from gemmars_b200.engine.model import DecoderModel
    from gemmars_b200.parts import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    _register_toy_parts()
    torch.manual_seed(4)
    h, vocab, width = 64, 97, 24
    norm = lambda n: PartSpec("rmsnorm", {"size": h, "eps": 1e-6}, {"weight": n})
    attn = lambda p, pos, kv=True: PartSpec(
        "attention", {"hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qk_norm": False,
                      "position": pos, "has_kv": kv},
        {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"} if kv else {"q": p + "q", "o": p + "o"})
    mlp = lambda p: PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 96},
                             {"gate": p + "g", "up": p + "u", "down": p + "d"})
    layers = [
        LayerSpec(attn("l0.", PartSpec("toy_shift", {"step": 0.01})), mlp("l0."), norm("l0.n1"), norm("l0.n2")),
        LayerSpec(PartSpec("toy_decay", {"hidden_size": h, "width": width, "decay": 0.9}, {"win": "l1.win", "wout": "l1.wout"}),
                  PartSpec("toy_routed", {"hidden_size": h, "experts": 3}, {"router": "l1.r", "experts": "l1.e"}),
                  norm("l1.n1"), norm("l1.n2")),
        LayerSpec(attn("l2.", PartSpec("rotary", {"head_dim": 16, "theta": 1e4}), kv=False), mlp("l2."), norm("l2.n1"), norm("l2.n2")),
    ]
    # layer 1 runs twice (each run with a state of its own); layer 2 reads the cache of entry 0
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=0), ScheduleEntry(1)]
    plan = ModelPlan(h, vocab, PartSpec("embedding", {"vocab_size": vocab, "hidden_size": h}, {"weight": "emb"}),
                     layers, schedule, norm("nf"), PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": h}, {"weight": "emb"}), 0)
    model = DecoderModel(plan, "float32", "cuda:0")
    shapes = model.expected_tensors()
    assert shapes["l1.e"] == (3, h, h) and "l2.k" not in shapes
    tensors = {n: (torch.rand(s) + 0.5 if len(s) == 1 else torch.randn(s) * 0.1).cuda() for n, s in shapes.items()}
    model.bind(tensors)
    needs = model.cache_needs()
    assert [e for e, _ in needs] == [0, 1, 3]
    runner = Runner(model, max_tokens=64 * 8, max_batch=4, use_graphs=False)
    assert len(runner.cache.state_groups) == 1 and runner.cache.state_groups[0].data.shape == (2, 5, width)
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, vocab, n).tolist() for n in (37, 5, 70)]
    whole = []
    for s in seqs:
        slot = runner.open()
        whole.append(runner.step([StepItem(slot, s, range(len(s)))]).cpu())
        runner.close(slot)
    # in pieces, batched, unequal; slots reused (their state must start from zero again)
    slots = [runner.open() for _ in seqs]
    cut = [30, 1, 64]
    first = runner.step([StepItem(sl, s[:c], range(c)) for sl, s, c in zip(slots, seqs, cut)]).cpu()
    got = [list(first[sum(cut[:i]):sum(cut[:i + 1])]) for i in range(3)]
    pos = list(cut)
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i in range(3) if pos[i] < len(seqs[i])]
        out = runner.step([StepItem(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
        for row, i in zip(out, live):
            got[i].append(row)
            pos[i] += 1
    for i in range(3):
        assert (torch.stack(got[i]) - whole[i]).abs().max().item() < 1e-4
    for sl in slots:
        runner.close(sl)
    assert runner.cache.pages_held() == 0
