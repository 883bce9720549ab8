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
                       page_size=page_size,
                       host={"seq_slot": list(range(len(news))), "seq_start": list(lengths_before), "seq_len": list(news)})


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
    cache = SequenceCache([(0, part.cache_needs())], 64 * 4, 2, 0, 64, torch.float32, "cuda")
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
        part.forward(ctx, x[start:start + n].contiguous(), got[start:start + n], cache.views(0), True)
    assert np.abs(got.cpu().numpy() - want).max() < 2e-5


# --------------------------------------------------------------------------- parts defined here

FAIL = {"on": False}      # makes the toy mixer raise in the middle of a step


def _register_toy_parts():
    from gemmars_b200.cache import StateNeed
    from gemmars_b200.parts import register_part
    from gemmars_b200.parts.base import Block, Part, TensorWant

    class DecayMixer(Part):
        """A recurrent toy mixer with two states of different shapes per sequence: the last two
        inputs (a shift register [2, hidden]) and a running sum [width]:
        u_t = (x_t + x_{t-1} / 2 + x_{t-2} / 4) W_in; s <- s * decay + u_t; out_t = s W_out.

        A step of whole prompts walks each sequence's tokens in order, from the batch's shape on
        the host (``ctx.host``).  A step of single tokens (which may be a captured one, padded
        with rows of ``ctx.pad_slot``) is one gather, one update and one scatter by slot, with no
        question to the host: padding rows read and write the spare row of the states only."""
        category = "mixer"

        def __init__(self, spec, compute):
            super().__init__(spec, compute)
            self.h, self.width, self.decay = spec.params["hidden_size"], spec.params["width"], spec.params["decay"]

        def wants(self):
            return {"win": TensorWant((self.width, self.h)), "wout": TensorWant((self.h, self.width))}

        def load(self, t):
            self.win, self.wout = t["win"].float(), t["wout"].float()

        def weight_bytes(self):
            return 4 * (self.win.numel() + self.wout.numel())

        def cache_needs(self):
            return [StateNeed((self.width,)), StateNeed((2, self.h))]

        def forward(self, ctx, h, residual, caches, writes_cache=True):
            if FAIL["on"]:
                raise RuntimeError("the toy mixer was told to fail")
            s_state, shift = caches
            x = h.float()
            if ctx.is_decode:
                slots = ctx.seq_slot.long()
                reg = shift[slots]
                s = s_state[slots] * self.decay + (x + 0.5 * reg[:, 0] + 0.25 * reg[:, 1]) @ self.win.T
                s_state.index_copy_(0, slots, s)
                shift.index_copy_(0, slots, torch.stack([x, reg[:, 0]], 1))
                residual += s @ self.wout.T
                return
            assert ctx.host is not None and ctx.pad_slot is None       # prompts are never padded
            outs, at = torch.empty((x.shape[0], self.width), device=x.device), 0
            for slot, n in zip(ctx.host["seq_slot"], ctx.host["seq_len"]):
                s, reg = s_state[slot].clone(), shift[slot].clone()
                for i in range(at, at + n):                 # every sequence's tokens in order
                    s = s * self.decay + (x[i] + 0.5 * reg[0] + 0.25 * reg[1]) @ self.win.T
                    reg = torch.stack([x[i], reg[0]])
                    outs[i] = s
                s_state[slot], shift[slot] = s, reg
                at += n
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

        def weight_bytes(self):
            return 4 * (self.router.numel() + self.experts.numel())

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

    class ThreeNormBlock(Block):
        """Another arrangement: pre-norm as usual, and a third norm on the stream when the layer
        is done.  It reads a part name (``out_norm``) that the package knows nothing of."""

        def __init__(self, layer_spec, compute):
            super().__init__(layer_spec, compute)
            self.built = {"mixer_norm": self.need("mixer_norm", "norm"), "mixer": self.need("mixer", "mixer"),
                          "ffn_norm": self.need("ffn_norm", "norm"), "ffn": self.need("ffn", "ffn"),
                          "out_norm": self.need("out_norm", "norm")}

        def parts(self):
            return self.built

        def forward(self, ctx, x, caches, writes_cache=True):
            p, mine = self.built, self.split_caches(caches)
            p["mixer"].forward(ctx, p["mixer_norm"].forward(ctx, x), x, mine["mixer"], writes_cache)
            p["ffn"].forward(ctx, p["ffn_norm"].forward(ctx, x), x)
            x.copy_(p["out_norm"].forward(ctx, x))

    register_part("mixer", "toy_decay", DecayMixer)
    register_part("ffn", "toy_routed", RoutedFFN)
    register_part("position", "toy_shift", ShiftEncoding)
    register_part("block", "toy_three_norms", ThreeNormBlock)


def _toy_model(h=64, vocab=97, width=24):
    """Layers that mix the package's attention (with the toy position encoding) and the toy
    recurrent mixer, dense and routed feed-forwards, a block with a third norm, a layer that runs
    twice and a layer that reads another's cache."""
    from gemmars_b200.engine.model import DecoderModel
    from gemmars_b200.parts import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
    _register_toy_parts()
    torch.manual_seed(4)
    norm = lambda n: PartSpec("rmsnorm", {"size": h, "eps": 1e-6}, {"weight": n})
    attn = lambda p, pos, kv=True: PartSpec(
        "attention", {"hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qk_norm": False,
                      "position": pos, "has_kv": kv},
        {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"} if kv else {"q": p + "q", "o": p + "o"})
    mlp = lambda p: PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 96},
                             {"gate": p + "g", "up": p + "u", "down": p + "d"})
    decay = PartSpec("toy_decay", {"hidden_size": h, "width": width, "decay": 0.9}, {"win": "l1.win", "wout": "l1.wout"})
    routed = PartSpec("toy_routed", {"hidden_size": h, "experts": 3}, {"router": "l1.r", "experts": "l1.e"})
    layers = [
        LayerSpec.prenorm(attn("l0.", PartSpec("toy_shift", {"step": 0.01})), mlp("l0."), norm("l0.n1"), norm("l0.n2")),
        LayerSpec({"mixer": decay, "ffn": routed, "mixer_norm": norm("l1.n1"), "ffn_norm": norm("l1.n2"),
                   "out_norm": norm("l1.n3")}, block="toy_three_norms"),
        LayerSpec.prenorm(attn("l2.", PartSpec("rotary", {"head_dim": 16, "theta": 1e4}), kv=False), mlp("l2."),
                          norm("l2.n1"), norm("l2.n2")),
    ]
    # layer 1 runs twice (each run with states of its own); layer 2 reads the cache of entry 0
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=0), ScheduleEntry(1)]
    plan = ModelPlan(h, vocab, PartSpec("embedding", {"vocab_size": vocab, "hidden_size": h}, {"weight": "emb"}),
                     layers, schedule, norm("nf"), PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": h}, {"weight": "emb"}), 0)
    model = DecoderModel(plan, "float32", "cuda:0")
    shapes = model.expected_tensors()
    assert shapes["l1.e"] == (3, h, h) and "l2.k" not in shapes and shapes["l1.n3"] == (h,)
    tensors = {n: (torch.rand(s) + 0.5 if len(s) == 1 else torch.randn(s) * 0.1).cuda() for n, s in shapes.items()}
    model.bind(tensors)
    return model


def _whole(runner, seqs):
    from gemmars_b200.engine import StepItem
    out = []
    for s in seqs:
        slot = runner.open()
        out.append(runner.step([StepItem(slot, s, range(len(s)))]).cpu())
        runner.close(slot)
    return out


def _in_pieces(runner, seqs, cut):
    """The prompts' first ``cut`` tokens in one step, the rest one token a step, as one batch whose
    shorter sequences end earlier."""
    from gemmars_b200.engine import StepItem
    slots = [runner.open() for _ in seqs]
    first = runner.step([StepItem(sl, s[:c], range(c)) for sl, s, c in zip(slots, seqs, cut)]).cpu()
    got = [list(first[sum(cut[:i]):sum(cut[:i + 1])]) for i in range(len(seqs))]
    pos = list(cut)
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i in range(len(seqs)) if pos[i] < len(seqs[i])]
        out = runner.step([StepItem(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu()
        for row, i in zip(out, live):
            got[i].append(row)
            pos[i] += 1
    for sl in slots:
        runner.close(sl)
    return [torch.stack(g) for g in got]


@pytest.mark.parametrize("use_graphs", [False, True])
def test_toy_parts_register_build_and_step(use_graphs):
    """Built from a plan and stepped whole, in pieces and batched, with the same result; the
    recurrent states follow their slot and start from zero when a slot is used again.  With
    captured decode steps the batch of 5, then 4, 3, ... sequences is padded with up to three rows
    of the spare slot, which must leave every real sequence's state alone."""
    from gemmars_b200.engine import Runner
    model = _toy_model()
    assert [e for e, _ in model.cache_needs()] == [0, 1, 3]
    assert [len(n) for _, n in model.cache_needs()] == [1, 2, 2]
    assert model.weight_bytes() > 0 and not model.capture_depends_on_length
    runner = Runner(model, max_tokens=64 * 12, max_batch=6, use_graphs=use_graphs)
    shapes = sorted(tuple(g.data.shape) for g in runner.cache.state_groups)
    assert shapes == [(2, 7, 2, 64), (2, 7, 24)]
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 97, n).tolist() for n in (37, 5, 70, 12, 9)]
    whole = _whole(runner, seqs)
    for round_ in range(2):                      # the second round runs in slots that were used before
        got = _in_pieces(runner, seqs, [30, 1, 64, 3, 2])
        for i in range(len(seqs)):
            assert (got[i] - whole[i]).abs().max().item() < 1e-4, (round_, i)
    assert runner.cache.pages_held() == 0
    if use_graphs:
        sizes = sorted(k[0] for k in runner._graphs)                       # one graph per padded batch size,
        assert 8 in sizes and len(set(sizes)) == len(sizes)                 # whatever the sequences' lengths


def test_a_failed_step_takes_nothing_with_it():
    """A step that raises half way leaves the lengths where they were.  A model that keeps only
    keys and values goes on as if nothing had happened; one with a state cannot, and its slot
    refuses further steps until it is closed."""
    import plain_qwen3 as plain
    from tiny_configs import TINY_A
    from gemmars_b200 import kernels
    from gemmars_b200.engine import Runner, StepItem
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.engine.step import StepError
    from gemmars_b200.weights.random_init import random_weights
    # keys and values only
    model = build_model(raw_config=TINY_A, tensors=random_weights(TINY_A, seed=5, device="cuda"), dtype="float32")
    runner = Runner(model, max_tokens=64 * 8, max_batch=2, use_graphs=False)
    toks = np.random.default_rng(1).integers(0, TINY_A["vocab_size"], 150).tolist()
    slot = runner.open()
    want = _whole(Runner(model, max_tokens=64 * 8, max_batch=2, use_graphs=False), [toks])[0]
    a = runner.step([StepItem(slot, toks[:70], range(70))]).cpu()
    held = runner.cache.pages_held()
    real, calls = kernels.gemm_swiglu, [0]

    def failing(*args, **kw):
        calls[0] += 1
        if calls[0] == 2:                       # the second layer's feed-forward: the first layer's keys are written
            raise kernels.KernelError("made to fail")
        return real(*args, **kw)

    kernels.gemm_swiglu = failing
    try:
        with pytest.raises(kernels.KernelError):
            runner.step([StepItem(slot, toks[70:], range(80))])
    finally:
        kernels.gemm_swiglu = real
    assert runner.length(slot) == 70 and runner.cache.pages_held() == held
    b = runner.step([StepItem(slot, toks[70:], range(80))]).cpu()
    assert torch.equal(torch.cat([a, b]), want)
    runner.close(slot)
    # with a state
    toy = Runner(_toy_model(), max_tokens=64 * 4, max_batch=2, use_graphs=False)
    slot = toy.open()
    toy.step([StepItem(slot, [1, 2, 3], [2])])
    FAIL["on"] = True
    try:
        with pytest.raises(RuntimeError, match="told to fail"):
            toy.step([StepItem(slot, [4], [0])])
    finally:
        FAIL["on"] = False
    assert toy.length(slot) == 3
    with pytest.raises(StepError, match="can only be closed"):
        toy.step([StepItem(slot, [4], [0])])
    toy.close(slot)
    assert toy.cache.pages_held() == 0 and toy.step([StepItem(toy.open(), [4], [0])]) is not None
