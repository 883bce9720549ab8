"""Schedules of the engine that the other files do not reach, each against the plain
implementation: weights stored in 32-bit (in both engines), decode batches of 40 and 70
sequences with heads of 128 (the unfused q/k/v product at 33 to 64 rows, the prompt product
kernel under a captured step padded to 128 rows, rows of the spare slot in the streaming
attention), a window whose ring of pages wraps several times inside one sequence, and the
float32 engine at the layer sizes of a released model."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from replay_util import Trace, run_trace
from tiny_configs import SMALL_64, SMALL_128, TINY_A, TINY_B, TOL_BF16

pytestmark = pytest.mark.gpu


def round_to_bfloat16(a):
    """float64 array -> the nearest bfloat16 values (ties to even), as float64."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


# ---------------------------------------------------------------------- weights stored in 32-bit

@pytest.mark.parametrize("name,cfg,lengths", [("A", TINY_A, [15, 70, 9]), ("B", TINY_B, [17, 150, 41])])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_stored_in_32_bit(name, cfg, lengths, dtype, model_folders, tmp_path):
    """A checkpoint whose tensors are float32 values that bfloat16 cannot hold.  The float32
    engine keeps them as they are; the bfloat16 engine rounds the matrices (not the vectors) to
    bfloat16 at load, as the reference does (src/safetensors.rs:707-733).  Through bin/trace_run,
    whole, last tokens one by one, and as a batch."""
    folder = model_folders(cfg, seed=3, dtype="float32")
    pcfg, w = plain.load_folder(folder)
    some = w[plain.tensor_prefix(w) + "layers.0.mlp.down_proj.weight"]
    assert not np.array_equal(some, round_to_bfloat16(some))            # the file really holds more than bfloat16
    if dtype == "bfloat16":
        w = {n: (round_to_bfloat16(a) if a.ndim == 2 else a) for n, a in w.items()}
    rng = np.random.default_rng(len(name))
    reqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    ref = [plain.forward(pcfg, w, r) for r in reqs]
    tr = Trace()
    tr.whole("w", reqs)
    tr.tail("t", reqs, n_tail=8)
    tr.batches("b", reqs, [[0, 1, 2]], [len(reqs[0]) - 4, 1, len(reqs[2])])
    got = run_trace(tr, folder, dtype, str(tmp_path / "out"))
    tol = 2e-5 if dtype == "float32" else TOL_BF16[name]
    scale = max(float(np.abs(r).max()) for r in ref)
    for tag in "wtb":
        for i, r in enumerate(ref):
            for p in range(len(r)):
                err = float(np.abs(got[(f"{tag}{i}", p)] - r[p]).max())
                assert err <= tol * scale, f"cutting {tag!r} request {i} position {p}: off by {err:.3e} (scale {scale:.2f})"
    if dtype == "float32":
        # a float32 engine that had rounded its matrices would sit ~2^-9 away: far outside 2e-5
        rounded = {n: (round_to_bfloat16(a) if a.ndim == 2 else a) for n, a in w.items()}
        away = float(np.abs(plain.forward(pcfg, rounded, reqs[1]) - ref[1]).max())
        assert away > 20 * tol * scale


# ---------------------------------------------------------------------- many sequences, heads of 128

@pytest.fixture(scope="module")
def small128(tmp_path_factory):
    from gemmars_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("small128"))
    write_random_model(folder, SMALL_128, seed=9)
    return (folder,) + plain.load_folder(folder)


@pytest.mark.parametrize("n_seqs", [40, 70])
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", TOL_BF16["S128"])])
def test_many_sequences_with_heads_of_128(small128, n_seqs, dtype, tol):
    """Unequal prompts in one step, then single tokens for all of them from a captured step
    (padded to 64 or 128 rows with rows of the spare slot), some of them past the window of the
    second layer and across page borders; then the odd sequences end and the rest go on (a
    captured step of another size).  Every row that is read back is compared."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, pcfg, w = small128
    vocab = SMALL_128["vocab_size"]
    rng = np.random.default_rng(n_seqs)
    lengths = [int(x) for x in rng.integers(3, 90, n_seqs)]
    lengths[0], lengths[1], lengths[2] = 260, 1, 64            # past the window of 200; a single token; a full page
    decode = 6
    seqs = [rng.integers(0, vocab, n + decode).tolist() for n in lengths]
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=64 * (n_seqs * 3 + 8), max_batch=n_seqs)
    slots = [runner.open() for _ in seqs]
    got = {i: {} for i in range(n_seqs)}
    first = runner.step([StepItem(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, lengths)]).cpu().numpy()
    for i in range(n_seqs):
        got[i][lengths[i] - 1] = first[i]
    live = list(range(n_seqs))
    for d in range(decode):
        if d == 3:
            for i in live[1::2]:
                runner.close(slots[i])
            live = live[0::2]
        out = runner.step([StepItem(slots[i], [seqs[i][lengths[i] + d]], [0]) for i in live]).cpu().numpy()
        for row, i in zip(out, live):
            got[i][lengths[i] + d] = row
    worst = (0.0, None)
    for i in range(n_seqs):
        ref = plain.forward(pcfg, w, seqs[i])
        scale = float(np.abs(ref).max())
        for p, row in got[i].items():
            err = float(np.abs(row - ref[p]).max()) / scale
            worst = max(worst, (err, (i, p)))
    assert worst[0] <= tol, f"sequence, position {worst[1]}: off by {worst[0]:.3e} of the largest logit"
    if dtype == "bfloat16":
        from gemmars_b200 import kernels
        assert kernels.attention_decode_stream_status() == 0 and kernels.gemm_tc_status() == 0


@pytest.fixture(scope="module")
def small64(tmp_path_factory):
    from gemmars_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("small64"))
    write_random_model(folder, SMALL_64, seed=12)
    return (folder,) + plain.load_folder(folder)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", TOL_BF16["S128"])])
@pytest.mark.parametrize("heads", [128, 64])
def test_random_schedules_with_heads_of_128_and_64(small128, small64, heads, dtype, tol):
    """The random schedules of test_long_gpu.py at heads of 128, where the bfloat16 engine takes
    other kernels (the streaming decode attention and its merge, the q/k/v product with the
    per-head work in its epilogue, norms inside the decode products, the tensor-core prompt
    attention): sequences start at random steps in slots just given back, move on by one token
    (captured steps) or by chunks, beside changing neighbours; every wanted row against the plain
    implementation of the same tokens whole."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, pcfg, w = small128 if heads == 128 else small64      # and at heads of 64, the kernels' other size
    rng = np.random.default_rng(23)
    toks = rng.integers(0, (SMALL_128 if heads == 128 else SMALL_64)["vocab_size"], 420).tolist()
    ref = plain.forward(pcfg, w, toks)
    scale = float(np.abs(ref).max())
    runner = Runner(build_model(folder, dtype=dtype), max_tokens=64 * 48, max_batch=6)
    live, started, checked = {}, 0, 0            # slot -> [fed, length]
    for step in range(70):
        while len(live) < 6 and started < 16 and rng.random() < 0.5:
            live[runner.open()] = [0, int(rng.integers(1, 420))]
            started += 1
        if not live:
            continue
        single = rng.random() < 0.6
        chosen = [s for s in live if rng.random() < 0.8] or [next(iter(live))]
        items, expect = [], []
        for s in chosen:
            fed, length = live[s]
            n = 1 if (single and fed > 0) else int(min(length - fed, rng.integers(1, 130)))
            if single:
                want = [n - 1]
            else:
                want = sorted(set(int(x) for x in rng.integers(0, n, size=rng.integers(0, 3))))
            items.append(StepItem(s, toks[fed:fed + n], want))
            expect += [fed + x for x in want]
            live[s][0] = fed + n
        out = runner.step(items)
        for row, pos in zip(out.cpu().numpy() if expect else [], expect):
            assert np.abs(row - ref[pos]).max() <= tol * scale, (step, pos)
            checked += 1
        for s in [s for s in live if live[s][0] >= live[s][1]]:
            runner.close(s)
            del live[s]
    assert started == 16 and checked > 70
    for s in list(live):
        runner.close(s)
    assert runner.cache.pages_held() == 0


@pytest.mark.parametrize("hidden,heads,inter", [(4096, 32, 12288), (1024, 16, 3072)])
def test_the_same_step_again_gives_the_same_bits(hidden, heads, inter):
    """A decode step at released layer sizes (two layers; 1, 8 and 40 sequences of 1,000 cached
    positions), taken back and run again 300 times: the logits are the same bits every time.  The
    partial sums of a product's ranks, the parts of the attention and of a split prompt tile are
    all added in a fixed order, whichever rank or CTA finishes first."""
    from gemmars_b200 import kernels
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import random_weights
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": inter,
           "vocab_size": 32000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
           "tie_word_embeddings": False, "max_position_embeddings": 4096}
    model = build_model(raw_config=cfg, tensors=random_weights(cfg, seed=1, device="cuda:0"), dtype="bfloat16", device="cuda:0")
    for batch in (1, 8, 40):
        runner = Runner(model, max_tokens=batch * 1100, max_batch=batch)
        slots = [runner.open() for _ in range(batch)]
        for s in slots:
            runner.cache.extend(s, 1000)
        runner.cache.sync()
        for g in runner.cache.kv_groups:
            g.k.normal_(0.0, 1.0)
            g.v.normal_(0.0, 1.0)
        first = None
        for _ in range(300):
            out = runner.step([StepItem(s, [11 + i], [0]) for i, s in enumerate(slots)])
            for s in slots:
                assert runner.cache.rollback(s, 1000)
            if first is None:
                first = out.clone()
                assert torch.isfinite(first).all()
            else:
                assert torch.equal(out, first)
        del runner
    kernels.check_status()


# ---------------------------------------------------------------------- a window's ring that wraps

@pytest.fixture(scope="module")
def windowed(tmp_path_factory):
    """TINY_B with a window of 40 on two layers and norm weights on q and k scaled up, so that
    attention picks single keys (some right at the window's edge) instead of averaging."""
    from gemmars_b200.weights import random_weights, write_safetensors
    cfg = dict(TINY_B, max_position_embeddings=1024)
    folders = {}
    for factor in (5.0, 1.0):
        tensors = random_weights(cfg, seed=33)
        for name in tensors:
            if name.endswith(("q_norm.weight", "k_norm.weight")):
                tensors[name] = (tensors[name].float() * factor).bfloat16()
        d = str(tmp_path_factory.mktemp("windowed"))
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(d, "model.safetensors"), tensors)
        folders[factor] = d
    return folders


@pytest.mark.parametrize("dtype,factor,tol", [("float32", 5.0, 2e-4), ("bfloat16", 1.0, TOL_BF16["B"])])
def test_the_ring_of_a_window_wraps(windowed, dtype, factor, tol):
    """With prompts cut into chunks of 16 tokens the ring of a window of 40 is 2 pages (128
    positions); a sequence of 460 tokens goes round it more than three times.  The rotation kernel
    writes through the wrapped table, the attention kernels read it, pages are written over while
    later keys still sit in them.  Whole (in chunks), one token at a time, and a prompt with single
    tokens after it, against the plain implementation and, in float32, bit for bit against a
    runner whose ring is long enough never to wrap."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder = windowed[factor]
    pcfg, w = plain.load_folder(folder)
    toks = np.random.default_rng(17).integers(0, pcfg["vocab_size"], 460).tolist()
    ref = plain.forward(pcfg, w, toks)
    scale = float(np.abs(ref).max())
    model = build_model(folder, dtype=dtype)

    def runner(chunk):
        r = Runner(model, max_tokens=64 * 20, max_batch=2, prefill_chunk=chunk, max_step_tokens=chunk)
        ring = [g.table_width for g in r.cache.kv_groups if g.need.window is not None]
        return r, ring

    wide, ring = runner(2048)
    assert ring[0] * 64 >= 460                           # the whole sequence fits without wrapping
    slot = wide.open()
    unwrapped = wide.step([StepItem(slot, toks, range(460))]).cpu().numpy()
    wide.close(slot)
    assert np.abs(unwrapped - ref).max() <= tol * scale

    r, ring = runner(16)
    assert ring == [2]                                   # 128 positions for a window of 40 and steps of 16
    # whole, in chunks of 16
    slot = r.open()
    whole = r.step([StepItem(slot, toks, range(460))]).cpu().numpy()
    r.close(slot)
    # a prompt that wraps once already, then single tokens (first eagerly, then from a captured step)
    slot = r.open()
    rows = list(r.step([StepItem(slot, toks[:250], range(250))]).cpu().numpy())
    for t in toks[250:]:
        rows.append(r.step([StepItem(slot, [t], [0])])[0].cpu().numpy())
    r.close(slot)
    stepped = np.stack(rows)
    # one token at a time from the first, beside a second sequence that keeps other pages busy
    slot, other = r.open(), r.open()
    r.step([StepItem(other, toks[:100], [])])
    rows = []
    for i, t in enumerate(toks):
        items = [StepItem(slot, [t], [0])]
        if i < 200:
            items.append(StepItem(other, [toks[100 + i]], [0]))
        rows.append(r.step(items)[0].cpu().numpy())
    single = np.stack(rows)
    for name, got in (("whole in chunks", whole), ("prompt then tokens", stepped), ("token by token", single)):
        err = np.abs(got - ref).max(axis=1)
        p = int(err.argmax())
        assert err[p] <= tol * scale, f"{name}: position {p} is off by {err[p]:.3e} (scale {scale:.2f})"
        if dtype == "float32":
            assert np.array_equal(got, unwrapped), f"{name}: differs from the runner whose ring never wraps"
    assert r.cache.pages_held() > 0
    r.close(slot)
    r.close(other)
    assert r.cache.pages_held() == 0


# ---------------------------------------------------------------------- float32 at a released model's layer sizes

def test_float32_at_released_layer_sizes_against_the_plain_implementation():
    """Two layers of hidden 4096, 32 / 8 heads of 128, intermediate 12288 (the vocabulary cut to
    4,099 so that NumPy can follow), weights stored in float32: the float32 engine against the
    plain implementation, whole, with the last tokens one by one, and as an unequal batch whose
    shorter request ends first; equal bits across the cuttings."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import random_weights
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
           "vocab_size": 4099, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
           "tie_word_embeddings": False, "max_position_embeddings": 4096}
    tensors = random_weights(cfg, seed=2, device="cpu", dtype=torch.float32)
    w = {n: t.double().numpy() for n, t in tensors.items()}
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (96, 40, 70)]
    ref = [plain.forward(cfg, w, s) for s in seqs]
    scale = max(float(np.abs(r).max()) for r in ref)
    model = build_model(raw_config=cfg, tensors={n: t.cuda() for n, t in tensors.items()}, dtype="float32")
    runner = Runner(model, max_tokens=64 * 8, max_batch=3)
    whole = []
    for s in seqs:
        slot = runner.open()
        whole.append(runner.step([StepItem(slot, s, range(len(s)))]).cpu().numpy())
        runner.close(slot)
    for got, want in zip(whole, ref):
        err = float(np.abs(got - want).max())
        assert err <= 1e-4 * scale, f"off by {err:.3e} (scale {scale:.2f})"
    # the last 32 tokens one by one
    slot = runner.open()
    head = len(seqs[0]) - 32
    rows = list(runner.step([StepItem(slot, seqs[0][:head], range(head))]).cpu().numpy())
    for t in seqs[0][head:]:
        rows.append(runner.step([StepItem(slot, [t], [0])])[0].cpu().numpy())
    runner.close(slot)
    assert np.array_equal(np.stack(rows), whole[0])
    # an unequal batch: prompts of 90, 1 and 70 tokens, then single tokens until each is through
    cut = [90, 1, 70]
    slots = [runner.open() for _ in seqs]
    first = runner.step([StepItem(sl, s[:c], range(c)) for sl, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    got = [list(first[sum(cut[:i]):sum(cut[:i + 1])]) for i in range(3)]
    pos = list(cut)
    runner.close(slots[2])                                                # all prompt: it ends first
    while any(p < len(s) for p, s in zip(pos, seqs)):
        live = [i for i in range(3) if pos[i] < len(seqs[i])]
        out = runner.step([StepItem(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for row, i in zip(out, live):
            got[i].append(row)
            pos[i] += 1
    for i in range(3):
        assert np.array_equal(np.stack(got[i]), whole[i]), f"request {i} depends on the batch"


def test_the_ring_wraps_under_the_fused_prompt_product(tmp_path_factory):
    """Heads of 128, bfloat16, a window of 40 on one layer, prompts cut into chunks of 128 tokens:
    the q/k/v product writes keys and values into the cache from its epilogue, through a ring of
    4 pages that a sequence of 600 tokens goes round more than twice; then single tokens."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import write_random_model
    cfg = dict(SMALL_128, sliding_window=40)
    folder = str(tmp_path_factory.mktemp("ring128"))
    write_random_model(folder, cfg, seed=12)
    pcfg, w = plain.load_folder(folder)
    toks = np.random.default_rng(4).integers(0, cfg["vocab_size"], 640).tolist()
    ref = plain.forward(pcfg, w, toks)
    scale = float(np.abs(ref).max())
    model = build_model(folder, dtype="bfloat16")
    r = Runner(model, max_tokens=64 * 24, max_batch=2, prefill_chunk=128, max_step_tokens=256)
    assert [g.table_width for g in r.cache.kv_groups if g.need.window is not None] == [4]
    slot, other = r.open(), r.open()
    # two sequences side by side, so that a sub-step packs 128 tokens of each (one starts at an odd place)
    r.step([StepItem(other, toks[:37], [])])
    out = r.step([StepItem(slot, toks[:600], range(600)), StepItem(other, toks[37:300], [262])]).float().cpu().numpy()
    err = np.abs(out[:600] - ref[:600]).max(axis=1)
    p = int(err.argmax())
    assert err[p] <= TOL_BF16["S128"] * scale, f"position {p} is off by {err[p]:.3e} (scale {scale:.2f})"
    assert np.abs(out[600] - ref[299]).max() <= TOL_BF16["S128"] * scale
    for i in range(600, 640):
        row = r.step([StepItem(slot, [toks[i]], [0])])[0].float().cpu().numpy()
        assert np.abs(row - ref[i]).max() <= TOL_BF16["S128"] * scale, i
