"""Long decoding, the first tokens of a sequence, and weights made so that faults show: norm
weights on q and k are scaled up, which makes attention pick single keys hundreds of positions
back (or right at a window's edge) instead of averaging, so a wrong key, page or slot changes
the logits by far more than rounding."""
import json
import os

import numpy as np
import pytest

import plain_qwen3 as plain
from tiny_configs import TINY_B, TOL_BF16

pytestmark = pytest.mark.gpu


def _model(tmp_path_factory, factor):
    from gemmars_b200.weights import random_weights, write_safetensors
    cfg = dict(TINY_B, max_position_embeddings=1024, sliding_window=70)
    tensors = random_weights(cfg, seed=21)
    for name in tensors:
        if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
            tensors[name] = (tensors[name].float() * factor).bfloat16()
    d = str(tmp_path_factory.mktemp("sharp"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    pcfg, w = plain.load_folder(d)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg["vocab_size"], 330).tolist()
    ref = plain.forward(pcfg, w, toks)
    return d, toks, ref


@pytest.fixture(scope="module")
def sharp_model(tmp_path_factory):
    return _model(tmp_path_factory, 5.0)


@pytest.fixture(scope="module")
def mild_model(tmp_path_factory):
    return _model(tmp_path_factory, 1.0)


# Scores are 25 times larger than with plain random weights (both norms times 5), and an absolute
# rounding error in a score is a relative error in its probability: the float32 floor is 25 times
# the usual 1e-5 or so.  A wrong or missing key moves the logits by more than 1e-3 of their size
# (test_sharp_weights_make_faults_visible), an order of magnitude above this tolerance.
# bfloat16 rounds q and k to 8 bits, which such scores turn into errors as large as the faults;
# it runs on the unscaled weights with its usual tolerance, and its attention kernels meet
# planted far keys in test_kernels_gpu.py, where inputs are the same bfloat16 values on both sides.
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", TOL_BF16["B"])])
def test_long_decoding_and_first_tokens(sharp_model, mild_model, dtype, tol):
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, toks, ref = sharp_model if dtype == "float32" else mild_model
    scale = float(np.abs(ref).max())
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=64 * 12, max_batch=2)
    # the first tokens, one by one from an empty slot, then a long run of single tokens across pages
    slot = runner.open()
    rows = []
    for t in toks[:3]:
        rows.append(runner.step([StepItem(slot, [t], [0])])[0].cpu().numpy())
    rows.extend(runner.step([StepItem(slot, toks[3:40], range(37))]).cpu().numpy())
    for t in toks[40:]:
        rows.append(runner.step([StepItem(slot, [t], [0])])[0].cpu().numpy())
    got = np.stack(rows)
    err = np.abs(got - ref).max(axis=1)
    worst = int(err.argmax())
    assert err[worst] <= tol * scale, f"position {worst} is off by {err[worst]:.3e} (scale {scale:.2f})"
    runner.close(slot)
    # the same slot and pages again, whole: what the first use left behind must not show
    slot2 = runner.open()
    assert slot2 == slot
    whole = runner.step([StepItem(slot2, toks, range(len(toks)))]).cpu().numpy()
    assert np.abs(whole - ref).max() <= tol * scale
    if dtype == "float32":
        assert np.array_equal(whole, got)
    runner.close(slot2)
    assert runner.cache.pages_held() == 0


def test_sharp_weights_make_faults_visible(sharp_model):
    """Sanity of the fixture: dropping one far key changes the oracle's logits far beyond tolerance."""
    folder, toks, ref = sharp_model
    pcfg, w = plain.load_folder(folder)
    changed = plain.forward(pcfg, w, toks[:200] + [(toks[200] + 1) % pcfg["vocab_size"]] + toks[201:])
    assert np.abs(changed[-1] - ref[-1]).max() > 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", TOL_BF16["B"])])
def test_prompts_cut_into_chunks_inside_one_step(sharp_model, mild_model, dtype, tol):
    """One step whose prompts are longer than the chunk and than the step's token budget: the
    runner feeds them in sub-steps of its own (some sequences wait for a later sub-step, the window
    of the sliding layers is crossed inside a prompt), and the wanted rows come from different
    sub-steps.  Against the plain implementation, and, in float32, bit for bit against a runner
    that takes the prompts whole."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, toks, ref = sharp_model if dtype == "float32" else mild_model
    scale = float(np.abs(ref).max())
    model = build_model(folder, dtype=dtype)
    prompts = [toks[:150], toks[:7], toks[:97]]
    wants = [[0, 15, 16, 79, 149], [6], [31, 32, 96]]

    def run(**kw):
        runner = Runner(model, max_tokens=64 * 12, max_batch=4, **kw)
        slots = [runner.open() for _ in prompts]
        out = runner.step([StepItem(s, p, w) for s, p, w in zip(slots, prompts, wants)]).cpu().numpy()
        # and the sequences go on afterwards from what the sub-steps left in the cache
        nxt = runner.step([StepItem(slots[0], [toks[150]], [0]), StepItem(slots[2], [toks[97]], [0])]).cpu().numpy()
        return out, nxt
    cut, cut_next = run(prefill_chunk=16, max_step_tokens=40)
    rows = [ref[w] for ws in wants for w in ws]
    assert cut.shape == (len(rows), ref.shape[1])
    for got, want in zip(cut, rows):
        assert np.abs(got - want).max() <= tol * scale
    assert np.abs(cut_next[0] - ref[150]).max() <= tol * scale and np.abs(cut_next[1] - ref[97]).max() <= tol * scale
    whole, whole_next = run()
    if dtype == "float32":
        assert np.array_equal(cut, whole) and np.array_equal(cut_next, whole_next)
    else:
        assert np.abs(cut - whole).max() <= tol * scale


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", TOL_BF16["B"])])
@pytest.mark.parametrize("graphs", [False, True])
def test_random_schedules(sharp_model, mild_model, dtype, tol, graphs):
    """Sequences that start at random steps, in slots that others have just given back, and move on
    by random numbers of tokens (often one: a decode step, captured or not; sometimes a chunk
    next to other sequences' single tokens), in batches of changing make-up, asking for logits at
    random places: every row against the plain implementation of the same tokens whole.  What a
    row's logits may not depend on is all varied at once: the cut into steps, the neighbours in
    the batch, the slot and the pages."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, toks, ref = sharp_model if dtype == "float32" else mild_model
    scale = float(np.abs(ref).max())
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=64 * 40, max_batch=5, use_graphs=graphs)
    rng = np.random.default_rng(17 + graphs)
    # every sequence is a prefix of the same token string, so one plain forward pass serves all
    live, started, checked = {}, 0, 0            # slot -> [fed, length]
    for step in range(60):
        while len(live) < 5 and started < 14 and rng.random() < 0.5:
            live[runner.open()] = [0, int(rng.integers(1, 330))]
            started += 1
        if not live:
            continue
        single = rng.random() < 0.6               # a step of single tokens for all, or a mixed one
        chosen = [s for s in live if rng.random() < 0.8] or [next(iter(live))]
        items, expect = [], []
        for s in chosen:
            fed, length = live[s]
            n = 1 if (single and fed > 0) else int(min(length - fed, rng.integers(1, 90)))
            want = sorted(set(int(x) for x in rng.integers(0, n, size=rng.integers(0, 3)))) if not single else [0] if n == 1 else [n - 1]
            items.append(StepItem(s, toks[fed:fed + n], want))
            expect += [fed + w for w in want]
            live[s][0] = fed + n
        out = runner.step(items).cpu().numpy() if expect else runner.step(items)
        for row, pos in zip(out if expect else [], expect):
            assert np.abs(row - ref[pos]).max() <= tol * scale, (step, pos)
            checked += 1
        for s in [s for s in live if live[s][0] >= live[s][1]]:
            runner.close(s)
            del live[s]
    assert started == 14 and checked > 60
    for s in list(live):
        runner.close(s)
    assert runner.cache.pages_held() == 0


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", TOL_BF16["B"])])
def test_a_batch_of_seventy_sequences(mild_model, dtype, tol):
    """More sequences than the decode kernels' 64-token tiles: the prompts in one step, then single
    tokens for all of them (replayed from a graph padded to 128 rows), then for the half that goes
    on after the others were closed and their slots given to new sequences."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, toks, _ = mild_model
    pcfg, w = plain.load_folder(folder)
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=64 * 160, max_batch=80)
    rng = np.random.default_rng(11)
    seqs = [rng.integers(0, pcfg["vocab_size"], int(rng.integers(6, 15))).tolist() for _ in range(70)]
    slots = [runner.open() for _ in seqs]
    fed = [len(s) - 4 for s in seqs]
    got = {i: [] for i in range(70)}
    first = runner.step([StepItem(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, fed)]).cpu().numpy()
    for i in range(70):
        got[i].append(first[i])
    for step in range(2):
        out = runner.step([StepItem(sl, [s[n + step]], [0]) for sl, s, n in zip(slots, seqs, fed)]).cpu().numpy()
        for i in range(70):
            got[i].append(out[i])
    for i in range(35, 70):
        runner.close(slots[i])
    new = [rng.integers(0, pcfg["vocab_size"], 9).tolist() for _ in range(20)]
    new_slots = [runner.open() for _ in new]
    assert set(new_slots) & set(slots[35:])                       # slots are used again
    new_out = runner.step([StepItem(sl, s, [8]) for sl, s in zip(new_slots, new)]).cpu().numpy()
    out = runner.step([StepItem(slots[i], [seqs[i][fed[i] + 2]], [0]) for i in range(35)]).cpu().numpy()
    for i in range(35):
        got[i].append(out[i])
    for i in list(range(0, 70, 9)) + [34, 69]:
        ref = plain.forward(pcfg, w, seqs[i])
        scale = float(np.abs(ref).max())
        for k_, row in enumerate(got[i]):
            assert np.abs(row - ref[fed[i] - 1 + k_]).max() <= tol * scale, (i, k_)
    for j in (0, 19):
        ref = plain.forward(pcfg, w, new[j])
        assert np.abs(new_out[j] - ref[8]).max() <= tol * float(np.abs(ref).max())


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", TOL_BF16["S128"])])
def test_heads_of_128_prompt_then_decoding(tmp_path_factory, dtype, tol):
    """A narrow model with heads of 128, so that the engine itself (not only the kernel tests) runs
    the kernels that the released sizes use: a 700-token prompt (tensor-core prompt attention over
    several tiles, the wide rotation kernel, the row-per-warp norm), a second prompt beside it, then
    forty single tokens for both (streaming decode attention over a dozen pages with a window on
    one layer, the q/k/v product with the per-head work in its epilogue, graphs)."""
    from tiny_configs import SMALL_128
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("small128"))
    write_random_model(folder, SMALL_128, seed=4)
    pcfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(8)
    a, b = rng.integers(0, 1003, 740).tolist(), rng.integers(0, 1003, 130).tolist()
    ra, rb = plain.forward(pcfg, w, a), plain.forward(pcfg, w, b)
    scale = float(max(np.abs(ra).max(), np.abs(rb).max()))
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=64 * 20, max_batch=2)
    sa, sb = runner.open(), runner.open()
    out = runner.step([StepItem(sa, a[:700], [0, 127, 128, 699]), StepItem(sb, b[:90], [89])]).cpu().numpy()
    for got, want in zip(out, [ra[0], ra[127], ra[128], ra[699], rb[89]]):
        assert np.abs(got - want).max() <= tol * scale
    for i in range(40):
        out = runner.step([StepItem(sa, [a[700 + i]], [0]), StepItem(sb, [b[90 + i]], [0])]).cpu().numpy()
        assert np.abs(out[0] - ra[700 + i]).max() <= tol * scale, i
        assert np.abs(out[1] - rb[90 + i]).max() <= tol * scale, i


def test_released_width_bfloat16_against_float32():
    """The layer sizes of a released model (hidden 4096, 32 / 8 heads of 128, intermediate 12288,
    vocabulary 151936; two layers, random weights): the bfloat16 engine, whose products, splits and
    tiles are the ones that serving uses at this width, against the float32 engine on the same
    weights, for two unequal prompts and a dozen single tokens.  (The float32 engine is checked
    against the plain implementation at small sizes; the plain implementation is too slow here.)"""
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import random_weights
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
           "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
           "tie_word_embeddings": False, "max_position_embeddings": 4096}
    tensors = random_weights(cfg, seed=0, device="cuda:0")
    rng = np.random.default_rng(0)
    a, b = rng.integers(0, cfg["vocab_size"], 330).tolist(), rng.integers(0, cfg["vocab_size"], 75).tolist()
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = build_model(raw_config=cfg, tensors=tensors, dtype=dtype, device="cuda:0")
        runner = Runner(model, max_tokens=64 * 16, max_batch=2)
        sa, sb = runner.open(), runner.open()
        rows = [runner.step([StepItem(sa, a[:300], [0, 150, 299]), StepItem(sb, b[:60], [59])]).float().cpu().numpy()]
        for i in range(12):
            rows.append(runner.step([StepItem(sa, [a[300 + i]], [0]), StepItem(sb, [b[60 + i]], [0])]).float().cpu().numpy())
        res[dtype] = np.concatenate(rows)
        del runner, model
    ref, got = res["float32"], res["bfloat16"]
    assert np.abs(got - ref).max() <= TOL_BF16["S128"] * np.abs(ref).max()
    # the token either engine would pick is, in the other engine, within that bound of the best
    for g, r in zip(got, ref):
        assert r.max() - r[int(g.argmax())] <= TOL_BF16["S128"] * np.abs(ref).max()


# hidden, query heads, kv heads, intermediate, tied head: the dense models of the family
RELEASED = {"0.6b": (1024, 16, 8, 3072, True), "1.7b": (2048, 16, 8, 6144, True), "4b": (2560, 32, 8, 9728, True),
            "14b": (5120, 40, 8, 17408, False), "32b": (5120, 64, 8, 25600, False)}


@pytest.mark.parametrize("name", list(RELEASED))
def test_released_layer_sizes_bfloat16_against_float32(name):
    """The layer sizes of the other released dense models (two layers each, random weights, the
    released vocabulary): widths that are no power of two, 40 heads, a hidden size smaller than
    heads x head size, tied heads.  Two unequal prompts and single tokens for them, then 70
    short prompts in one step and single tokens for 70, 40 and 20 of them (the prompt product
    under a captured step of 128 rows, tiles of 64 and of 32 tokens): the bfloat16 engine against
    the float32 engine on the same weights.  Measured: 0.8e-2 to 1.06e-2 of the largest logit."""
    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine import Runner, StepItem, build_model
    from gemmars_b200.weights import random_weights
    h, nh, nkv, inter, tied = RELEASED[name]
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": h,
           "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": 128, "intermediate_size": inter,
           "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
           "tie_word_embeddings": tied, "max_position_embeddings": 4096}
    tensors = random_weights(cfg, seed=0, device="cuda:0")
    rng = np.random.default_rng(0)
    a, b = rng.integers(0, cfg["vocab_size"], 330).tolist(), rng.integers(0, cfg["vocab_size"], 75).tolist()
    many = [rng.integers(0, cfg["vocab_size"], int(n)).tolist() for n in rng.integers(4, 90, 70)]
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = build_model(raw_config=cfg, tensors=tensors, dtype=dtype, device="cuda:0")
        runner = Runner(model, max_tokens=64 * 200, max_batch=72)
        sa, sb = runner.open(), runner.open()
        rows = [runner.step([StepItem(sa, a[:300], [0, 150, 299]), StepItem(sb, b[:60], [59])]).float().cpu().numpy()]
        for i in range(6):
            rows.append(runner.step([StepItem(sa, [a[300 + i]], [0]), StepItem(sb, [b[60 + i]], [0])]).float().cpu().numpy())
        slots = [runner.open() for _ in many]
        rows.append(runner.step([StepItem(s, p[:-3], [len(p) - 4]) for s, p in zip(slots, many)]).float().cpu().numpy())
        for n_live, back in ((70, 3), (40, 2), (20, 1)):
            rows.append(runner.step([StepItem(s, [p[-back]], [0]) for s, p in list(zip(slots, many))[:n_live]]).float().cpu().numpy())
        res[dtype] = np.concatenate(rows)
        del runner, model
    kernels.check_status()
    ref, got = res["float32"], res["bfloat16"]
    bound = 1.5e-2 * np.abs(ref).max()
    assert np.abs(got - ref).max() <= bound
    for g, r in zip(got, ref):
        assert r.max() - r[int(g.argmax())] <= bound
    del tensors
    torch.cuda.empty_cache()
