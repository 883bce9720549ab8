"""Generation through the Python entry point and the command line, and the device sampler."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import TINY_A, TINY_B

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _prompts(cfg, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B], ids=["A", "B"])
def test_greedy_generation_matches_plain(cfg, model_folders):
    from gemmars_b200 import Engine
    folder = model_folders(cfg)
    pcfg, w = plain.load_folder(folder)
    eng = Engine.load(folder, "dtype=float32;max_batch=3;max_tokens=2048")
    prompts = _prompts(cfg, [7, 13, 1, 40, 66])
    # a stop token that greedy decoding really meets: the 5th token the plain model generates for prompt 0
    free_run, _ = plain.generate(pcfg, w, prompts[0], 12)
    stop = [free_run[4]]
    res = eng.generate(prompts, max_tokens=12, stop_ids=stop)
    for p, r in zip(prompts, res):
        want, reason = plain.generate(pcfg, w, p, 12, stop=stop)
        assert r.tokens == want and r.reason == reason
    assert res[0].reason == "stop" and len(res[0].tokens) <= 5
    assert eng.runner.cache.pages_held() == 0 and eng.runner.cache.slots.free_count == eng.runner.cache.n_slots
    # the same requests in another batch composition give the same tokens
    again = eng.generate(list(reversed(prompts)), max_tokens=12, stop_ids=stop)
    assert [r.tokens for r in reversed(again)] == [r.tokens for r in res]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_give_the_same_tokens(dtype, model_folders):
    """The next decode step is launched from the sampler's tokens on the device before the host has
    read them.  Greedy and seeded temperature generation must give exactly what the engine gives
    when every step waits for the host, stop tokens met along the way and batches of unequal
    lengths included; and steps must really have been launched ahead."""
    from gemmars_b200 import Engine, SamplingParams
    folder = model_folders(TINY_B)
    prompts = _prompts(TINY_B, [7, 13, 1, 40, 66, 5], seed=5)
    results = {}
    for ahead in ("true", "false"):
        eng = Engine.load(folder, f"dtype={dtype};max_batch=4;max_tokens=4096;decode_ahead={ahead}")
        free_run = eng.generate(prompts[:1], max_tokens=10, stop_ids=[])[0].tokens
        greedy = eng.generate(prompts, max_tokens=14, stop_ids=[free_run[6]])
        sampled = eng.generate(prompts, max_tokens=9, stop_ids=[], sampling=SamplingParams(0.9, 40, 0.9, seed=3))
        results[ahead] = ([(r.tokens, r.reason) for r in greedy], [(r.tokens, r.reason) for r in sampled], eng.stats.decode_steps)
        assert eng.runner.cache.pages_held() == 0
    assert results["true"][:2] == results["false"][:2]
    assert any(reason == "stop" for _, reason in results["true"][0])


def test_two_engines_take_turns_on_one_device(model_folders, tmp_path_factory):
    """Two engines of different shapes on the same device, one after the other and again, each
    with captured decode steps of its own: they share the kernels' per-device scratch and the
    loaded units, and each still generates what it generates alone."""
    from gemmars_b200 import Engine
    from gemmars_b200.weights import write_random_model
    small = model_folders(TINY_B)
    wide_cfg = dict(TINY_B, hidden_size=256, num_attention_heads=16, num_key_value_heads=1, head_dim=64,
                    intermediate_size=320, use_sliding_window=False, layer_types=["full_attention"] * TINY_B["num_hidden_layers"])
    wide = str(tmp_path_factory.mktemp("wide"))
    write_random_model(wide, wide_cfg, seed=9)
    alone = {}
    for name, folder, cfg in (("small", small, TINY_B), ("wide", wide, wide_cfg)):
        eng = Engine.load(folder, "dtype=bfloat16;max_batch=4;max_tokens=4096")
        alone[name] = [r.tokens for r in eng.generate(_prompts(cfg, [70, 9, 300, 33], seed=2), max_tokens=24)]
        del eng
    torch.cuda.empty_cache()
    a = Engine.load(small, "dtype=bfloat16;max_batch=4;max_tokens=4096")
    first = [r.tokens for r in a.generate(_prompts(TINY_B, [70, 9, 300, 33], seed=2), max_tokens=24)]     # captures its steps
    b = Engine.load(wide, "dtype=bfloat16;max_batch=4;max_tokens=4096")
    for _ in range(2):
        assert [r.tokens for r in b.generate(_prompts(wide_cfg, [70, 9, 300, 33], seed=2), max_tokens=24)] == alone["wide"]
        assert [r.tokens for r in a.generate(_prompts(TINY_B, [70, 9, 300, 33], seed=2), max_tokens=24)] == alone["small"]
    assert first == alone["small"]


def test_bfloat16_generation_runs_and_mostly_agrees(model_folders):
    from gemmars_b200 import Engine
    folder = model_folders(TINY_A)
    pcfg, w = plain.load_folder(folder)
    eng = Engine.load(folder, "dtype=bfloat16;max_batch=4")
    prompts = _prompts(TINY_A, [9, 3, 30, 17], seed=3)
    res = eng.generate(prompts, max_tokens=8, stop_ids=[])
    # greedy tokens can differ from the float64 oracle only where two logits are nearly tied
    for p, r in zip(prompts, res):
        seq = list(p)
        for tok in r.tokens:
            logits = plain.forward(pcfg, w, seq)[-1]
            assert logits.max() - logits[tok] <= 2e-2 * np.abs(logits).max()
            seq.append(tok)


def test_conversation_keeps_its_cache(model_folders):
    from gemmars_b200 import Engine
    folder = model_folders(TINY_B)
    pcfg, w = plain.load_folder(folder)
    eng = Engine.load(folder, "dtype=float32")
    eng.set("max_tokens", 5)
    eng.set("stop", "")
    first = [5, 9, 200, 31]
    r1 = eng.send(first)
    want1, _ = plain.generate(pcfg, w, first, 5)
    assert r1.tokens == want1 and r1.reason == "length"
    # the second turn continues from the cache; the last generated token was not run and is fed first
    second = [77, 12]
    r2 = eng.send(second)
    want2, _ = plain.generate(pcfg, w, first + want1 + second, 5)
    assert r2.tokens == want2
    eng.reset()
    assert eng.send(first).tokens == want1


def test_device_sampler_matches_the_plain_sampler():
    from gemmars_b200 import kernels
    rng = np.random.default_rng(5)
    vocab = 3001
    logits = (rng.standard_normal((6, vocab)) * 3).astype(np.float32)
    logits[1, 100] = logits[1, 2000] = logits[1].max() + 1.0        # a tie at the top: lower id wins
    logits[4, :50] = 2.5                                               # many ties around the k-th place
    params = [(0.0, 64, 0.95), (0.0, 64, 0.95), (0.7, 64, 0.95), (1.3, 1, 1.0), (1.0, 20, 0.5), (0.9, 1024, 1.0),
              (1.1, 0, 0.9), (0.8, 0, 1.0), (1.0, 2000, 0.97), (2.0, 5000, 1.0)]     # the last four: sorted in global memory
    logits = np.concatenate([logits, (rng.standard_normal((4, vocab)) * 3).astype(np.float32)])
    logits[7, 5:400:7] = logits[7].max()                               # many equal maxima among all tokens
    dev = torch.from_numpy(logits).cuda()
    out = torch.empty(len(params), dtype=torch.int32, device="cuda")
    for trial in range(20):
        samplers = [plain.Sampler(t, k, p, seed=trial * 7 + i + 1) for i, (t, k, p) in enumerate(params)]
        us = []
        for s in samplers:
            state = s.rng
            us.append(float(s.next_f32()) if s.temperature > 0 else 0.0)
            s.rng = state
        kernels.sample(dev, out,
                       torch.tensor([p[0] for p in params], dtype=torch.float32, device="cuda"),
                       torch.tensor([p[1] for p in params], dtype=torch.int32, device="cuda"),
                       torch.tensor([p[2] for p in params], dtype=torch.float32, device="cuda"),
                       torch.tensor(us, dtype=torch.float32, device="cuda"), wide=True)
        got = out.tolist()
        want = [s.sample(logits[i]) for i, s in enumerate(samplers)]
        assert got == want, f"trial {trial}: {got} != {want}"
    kernels.sample(dev, out)                                           # all greedy
    assert out.tolist() == [plain.argmax(r) for r in logits]


def test_device_sampler_at_a_released_vocabulary():
    """Sixteen rows of 151,936 logits: every row is cut into slices that different CTAs select
    from, so the candidates of a row come from several CTAs; ties are planted across the slices'
    borders and at the k-th place.  Token for token against the plain sampler."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(6)
    rows, vocab = 16, 151936
    logits = (rng.standard_normal((rows, vocab)) * 2.5).astype(np.float32)
    top = float(logits.max()) + 1.0
    logits[0, [5, 40000, 151935]] = top                              # equal maxima far apart: the lowest id first
    logits[1, 9000:9100] = logits[1, 120000:120050] = 4.0            # 150 equal values around the 64-th place
    logits[2, ::1000] = top                                          # 152 equal maxima, k = 100
    logits[3, 151935] = top                                          # the last token of the last slice
    params = [(0.0, 64, 0.95), (0.8, 64, 0.95), (1.0, 100, 1.0), (0.0, 1, 1.0)] + [
        (0.6 + 0.1 * i, [1, 7, 64, 333, 1024][i % 5], [0.5, 0.9, 0.95, 1.0][i % 4]) for i in range(12)]
    dev = torch.from_numpy(logits).cuda()
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    for trial in range(6):
        samplers = [plain.Sampler(t, k, p, seed=trial * 31 + i + 1) for i, (t, k, p) in enumerate(params)]
        us = []
        for s in samplers:
            state = s.rng
            us.append(float(s.next_f32()) if s.temperature > 0 else 0.0)
            s.rng = state
        args = (torch.tensor([p[0] for p in params], dtype=torch.float32, device="cuda"),
                torch.tensor([p[1] for p in params], dtype=torch.int32, device="cuda"),
                torch.tensor([p[2] for p in params], dtype=torch.float32, device="cuda"),
                torch.tensor(us, dtype=torch.float32, device="cuda"))
        kernels.sample(dev, out, *args, cap=1024)
        want = [s.sample(logits[i]) for i, s in enumerate(samplers)]
        assert out.tolist() == want, f"trial {trial}"
    kernels.sample(dev, out)                                           # all greedy
    assert out.tolist() == [int(np.argmax(r)) for r in logits]
    # a cap below a row's top_k would drop candidates: the sampler object computes it from its rows
    from gemmars_b200.sampling.sampler import BatchSampler, SamplingParams
    assert BatchSampler([SamplingParams(0.7, 64), SamplingParams(0.0, 900), SamplingParams(1.0, 0)], "cuda").cap == 64


def test_temperature_sampling_is_seeded(model_folders):
    from gemmars_b200 import Engine, SamplingParams
    folder = model_folders(TINY_A)
    eng = Engine.load(folder, "dtype=float32;max_batch=2")
    prompts = _prompts(TINY_A, [5, 11, 8], seed=9)
    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=123)
    a = eng.generate(prompts, max_tokens=10, sampling=sp, stop_ids=[])
    b = eng.generate(prompts, max_tokens=10, sampling=sp, stop_ids=[])
    c = eng.generate(prompts, max_tokens=10, sampling=SamplingParams(0.8, 50, 0.9, seed=124), stop_ids=[])
    assert [r.tokens for r in a] == [r.tokens for r in b] != [r.tokens for r in c]
    # against the plain model and sampler, sequence i seeded seed + i
    pcfg, w = plain.load_folder(folder)
    for i, (p, r) in enumerate(zip(prompts, a)):
        want, _ = plain.generate(pcfg, w, p, 10, temperature=0.8, top_k=50, top_p=0.9, seed=123 + i)
        assert r.tokens == want
    # top_k = 0: every token is a candidate (src/sampler.rs:43-47)
    sp0 = SamplingParams(temperature=1.1, top_k=0, top_p=0.9, seed=7)
    for i, (p, r) in enumerate(zip(prompts, eng.generate(prompts, max_tokens=6, sampling=sp0, stop_ids=[]))):
        want, _ = plain.generate(pcfg, w, p, 6, temperature=1.1, top_k=0, top_p=0.9, seed=7 + i)
        assert r.tokens == want
    with pytest.raises(ValueError, match="top_k"):
        eng.generate(prompts, sampling=SamplingParams(temperature=1.0, top_k=-1))


def test_command_line(model_folders, tmp_path):
    folder = model_folders(TINY_A)
    pcfg, w = plain.load_folder(folder)
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    base = [sys.executable, "-m", "gemmars_b200", "--model", folder, "--dtype", "float32"]
    p = subprocess.run(base + ["--tokens", ",".join(map(str, prompt)), "-n", "6"], capture_output=True, text=True,
                       cwd=ROOT, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    want, _ = plain.generate(pcfg, w, prompt, 6, stop=[7])
    assert [int(x) for x in p.stdout.strip().split(",")] == want
    assert "tok/s" in p.stderr
    dump = tmp_path / "logits.bin"
    p = subprocess.run(base + ["--tokens", ",".join(map(str, prompt)), "--dump-logits", str(dump)],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    got = np.fromfile(dump, dtype="<f4")
    assert np.abs(got - plain.forward(pcfg, w, prompt)[-1]).max() < 2e-5
    p = subprocess.run(base + ["--tokens", ",".join(map(str, prompt)), "-n", "6", "--profile"], capture_output=True,
                       text=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.strip().split(",")] == want
    # per category (time, calls, bytes, bandwidth) and per kernel, per forward token
    assert "ms/tok" in p.stderr and "attention_ref" in p.stderr and "gemm_ref" in p.stderr
    cats = {l.split()[0]: l.split() for l in p.stderr.splitlines() if l.split() and l.split()[0] in
            ("matmul", "attention", "norm", "elementwise", "embed", "lm_head", "sampling")}
    assert set(cats) == {"matmul", "attention", "norm", "elementwise", "embed", "lm_head", "sampling"}
    assert float(cats["matmul"][4]) > 0 and float(cats["attention"][4]) > 0 and float(cats["lm_head"][5]) > 0
    batch = tmp_path / "batch.txt"
    batch.write_text("1 2 3\n9,8,7,6,5\n")
    p = subprocess.run(base + ["--batch-file", str(batch), "-n", "4"], capture_output=True, text=True, cwd=ROOT,
                       timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    rows = [json.loads(l) for l in p.stdout.splitlines()]
    assert rows[1]["tokens"] == plain.generate(pcfg, w, [9, 8, 7, 6, 5], 4, stop=[7])[0]
