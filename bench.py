#!/usr/bin/env python3
"""Decode and prefill throughput of Qwen3-shaped models with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--config 8b|4b|32b]

``--config 8b`` (the default) is the headline benchmark.  A step is one decode step of a batch
of 8 sequences at a context of 8,192 tokens.  One JSON line is printed: ``value`` = decoded
tokens a second measured on the device over exactly K steps; ``e2e`` = the same through
``Engine.generate`` (host token ids in, host token ids out, every step's host-to-device and
device-to-host copies included) over 256 generated tokens a sequence; ``prefill`` = one prompt
of 2,048 tokens; ``roofline`` = bytes a decode step has to read (every weight once, the cache of
the live requests) over its time, against the measured copy bandwidth; ``points`` = decode at
batch 1 and 64, with the time, bytes, fraction and clocks of each under ``points_detail``.

``--config 4b``: 16 prompts of 128 to 4,096 tokens (uniform, seeded), 256 tokens each at
temperature 0.7 with a fixed seed, through ``Engine.generate``.  ``--config 32b``: a prompt of
2,048 tokens, then greedy decoding at batch 1 and 32 up to a context of 4,096.  Each prints one
line of the same form.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else 6.65 TB/s and
1.59 PFLOP/s (an earlier measurement on the same pool).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


from gemmars_b200.tuning import SHAPES as CONFIGS, random_engine, synthetic_fill   # noqa: E402  (the layer sizes measured at)

CONTEXT = 8192
PREFILL_TOKENS = 2048
E2E_TOKENS = 256


def peaks():
    """(copy GB/s, bf16 TFLOP/s as a burst, bf16 TFLOP/s sustained under the power cap, where from)."""
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    hbm, tf, tf_sustained, src = 6650.0, 1590.0, 1400.0, "fallback"
    try:
        with open(path) as f:
            p = json.load(f)
        hbm = float(p.get("hbm_gbs", hbm))
        tf = float(p.get("bf16_tflops", tf))
        tf_sustained = float(p.get("bf16_tflops_sustained", min(tf, tf_sustained)))
        src = "measured"
    except (OSError, ValueError):
        pass
    return hbm, tf, tf_sustained, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(r[0]))
                mx.append(int(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def kv_bytes_per_token(runner):
    """Bytes of keys and values one cached position takes over all layers (groups that keep all keys)."""
    return sum(2 * g.n_layers * g.need.num_kv_heads * g.need.head_dim * g.k.element_size() for g in runner.cache.kv_groups)


def decode_bytes(model, runner, lengths):
    """Bytes one decode step has to read: every weight once and the cached keys and values of
    the live sequences."""
    kv = 0
    for g in runner.cache.kv_groups:
        per_token = 2 * g.n_layers * g.need.num_kv_heads * g.need.head_dim * g.k.element_size()
        for n in lengths:
            kv += per_token * (min(n, g.need.window) if g.need.window else n)
    return model.weight_bytes() + kv


def prefill_flops(cfg, t):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token = 2 * (h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i)
    attn = 4 * nh * hd * (t * (t + 1) // 2)           # QK^T and PV over the causal half
    return cfg["num_hidden_layers"] * (per_token * t + attn) + 2 * h * v  # logits of the last row only


def fill_cache(runner, slots, length, real, vocab, gen):
    """Brings every slot to ``length`` cached tokens: by running prompts (real) or by
    reserving the pages and writing random keys and values (synthetic)."""
    import torch
    from gemmars_b200.engine.step import StepItem
    if real:
        for s in slots:
            toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
            runner.step([StepItem(s, toks, [])])
        return
    synthetic_fill(runner, slots, length)


def time_decode(eng, batch, ctx_end, steps, warmup, real_fill, hbm_gbs):
    """Device time of exactly ``steps`` decode steps of ``batch`` sequences ending at ``ctx_end``,
    with the clocks sampled meanwhile: {"tokens_per_s", "ms_per_step", "steps", "bytes_per_step",
    "achieved_gbs", "frac", "clocks", "launches"}."""
    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine.step import StepItem
    from gemmars_b200.sampling.sampler import BatchSampler, SamplingParams
    runner, vocab = eng.runner, eng.model.plan.vocab_size
    gen = torch.Generator().manual_seed(1)
    slots = [runner.open() for _ in range(batch)]
    start_len = ctx_end - steps - warmup
    fill_cache(runner, slots, start_len, real_fill, vocab, gen)
    sampler = BatchSampler([SamplingParams()] * batch, runner.device)
    toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()

    rows = list(range(batch))
    ahead = eng.options.decode_ahead and runner.use_graphs

    def one(logits):
        """A step as the generation loop runs it: draw from the logits, launch the next step from
        the drawn tokens where they lie, then read them on the host (what generation needs them
        for: stop tokens, limits, the caller)."""
        drawn = sampler.draw(logits, rows)
        nxt = runner.decode_from_device(slots, drawn) if ahead else None
        toks = sampler.read(drawn)
        if nxt is None:
            nxt = runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
        return nxt

    logits = runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
    for _ in range(warmup - 1):
        logits = one(logits)
    torch.cuda.synchronize()
    clocks = ClockSampler().start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    e0.record()
    for _ in range(steps):
        logits = one(logits)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    clock_rec = clocks.stop()
    lengths = [runner.length(s) for s in slots]
    nbytes = decode_bytes(eng.model, runner, lengths)
    for s in slots:
        runner.close(s)
    kernels.check_status()
    achieved = nbytes / (ms / 1e3) / 1e9
    return {"tokens_per_s": round(batch / (ms / 1e3), 1), "ms_per_step": round(ms, 4), "steps": steps,
            "bytes_per_step": nbytes, "achieved_gbs": round(achieved, 1), "frac": round(achieved / hbm_gbs, 4),
            "clocks": clock_rec, "launches": kernels.launch_count() - launches0}


def time_prefill(eng, cfg, tokens, tflops, tflops_sustained):
    """The median of seven prompts of ``tokens`` tokens after three warm-up prompts."""
    import torch
    from gemmars_b200.engine.step import StepItem
    runner = eng.runner
    toks = torch.randint(0, cfg["vocab_size"], (tokens,), generator=torch.Generator().manual_seed(3)).tolist()
    pre_ms = []
    for it in range(10):
        s = runner.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepItem(s, toks, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            pre_ms.append(e0.elapsed_time(e1))
        runner.close(s)
    pre = statistics.median(pre_ms)
    frac = prefill_flops(cfg, tokens) / (pre / 1e3) / (tflops * 1e12)
    return {"value": round(tokens / (pre / 1e3), 1), "tokens": tokens, "ms": round(pre, 3), "frac": round(frac, 4),
            # a prompt is tens of milliseconds of products under the power cap: also against the sustained rate
            "frac_sustained": round(frac * tflops / tflops_sustained, 4)}


def make_engine(cfg, max_batch, cache_tokens, options=""):
    return random_engine(cfg, max_batch, cache_tokens, options)


def config_record(name, cfg, layers_full, batch, context, fill, peak_line):
    return {"model": name, "layers": cfg["num_hidden_layers"], "layers_full": layers_full,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"],
            "tie_word_embeddings": cfg["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "cache_fill": fill,
            "points_cache_fill": "synthetic", "l2": "weights and cache read per step exceed L2 (no flush needed)",
            "peaks": peak_line}


def run_8b(args, name, cfg, layers_full):
    import torch
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    warmup = max(3, args.warmup)
    points = not args.no_points
    max_batch = 64 if points else args.batch
    eng = make_engine(cfg, max_batch, max_batch * (args.context + 64), args.options)
    vocab = cfg["vocab_size"]
    # a prompt first: it is a burst of work on a GPU that was waiting
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    main = time_decode(eng, args.batch, args.context, args.steps, warmup, args.fill == "real", hbm_gbs)

    # end to end through the entry point: host ids in, host ids out, 256 tokens a sequence
    gen = torch.Generator().manual_seed(2)
    e2e_new = max(2, args.e2e_tokens)
    prompts = [torch.randint(0, vocab, (args.context - e2e_new,), generator=gen).tolist() for _ in range(args.batch)]
    clocks = ClockSampler().start()
    res = eng.generate(prompts, max_tokens=e2e_new, stop_ids=[])
    e2e_clocks = clocks.stop()
    st = eng.stats
    assert all(len(r.tokens) == e2e_new for r in res)

    pts, detail = {}, {}
    if points:
        for b in (1, 64):
            d = time_decode(eng, b, args.context, min(args.steps, 16), 3, False, hbm_gbs)
            pts[f"decode_b{b}"] = d["tokens_per_s"]
            detail[f"decode_b{b}"] = {k: d[k] for k in ("ms_per_step", "steps", "bytes_per_step", "achieved_gbs", "frac", "clocks")}
    return {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({name}, bf16, random weights)",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": config_record(name, cfg, layers_full, args.batch, args.context, args.fill,
                                f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})"),
        "clocks": main["clocks"],
        "e2e": {"value": round(st.generated_tokens / max(st.decode_secs, 1e-9), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": (8 * args.batch + 1) * 4, "d2h_bytes_per_step": args.batch * 4,
                "generated": st.generated_tokens, "decode_steps": st.decode_steps,
                "prefill_secs": round(st.prefill_secs, 3), "sm_mhz": e2e_clocks["sm_mhz"]},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main["achieved_gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main["frac"], "bytes_per_step": main["bytes_per_step"]},
        "points": pts,
        "points_detail": detail,
    }


def run_4b(args, name, cfg, layers_full):
    """16 prompts of 128 to 4,096 tokens, 256 tokens each at temperature 0.7, seed fixed, through
    ``Engine.generate``."""
    import numpy as np
    import torch
    from gemmars_b200.sampling.sampler import SamplingParams
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    batch, new = 16, 256
    rng = np.random.default_rng(4)
    lengths = [int(x) for x in rng.integers(128, 4097, batch)]
    eng = make_engine(cfg, batch, batch * (4096 + new + 64), args.options)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    sampling = SamplingParams(temperature=0.7, top_k=64, top_p=0.95, seed=42)
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    eng.generate([p[:64] for p in prompts], max_tokens=8, sampling=sampling, stop_ids=[])      # warm-up: builds, graphs
    clocks = ClockSampler().start()
    res = eng.generate(prompts, max_tokens=new, sampling=sampling, stop_ids=[])
    clock_rec = clocks.stop()
    st = eng.stats
    assert all(len(r.tokens) == new for r in res)
    # bytes the decode steps had to read: the weights every step, and each sequence's cache as it grows
    per_tok = kv_bytes_per_token(eng.runner)
    steps = st.decode_steps
    kv = sum(per_tok * (n + k) for n in lengths for k in range(1, steps + 1))
    nbytes = steps * eng.model.weight_bytes() + kv
    achieved = nbytes / max(st.decode_secs, 1e-9) / 1e9
    ms = st.decode_secs * 1e3 / max(steps, 1)
    value = st.generated_tokens / max(st.decode_secs, 1e-9)
    return {
        "metric": f"decode tok/s, 16 prompts of 128-4096 tokens, 256 tokens each at temperature 0.7 ({name}, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 8,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": dict({k: v for k, v in config_record(name, cfg, layers_full, batch, max(lengths) + new, "real",
                                                       f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})").items()
                        if k not in ("cache_fill", "points_cache_fill")},
                       prompt_tokens=sum(lengths), mean_prompt=round(sum(lengths) / batch, 1),
                       sampling="temperature 0.7, top_k 64, top_p 0.95, seed 42", timing="wall clock through Engine.generate"),
        "clocks": clock_rec,
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": (8 * batch + 1) * 4 + 16 * batch,
                "d2h_bytes_per_step": batch * 4, "generated": st.generated_tokens, "decode_steps": steps,
                "prefill_secs": round(st.prefill_secs, 3),
                "prefill_tokens_per_s": round(sum(lengths) / max(st.prefill_secs, 1e-9), 1)},
        "gpu_launches": None,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "bytes_per_step": nbytes // max(steps, 1)},
        "points": {},
    }


def run_32b(args, name, cfg, layers_full):
    """A prompt of 2,048 tokens, then greedy decoding at batch 1 and 32 up to a context of 4,096."""
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    context, steps, warmup = 4096, args.steps, max(3, args.warmup)
    eng = make_engine(cfg, 32, 32 * (context + 64), args.options)
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    main = time_decode(eng, 32, context, steps, warmup, args.fill == "real", hbm_gbs)
    one = time_decode(eng, 1, context, steps, warmup, args.fill == "real", hbm_gbs)
    keep = ("ms_per_step", "steps", "bytes_per_step", "achieved_gbs", "frac", "clocks")
    return {
        "metric": f"decode tok/s at batch 32, context {context} ({name}, bf16, random weights)",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": config_record(name, cfg, layers_full, 32, context, args.fill,
                                f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})"),
        "clocks": main["clocks"], "gpu_launches": main["launches"], "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main["achieved_gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main["frac"], "bytes_per_step": main["bytes_per_step"]},
        "points": {"decode_b1": one["tokens_per_s"], "decode_b32": main["tokens_per_s"]},
        "points_detail": {"decode_b1": {k: one[k] for k in keep}, "decode_b32": {k: main[k] for k in keep}},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="8b", help="which model shape and workload")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--fill", choices=["real", "synthetic"], default="real",
                    help="how the cache is brought to the context length before decoding is timed")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--e2e-tokens", type=int, default=E2E_TOKENS,
                    help="tokens a sequence generates in the end-to-end run (fewer for runs under a profiler)")
    ap.add_argument("--options", default="", help='further engine options, "key=value;key=value"')
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (oxinfer); no cargo/rustc offline, so pip cannot build it; "
                          "it publishes no NVIDIA path that runs decode on the GPU"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported", flush=True)
        return 2
    name, cfg = CONFIGS[args.config]
    layers_full = cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=args.layers or layers_full)
    # three shapes have workloads of their own; any other runs the 8B workload at its own sizes
    line = {"4b": run_4b, "32b": run_32b}.get(args.config, run_8b)(args, name, cfg, layers_full)
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
