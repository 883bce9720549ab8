#!/usr/bin/env python3
"""Decode and prefill throughput of a Qwen3-8B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of a batch of 8 sequences at a context of 8,192 tokens.  One JSON
line is printed: ``value`` = decoded tokens a second measured on the device over exactly K
steps; ``e2e`` = the same through ``Engine.generate`` (host token ids in, host token ids out,
every step's host-to-device and device-to-host copies included); ``prefill`` = one prompt of
2,048 tokens; ``roofline`` = bytes a decode step has to read (every weight once, the cache of
the live requests) over its time, against the measured copy bandwidth; ``points`` = decode at
batch 1 and 64.  Peaks come from MEASURED_PEAKS.json beside this file when it exists, else
6.65 TB/s and 1.59 PFLOP/s (an earlier measurement on the same pool).
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

# The layer sizes of the benchmark configuration (Qwen3-8B).
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": False,
    "max_position_embeddings": 40960,
}
FULL_LAYERS = 36
CONTEXT = 8192
PREFILL_TOKENS = 2048


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


def decode_bytes(model, runner, lengths):
    """Bytes one decode step has to read: every weight matrix once and the cached keys and
    values of the live sequences."""
    kv = 0
    for g in runner.cache.kv_groups:
        per_token = 2 * g.n_layers * g.need.num_kv_heads * g.need.head_dim * g.k.element_size()
        for n in lengths:
            kv += per_token * (min(n, g.need.window) if g.need.window else n)
    return model.weight_bytes() + kv


def prefill_flops(cfg, layers, t):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token = 2 * (h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i)
    attn = 4 * nh * hd * (t * (t + 1) // 2)           # QK^T and PV over the causal half
    return layers * (per_token * t + attn) + 2 * h * v  # logits of the last row only


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
    for s in slots:
        runner.cache.extend(s, length)
    runner.cache.sync()
    for g in runner.cache.kv_groups:
        for t in (g.k, g.v):
            for layer in range(t.shape[0]):
                t[layer].normal_(0.0, 1.0)


def time_decode(runner, batch, ctx_end, steps, warmup, real_fill, vocab, sampler_cls, params_cls):
    """Device time of exactly ``steps`` decode steps of ``batch`` sequences ending at ``ctx_end``."""
    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine.step import StepItem
    gen = torch.Generator().manual_seed(1)
    slots = [runner.open() for _ in range(batch)]
    start_len = ctx_end - steps - warmup
    fill_cache(runner, slots, start_len, real_fill, vocab, gen)
    sampler = sampler_cls([params_cls()] * batch, runner.device)
    toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()

    def one(toks):
        logits = runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
        return sampler.sample_device(logits, list(range(batch)))

    for _ in range(warmup):
        toks = one(toks).tolist()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    cur = toks
    e0.record()
    for _ in range(steps):
        cur = one(cur).tolist()          # the next step's tokens come back to the host, as in generation
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = kernels.launch_count() - launches0
    lengths = [runner.length(s) for s in slots]
    for s in slots:
        runner.close(s)
    return ms / steps, launches, lengths


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--fill", choices=["real", "synthetic"], default="real",
                    help="how the cache is brought to the context length before decoding is timed")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
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
    warmup = max(3, args.warmup)

    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine.engine import Engine, EngineOptions
    from gemmars_b200.engine.step import StepItem
    from gemmars_b200.sampling.sampler import BatchSampler, SamplingParams
    from gemmars_b200.weights.random_init import random_weights

    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    vocab = cfg["vocab_size"]
    torch.cuda.set_device(0)
    tensors = random_weights(cfg, seed=0, device="cuda:0")
    points = not args.no_points
    max_batch = 64 if points else args.batch
    cache_tokens = max_batch * (args.context + 64)
    opts = EngineOptions.parse({"dtype": "bfloat16", "max_batch": str(max_batch), "max_tokens": str(cache_tokens),
                                "prefill_chunk": "2048"})
    for pair in filter(None, (p.strip() for p in args.options.split(";"))):
        opts.set(*[x.strip() for x in pair.split("=", 1)])
    eng = Engine.from_config(cfg, tensors, opts)
    del tensors
    runner, model = eng.runner, eng.model

    # ---- prefill of 2,048 tokens (first: a prompt is a burst of work on a GPU that was waiting)
    toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(3)).tolist()
    pre_ms = []
    for it in range(10):
        s = runner.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepItem(s, toks, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:                        # three warm-up prompts
            pre_ms.append(e0.elapsed_time(e1))
        runner.close(s)
    pre = statistics.median(pre_ms)
    pre_frac = prefill_flops(cfg, args.layers, PREFILL_TOKENS) / (pre / 1e3) / (tflops * 1e12)

    # ---- the timed decode steps (device time, CUDA events)
    clocks = ClockSampler()
    clocks.start()
    ms_step, launches, lengths = time_decode(runner, args.batch, args.context, args.steps, warmup,
                                             args.fill == "real", vocab, BatchSampler, SamplingParams)
    clock_rec = clocks.stop()
    value = args.batch / (ms_step / 1e3)
    step_bytes = decode_bytes(model, runner, lengths)
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- end to end through the entry point: host ids in, host ids out
    gen = torch.Generator().manual_seed(2)
    e2e_new = args.steps + 1
    prompt_len = args.context - e2e_new
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in range(args.batch)]
    res = eng.generate(prompts, max_tokens=e2e_new, stop_ids=[])
    st = eng.stats
    e2e_value = st.generated_tokens / max(st.decode_secs, 1e-9)
    h2d = (8 * args.batch + 1) * 4
    d2h = args.batch * 4

    pts = {}
    if points:
        for b in (1, 64):
            ms_b, _, _ = time_decode(runner, b, args.context, min(args.steps, 16), 3, False, vocab, BatchSampler,
                                     SamplingParams)
            pts[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)

    line = {
        "metric": "decode tok/s at batch 8, context 8192 (Qwen3-8B shape, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": vocab, "global_batch": args.batch, "seq_len": args.context,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "cache_fill": args.fill,
            "points_cache_fill": "synthetic", "l2": "weights and cache read per step exceed L2 (no flush needed)",
            "peaks": f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})",
        },
        "clocks": clock_rec,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "generated": st.generated_tokens,
                "prefill_secs": round(st.prefill_secs, 3)},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (pre / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre, 3),
                    "frac": round(pre_frac, 4),
                    # the prompt is a 30 ms run of products under the power cap: also against the sustained rate
                    "frac_sustained": round(pre_frac * tflops / tflops_sustained, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "bytes_per_step": step_bytes},
        "points": pts,
    }
    assert all(len(r.tokens) == e2e_new for r in res)
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
