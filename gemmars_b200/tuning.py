"""Measurements that the dispatch rules rest on, to be run again on another GPU or another width.

    python -m gemmars_b200.tuning products [--shapes 4b,8b,32b] [--tokens 1,8,16,32,64]      (shapes: 0.6b 1.7b 4b 8b 14b 32b)
    python -m gemmars_b200.tuning timeline --shape 8b --batch 8 --context 8192 [--layers 6] [--prompt 2048]
                                           [--temperature 0.7]

``products``: every decode-shaped matrix product of a model shape (q/k/v, o, gate/up, down) with cold
weights, timed for every split of the inner dimension, beside the split ``kernels.gemm_tc_tiling``
picks by itself.  ``timeline``: the kernels of one replayed decode step (or, with ``--prompt``, of
one prompt step) as the device ran them, from CUPTI's kernel records: start, duration, and the gap
to the kernel before, which inside a replayed step is negative where dependent launch lets a kernel
start under its predecessor.  Both print plain text.
"""
from __future__ import annotations

import argparse
import re
import sys


def qwen3_shape(layers, hidden, heads, kv_heads, inter, tied):
    """A Qwen3 config.json object of the given layer sizes (heads of 128, the released vocabulary)."""
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
            "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
            "intermediate_size": inter, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "attention_bias": False, "tie_word_embeddings": tied, "max_position_embeddings": 40960}


# The layer sizes of the released Qwen3 dense models; the dispatch rules were measured at 4b, 8b and 32b.
SHAPES = {
    "8b": ("Qwen3-8B shape", qwen3_shape(36, 4096, 32, 8, 12288, False)),
    "4b": ("Qwen3-4B shape", qwen3_shape(36, 2560, 32, 8, 9728, True)),
    "32b": ("Qwen3-32B shape", qwen3_shape(64, 5120, 64, 8, 25600, False)),
    "0.6b": ("Qwen3-0.6B shape", qwen3_shape(28, 1024, 16, 8, 3072, True)),
    "1.7b": ("Qwen3-1.7B shape", qwen3_shape(28, 2048, 16, 8, 6144, True)),
    "14b": ("Qwen3-14B shape", qwen3_shape(40, 5120, 40, 8, 17408, False)),
}


def random_engine(cfg, max_batch, cache_tokens, options=""):
    """An engine over random weights of ``cfg`` made on the device; the tensors are taken out of
    their dict as they are bound, so that a model of 65 GB and its stacked q/k/v and gate/up copies
    never sit in memory side by side."""
    import torch
    from .engine.engine import Engine, EngineOptions
    from .weights.random_init import random_weights
    torch.cuda.set_device(0)
    tensors = random_weights(cfg, seed=0, device="cuda:0")
    opts = EngineOptions.parse({"dtype": "bfloat16", "max_batch": str(max_batch), "max_tokens": str(cache_tokens),
                                "prefill_chunk": "2048"})
    for pair in filter(None, (p.strip() for p in options.split(";"))):
        opts.set(*[x.strip() for x in pair.split("=", 1)])
    return Engine.from_config(cfg, tensors, opts, consume=True)


def synthetic_fill(runner, slots, length):
    """Brings every slot to ``length`` cached tokens by reserving the pages and writing random
    keys and values (what a timing needs of a cache, without running prompts)."""
    for s in slots:
        runner.cache.extend(s, length)
    runner.cache.sync()
    for g in runner.cache.kv_groups:
        for t in (g.k, g.v):
            for layer in range(t.shape[0]):
                t[layer].normal_(0.0, 1.0)


# ---------------------------------------------------------------------------------------- products

def sweep_products(shapes, tokens, hbm_gbs=6542.0, out=sys.stdout):
    import torch
    from . import kernels
    torch.manual_seed(0)
    for name in shapes:
        cfg = SHAPES[name][1]
        h, hd = cfg["hidden_size"], cfg["head_dim"]
        qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * hd
        ao, inter = cfg["num_attention_heads"] * hd, cfg["intermediate_size"]
        products = [("qkv", qkv, h, "bf16"), ("o", h, ao, "acc"), ("gate_up", inter, h, "gated"), ("down", h, inter, "acc")]
        for m in tokens:
            for what, n, k, mode in products:
                rows = 2 * n if mode == "gated" else n
                copies = max(2, int(1.0e9 // (rows * k * 2)))          # more weights than L2 holds: every launch reads cold
                ws = [torch.randn(rows, k, device="cuda").bfloat16() for _ in range(copies)]
                x = torch.randn(m, k, device="cuda").bfloat16()
                y = torch.zeros(m, n, device="cuda", dtype=torch.float32 if mode == "acc" else torch.bfloat16)
                auto = kernels.gemm_tc_tiling(m, n, k, gated=(mode == "gated"))
                res = []
                for splits in (1, 2, 4, 8):
                    if k // 64 // splits < 2:
                        continue

                    def run():
                        for w in ws:
                            kernels.gemm_tc(x, w, y, accumulate=(mode == "acc"), splits=splits, swiglu=(mode == "gated"))
                    run()
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        run()
                    g.replay()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5):
                        g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    res.append((e0.elapsed_time(e1) * 1e3 / 5 / copies, splits))
                best = min(res)
                ideal = rows * k * 2 / hbm_gbs / 1e3
                chosen = dict((sp, us) for us, sp in res).get(auto[1], float("nan"))
                print(f"{name:3s} {m:3d} tokens {what:8s} {rows:6d} x {k:5d}  bytes take {ideal:6.1f} us | "
                      + " ".join(f"x{sp}: {us:6.1f}" for us, sp in res)
                      + f" | best x{best[1]} {best[0]:6.1f} us | chosen x{auto[1]} (tile {auto[0]}) {chosen:6.1f} us", file=out, flush=True)
                del ws
    kernels.check_status()


# ---------------------------------------------------------------------------------------- timeline

def _short(name: str) -> str:
    name = name.replace("void ", "").replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
    m = re.match(r"([A-Za-z0-9_]+)(<[^>]*>)?", name)
    return ((m.group(1) + (m.group(2) or "")) if m else name)[:46]


def timeline(shape, batch, context, layers, prompt, temperature, out=sys.stdout):
    import torch
    from torch.profiler import ProfilerActivity, profile
    from .engine.step import StepItem
    from .sampling.sampler import BatchSampler, SamplingParams
    label, cfg = SHAPES[shape]
    cfg = dict(cfg, num_hidden_layers=layers or cfg["num_hidden_layers"])
    eng = random_engine(cfg, max(batch, 1), max(batch, 1) * (max(context, prompt) + 128))
    runner, vocab = eng.runner, cfg["vocab_size"]
    if prompt:
        toks = torch.randint(0, vocab, (prompt,), generator=torch.Generator().manual_seed(3)).tolist()

        def step():
            s = runner.open()
            runner.step([StepItem(s, toks, [prompt - 1])])
            torch.cuda.synchronize()
            runner.close(s)
        what = f"prompt of {prompt} tokens"
    else:
        slots = [runner.open() for _ in range(batch)]
        synthetic_fill(runner, slots, context - 50)
        sampler = BatchSampler([SamplingParams(temperature=temperature)] * batch, runner.device)
        rows = list(range(batch))
        state = {"logits": runner.step([StepItem(s, [5], [0]) for s in slots])}

        def step():
            # as the generation loop steps: draw, launch the next step from the drawn tokens where
            # they lie, then read them on the host
            drawn = sampler.draw(state["logits"], rows)
            nxt = runner.decode_from_device(slots, drawn) if eng.options.decode_ahead else None
            toks = sampler.read(drawn)
            state["logits"] = nxt if nxt is not None else runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
        what = f"decode step, batch {batch}, context {context}" + (f", temperature {temperature}" if temperature > 0 else "")
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(8):
        step()
    e1.record()
    torch.cuda.synchronize()
    print(f"{label}, {cfg['num_hidden_layers']} layers, {what}: {e0.elapsed_time(e1) / 8 * 1e3:.1f} us a step "
          "(CUDA events, host turnaround included)", file=out)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Memset" not in e.name]
    ev.sort(key=lambda e: e.time_range.start)
    last = ev[-(len(ev) // 3):]
    t0, prev_end, rows = last[0].time_range.start, last[0].time_range.start, []
    for e in last:
        rows.append((_short(e.name), e.time_range.start - t0, e.time_range.end - e.time_range.start,
                     e.time_range.start - prev_end))
        prev_end = max(prev_end, e.time_range.end)
    print(f"{len(rows)} kernels and copies in the step, {last[-1].time_range.end - t0:.1f} us from the first start to the last end", file=out)
    mid = len(rows) // 2
    print("-- the middle of the step (us: start, duration, gap to the end of everything before)", file=out)
    for name, s, d, gap in rows[max(0, mid - 6): mid + 12]:
        print(f"{name:46s} {s:9.1f} {d:8.1f} {gap:7.1f}", file=out)
    print("-- the end of the step", file=out)
    for name, s, d, gap in rows[-8:]:
        print(f"{name:46s} {s:9.1f} {d:8.1f} {gap:7.1f}", file=out)
    print("-- per kernel (calls, sum and mean of durations, sum of gaps)", file=out)
    tot = {}
    for name, s, d, gap in rows:
        a = tot.setdefault(name, [0, 0.0, 0.0])
        a[0] += 1
        a[1] += d
        a[2] += gap
    for k, (n, d, g) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
        print(f"{k:46s} {n:4d} {d:9.1f} {d / n:8.1f} {g:8.1f}", file=out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m gemmars_b200.tuning", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("products", help="decode-shaped products at every split, with cold weights")
    p.add_argument("--shapes", default="4b,8b,32b")
    p.add_argument("--tokens", default="1,8,16,32,64")
    t = sub.add_parser("timeline", help="the kernels of one replayed decode step or one prompt step")
    t.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=8192)
    t.add_argument("--layers", type=int, default=6, help="layers of the model that is built (0: all)")
    t.add_argument("--prompt", type=int, default=0, help="time a prompt of this many tokens instead of a decode step")
    t.add_argument("--temperature", type=float, default=0.0)
    args = ap.parse_args(argv)
    if args.command == "products":
        sweep_products([s.strip() for s in args.shapes.split(",")], [int(x) for x in args.tokens.split(",")])
    else:
        timeline(args.shape, args.batch, args.context, args.layers, args.prompt, args.temperature)
    return 0


if __name__ == "__main__":
    sys.exit(main())
