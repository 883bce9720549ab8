"""Command line, in the manner of the reference's ``oxinfer`` (src/main.rs:82-168, 170-352).

Options the reference has keep their names and meanings: ``--model/-m``, ``--prompt/-p`` (else
standard input), ``--raw``, ``--max-tokens/-n`` (1024), ``--temp/-t`` (0 = greedy), ``--top-k``
(64), ``--top-p`` (0.95), ``--seed`` (42), ``--prefill-chunk``, ``--profile``,
``--dump-logits FILE`` (float32 little-endian logits of the last prompt token, then exit;
src/main.rs:778-791), ``--show-tokens``, ``--print-prompt``, ``--chat``, ``--system``,
``--no-system``, ``--think``, ``--device``, ``--devices``.  Added here: ``--tokens`` and
``--tokens-file`` (ids in, ids out, no tokenizer needed), ``--batch-file`` (one prompt of ids a
line, generated as batches), ``--dtype``, ``--options`` and ``--random-weights`` (write a model
folder from ``--config`` and ``--seed``, then exit).
"""
from __future__ import annotations

import argparse
import json
import sys

END_OF_TURN = "<|im_end|>"


def chat_prompt(system, user, think):
    """Qwen3's ChatML turn (src/chat.rs:216-238, 296-302)."""
    s = f"<|im_start|>system\n{system}<|im_end|>\n" if system else ""
    tail = "" if think else "<think>\n\n</think>\n\n"
    return s + f"<|im_start|>user\n{user}<|im_end|>\n<|im_start|>assistant\n{tail}"


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gemmars_b200", description="Qwen3 text generation on one B200.")
    ap.add_argument("--model", "-m", help="model folder (config.json, model.safetensors)")
    ap.add_argument("--prompt", "-p", help="single prompt (default: read from stdin)")
    ap.add_argument("--chat", action="store_true", help="interactive multi-turn chat")
    ap.add_argument("--system", help="system prompt")
    ap.add_argument("--no-system", action="store_true", help="no system prompt")
    ap.add_argument("--print-prompt", action="store_true", help="print the formatted prompt and exit")
    ap.add_argument("--think", action="store_true", help="enable thinking mode")
    ap.add_argument("--raw", action="store_true", help="no chat template (prompt is fed as-is)")
    ap.add_argument("--max-tokens", "-n", type=int, default=1024, help="max new tokens (default 1024)")
    ap.add_argument("--temp", "-t", type=float, default=0.0, help="temperature, 0 = greedy (default 0)")
    ap.add_argument("--top-k", type=int, default=64, help="top-k (default 64)")
    ap.add_argument("--top-p", type=float, default=0.95, help="top-p (default 0.95)")
    ap.add_argument("--seed", type=int, default=42, help="RNG seed")
    ap.add_argument("--profile", action="store_true", help="print per-step timing")
    ap.add_argument("--prefill-chunk", type=int, help="tokens per prefill chunk (default 2048)")
    ap.add_argument("--devices", action="store_true", help="list CUDA devices, then exit")
    ap.add_argument("--device", default="auto", help="auto (default) | cuda | cuda:N")
    ap.add_argument("--dump-logits", metavar="FILE", help="write last-prompt-token logits (f32 LE) and exit")
    ap.add_argument("--show-tokens", action="store_true", help="print token ids")
    ap.add_argument("--tokens", help="prompt as comma-separated token ids (no tokenizer needed)")
    ap.add_argument("--tokens-file", help="file with the prompt's token ids (comma or space separated)")
    ap.add_argument("--batch-file", help="file with one prompt of token ids a line; generated in batches")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--options", default="", help='engine options "key=value;key=value"')
    ap.add_argument("--random-weights", metavar="DIR", help="write a random model folder from --config, then exit")
    ap.add_argument("--config", help="config.json for --random-weights")
    return ap


def _ids(text):
    return [int(x) for x in text.replace(",", " ").split()]


def main(argv=None) -> int:
    args = parser().parse_args(argv)
    if args.devices:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
        for i in range(n):
            p = torch.cuda.get_device_properties(i)
            print(f"cuda:{i} {p.name} sm_{p.major}{p.minor} {p.total_memory / 2**30:.0f} GiB {p.multi_processor_count} SMs")
        if n == 0:
            print("no CUDA device")
        return 0
    if args.random_weights:
        if not args.config:
            print("--random-weights needs --config FILE", file=sys.stderr)
            return 2
        from .weights.random_init import write_random_model
        with open(args.config) as f:
            write_random_model(args.random_weights, json.load(f), args.seed)
        print(f"wrote {args.random_weights}", file=sys.stderr)
        return 0
    if not args.model:
        parser().print_usage(sys.stderr)
        return 2

    from .engine.engine import Engine, EngineOptions
    from .engine.step import StepItem
    opts = EngineOptions.parse(args.options)
    opts.set("dtype", args.dtype)
    opts.set("device", args.device)
    if args.prefill_chunk:
        opts.set("prefill_chunk", str(args.prefill_chunk))
    if args.profile:
        opts.set("profile", "true")
    eng = Engine.load(args.model, opts)
    if args.profile:
        eng.profile_start()
    for k, v in (("max_tokens", args.max_tokens), ("temperature", args.temp), ("top_k", args.top_k),
                 ("top_p", args.top_p), ("seed", args.seed)):
        eng.set(k, v)

    if args.batch_file:
        with open(args.batch_file) as f:
            prompts = [_ids(line) for line in f if line.strip()]
        for r in eng.generate(prompts):
            print(json.dumps({"tokens": r.tokens, "reason": r.reason}))
        print(eng.stats.line(), file=sys.stderr)
        if args.profile:
            print(eng.profile_report(), file=sys.stderr)
        return 0

    by_ids = bool(args.tokens or args.tokens_file)
    tok = None if by_ids else eng.tokenizer()
    if tok is not None and tok.token_to_id(END_OF_TURN) is not None and not args.raw:
        end = tok.token_to_id(END_OF_TURN)       # src/chat.rs:430-437
        if end not in eng.stop_ids:
            eng.stop_ids.append(end)
    system = None if args.no_system else args.system

    def encode(text, first):
        if args.raw:
            return tok.encode(text, add_special_tokens=False).ids
        return tok.encode(chat_prompt(system if first else None, text, args.think), add_special_tokens=False).ids

    def show(ids):
        if tok is None or args.show_tokens:
            print(",".join(str(i) for i in ids))
        if tok is not None:
            print(tok.decode(ids))

    if args.chat:
        first = True
        while True:
            try:
                line = input("> ")
            except EOFError:
                break
            if not line.strip():
                continue
            ids = _ids(line) if by_ids else encode(line, first)
            if not first and tok is not None and not args.raw:
                ids = tok.encode(END_OF_TURN + "\n", add_special_tokens=False).ids + ids
            first = False
            r = eng.send(ids)
            show(r.tokens)
            print(eng.stats.line(), file=sys.stderr)
        return 0

    if args.tokens:
        ids = _ids(args.tokens)
    elif args.tokens_file:
        with open(args.tokens_file) as f:
            ids = _ids(f.read())
    else:
        text = args.prompt if args.prompt is not None else sys.stdin.read()
        if args.print_prompt:
            print(text if args.raw else chat_prompt(system, text, args.think))
            return 0
        ids = encode(text, True)
    if args.show_tokens:
        print("prompt:", ",".join(str(i) for i in ids), file=sys.stderr)
    if args.dump_logits:
        slot = eng.runner.open()
        logits = eng.runner.step([StepItem(slot, ids, [len(ids) - 1])])[0].cpu().numpy().astype("<f4")
        eng.runner.close(slot)
        with open(args.dump_logits, "wb") as f:
            f.write(logits.tobytes())
        top = sorted(range(len(logits)), key=lambda i: -logits[i])[:10]
        print("top 10:", " ".join(f"{i}:{logits[i]:.4f}" for i in top), file=sys.stderr)
        return 0
    r = eng.send(ids)
    show(r.tokens)
    print(eng.stats.line(), file=sys.stderr)
    if args.profile:
        print(eng.profile_report(), file=sys.stderr)
    return 0
