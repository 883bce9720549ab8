"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds the model
with ``build_model`` and drives ``Runner.step``, the same objects generation uses.

Input, one JSON object a line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the places among them whose logits are
wanted; ``end`` names the requests that are finished after the step (their slot and pages are
given back).  For a step in which something is wanted, ``<out>/<step>.f32`` receives the
logits as little-endian float32 [wanted, vocab], in the order of the entries and of ``want``.
After every step a line ``done <step>`` is printed and flushed.

Reference analogue: ``--dump-logits`` (src/main.rs:778-791) with tools/ref_logits.py.
"""
from __future__ import annotations

import json
import os
import sys

import torch

from .. import kernels
from ..cache.pool import PAGE_SIZE
from .model import build_model
from .step import Runner, StepItem


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines=None, report=None,
           device: str = "cuda:0") -> int:
    lines = sys.stdin if lines is None else lines
    report = sys.stdout if report is None else report
    if not torch.cuda.is_available():
        raise RuntimeError("trace_run needs a CUDA device: the engine has no CPU path")
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    os.makedirs(out_dir, exist_ok=True)
    model = build_model(model_dir, dtype=dtype, device=device)
    pages = max(1, -(-max_tokens // PAGE_SIZE))
    runner = Runner(model, max_tokens=max_tokens, max_batch=min(pages, 4096))
    slots = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        items = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = runner.open()
            items.append(StepItem(slots[rid], e["tokens"], e.get("want", [])))
        if items:
            logits = runner.step(items)
            if logits is not None:
                data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                kernels.check_status()
                with open(os.path.join(out_dir, f"{rec['step']}.f32"), "wb") as f:
                    f.write(data.tobytes())
        for rid in rec.get("end", []):
            if rid in slots:
                runner.close(slots.pop(rid))
        report.write(f"done {rec['step']}\n")
        report.flush()
    return 0
