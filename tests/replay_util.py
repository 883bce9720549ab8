"""Builds traces for bin/trace_run, runs it as a user would, and reads its output back."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """Collects steps and remembers which (request, position) each written row holds."""

    def __init__(self):
        self.steps, self.rows = [], {}

    def step(self, entries, end=()):
        """entries: [(id, tokens, first position of these tokens, want places)]."""
        n = len(self.steps)
        rows = [(rid, pos0 + w) for rid, toks, pos0, want in entries for w in want]
        if rows:
            self.rows[n] = rows
        self.steps.append({"step": n, "entries": [{"id": rid, "tokens": list(map(int, toks)), "want": list(want)}
                                                   for rid, toks, pos0, want in entries], "end": list(end)})

    # ---- the three ways of cutting the same requests
    def whole(self, tag, requests):
        """Each request alone and whole, one after the other."""
        for i, toks in enumerate(requests):
            rid = f"{tag}{i}"
            self.step([(rid, toks, 0, range(len(toks)))], end=[rid])

    def tail(self, tag, requests, n_tail=32):
        """All but the last n_tail tokens in one step, then the last n_tail one by one."""
        for i, toks in enumerate(requests):
            rid = f"{tag}{i}"
            head = max(1, len(toks) - n_tail)
            self.step([(rid, toks[:head], 0, range(head))])
            for p in range(head, len(toks)):
                self.step([(rid, [toks[p]], p, [0])], end=[rid] if p == len(toks) - 1 else [])
            if head == len(toks):
                self.step([], end=[rid])

    def batches(self, tag, requests, groups, prompt_lens):
        """groups: lists of request indices that start together, one group after another.
        Request i brings prompt_lens[i] tokens in the first step, then one token a step; a
        request that runs out of tokens ends and the batch goes on without it."""
        for g in groups:
            ids = {i: f"{tag}{i}" for i in g}
            first = [(ids[i], requests[i][:prompt_lens[i]], 0, range(prompt_lens[i])) for i in g]
            done = [ids[i] for i in g if prompt_lens[i] == len(requests[i])]
            self.step(first, end=done)
            pos = {i: prompt_lens[i] for i in g if prompt_lens[i] < len(requests[i])}
            while pos:
                entries = [(ids[i], [requests[i][p]], p, [0]) for i, p in pos.items()]
                ended = [ids[i] for i, p in pos.items() if p + 1 == len(requests[i])]
                self.step(entries, end=ended)
                pos = {i: p + 1 for i, p in pos.items() if p + 1 < len(requests[i])}

    def max_tokens(self):
        """The most tokens live requests hold at any time, each rounded up to 64."""
        live, worst = {}, 0
        for s in self.steps:
            for e in s["entries"]:
                live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
            worst = max(worst, sum(-(-n // 64) * 64 for n in live.values()))
            for rid in s["end"]:
                live.pop(rid, None)
        return worst

    def text(self):
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def run_trace(trace, model_dir, dtype, out_dir, max_tokens=None, timeout=600, env=None):
    """Runs bin/trace_run on the trace; returns {(request id, position): logits row}."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or trace.max_tokens())]
    p = subprocess.run(cmd, input=trace.text(), capture_output=True, text=True, timeout=timeout, env=env)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(trace.steps))], "a 'done <step>' line is missing or out of order"
    out = {}
    for n, rows in trace.rows.items():
        data = np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4")
        assert data.size % len(rows) == 0, f"step {n}: file size does not fit {len(rows)} rows"
        data = data.reshape(len(rows), -1)
        for r, key in zip(data, rows):
            assert key not in out
            out[key] = r
    return out
