"""The step function: one batch of sequences through the model, from the cache.

``Runner.step`` takes, for each sequence of the batch, its slot and the next tokens it brings
(a whole prompt, or one decoded token; lengths may differ), runs exactly those tokens as one
packed batch against what earlier steps left in the cache, appends their keys and values, and
returns float32 logits at the places asked for.  Nothing else is computed: no padding token
is run, and the result at a position does not depend on how the tokens were cut into steps or
on which other sequences share the batch.

The reference runs one sequence per call (``forward_hidden_mm`` appends T tokens at
``sess.pos``, src/qwen.rs:647-701; ``logits`` src/qwen.rs:632-638); the batch of sequences
that start together and the requested rows are this engine's own.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple

import torch

from ..cache.pool import CacheError, SequenceCache
from ..parts.base import StepContext
from .model import DecoderModel


class StepError(ValueError):
    pass


@dataclasses.dataclass
class StepItem:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are asked for


class Runner:
    """A model with its cache: opens and closes sequences and runs steps."""

    def __init__(self, model: DecoderModel, max_tokens: int, max_batch: int = 256,
                 prefill_chunk: int = 2048, max_step_tokens: int = 16384, use_graphs: bool = True):
        self.model = model
        self.device = model.device
        self.prefill_chunk = max(1, prefill_chunk)
        self.max_step_tokens = max(self.prefill_chunk, max_step_tokens)
        self.cache = SequenceCache(model.cache_needs(), max_tokens, max_batch, model.plan.max_positions,
                                   self.prefill_chunk, model.act_dtype, self.device)
        self.vocab_size = model.plan.vocab_size
        self.use_graphs = use_graphs
        self._graphs = {}
        self._pool = None
        self.steps_run = 0
        self.launch_count = 0

    def _graph_pool(self):
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        return self._pool

    # ---- sequences
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # ---- the step
    def step(self, items: Sequence[StepItem]) -> Optional[torch.Tensor]:
        """Runs the items' tokens; returns float32 logits [wanted, vocab] in the order of the
        items and of each item's ``want`` (None when nothing is wanted)."""
        items = list(items)
        seen = set()
        for it in items:
            if it.slot in seen:
                raise StepError(f"slot {it.slot} appears twice in one step")
            seen.add(it.slot)
            if it.slot not in self.cache.lengths:
                raise StepError(f"slot {it.slot} is not open")
            if len(it.tokens) == 0:
                raise StepError(f"slot {it.slot} brings no token")
            for t in it.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise StepError(f"token id {t} is outside the vocabulary (0..{self.vocab_size - 1})")
            for w in it.want:
                if not 0 <= int(w) < len(it.tokens):
                    raise StepError(f"wanted place {w} is outside the {len(it.tokens)} tokens of slot {it.slot}")
        if not self.cache.can_extend([(it.slot, len(it.tokens)) for it in items]):
            raise CacheError("the step does not fit in the cache "
                             f"({sum(len(it.tokens) for it in items)} new tokens; "
                             f"longest sequence allowed {self.cache.max_seq_len})")
        n_want = sum(len(it.want) for it in items)
        out = (torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
               if n_want else None)
        # where each item's wanted rows go in the output
        out_base, acc = [], 0
        for it in items:
            out_base.append(acc)
            acc += len(it.want)
        done = [0] * len(items)
        while True:
            # one sub-step: up to prefill_chunk tokens of each unfinished sequence, within the budget
            budget, part = self.max_step_tokens, []
            for i, it in enumerate(items):
                left = len(it.tokens) - done[i]
                if left <= 0 or budget <= 0:
                    continue
                n = min(left, self.prefill_chunk, budget)
                part.append((i, done[i], n))
                budget -= n
            if not part:
                break
            self._run(items, part, out, out_base)
            for i, _, n in part:
                done[i] += n
        self.steps_run += 1
        return out

    def _run(self, items, part, out, out_base):
        cache = self.cache
        tokens, tok_pos, tok_seq, seq_slot, seq_start, seq_len, cu = [], [], [], [], [], [], [0]
        rows, dest = [], []
        max_total = 0
        for b, (i, off, n) in enumerate(part):
            it = items[i]
            start = cache.extend(it.slot, n)
            tokens.extend(int(t) for t in it.tokens[off:off + n])
            tok_pos.extend(range(start, start + n))
            tok_seq.extend([b] * n)
            seq_slot.append(it.slot)
            seq_start.append(start)
            seq_len.append(n)
            for j, w in enumerate(it.want):
                if off <= w < off + n:
                    rows.append(cu[-1] + (w - off))
                    dest.append(out_base[i] + j)
            cu.append(cu[-1] + n)
            max_total = max(max_total, start + n)
        cache.sync()
        t, b = len(tokens), len(part)
        if self.use_graphs and t == b and len(rows) == b and rows == list(range(b)):
            # every sequence brings one token and wants its logits: replay the captured step
            logits = self._decode_graph(tokens, tok_pos, seq_slot, seq_start, max_total)
            if dest == list(range(dest[0], dest[0] + b)):
                out[dest[0]:dest[0] + b].copy_(logits)
            else:
                out[torch.tensor(dest, device=self.device)] = logits
            return
        host = torch.tensor(tokens + tok_pos + tok_seq + seq_slot + seq_start + seq_len + cu + rows,
                            dtype=torch.int32).pin_memory()
        dev = host.to(self.device, non_blocking=True)
        o = 0

        def take(n):
            nonlocal o
            v = dev[o:o + n]
            o += n
            return v

        d_tokens, d_pos, d_seq = take(t), take(t), take(t)
        d_slot, d_start, d_len, d_cu, d_rows = take(b), take(b), take(b), take(b + 1), take(len(rows))
        ctx = StepContext(
            compute=self.model.compute, act_dtype=self.model.act_dtype, device=self.device, n_tokens=t, n_seqs=b,
            tok_pos=d_pos, tok_seq=d_seq, seq_slot=d_slot, seq_start=d_start, seq_len=d_len, cu_seqlens=d_cu,
            is_decode=all(n == 1 for n in seq_len), max_new=max(seq_len), max_total=max_total, cache=cache,
            page_size=cache.page_size)
        x = self.model.forward(ctx, d_tokens)
        if rows:
            logits = self.model.logits(ctx, x, d_rows)
            if dest == list(range(dest[0], dest[0] + len(dest))):
                out[dest[0]:dest[0] + len(dest)].copy_(logits)
            else:
                out[torch.tensor(dest, device=self.device)] = logits

    # ---- decode steps replayed from CUDA graphs
    def _decode_graph(self, tokens, tok_pos, seq_slot, seq_start, max_total):
        """One token per sequence through a captured graph.  The batch is padded to a power of
        two with rows that belong to no sequence: they use the page table's spare row, write into
        page 0 and read nothing that a real row reads, so they change no result."""
        b = len(tokens)
        bp = 1
        while bp < b:
            bp *= 2
        len_bucket = 256
        while len_bucket < max_total:
            len_bucket *= 2
        key = (bp, len_bucket)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, bp, len_bucket)
        return g.run(tokens, tok_pos, seq_slot, seq_start)[:b]


class _DecodeGraph:
    """A captured decode step for a padded batch of ``bp`` rows and sequences up to ``len_bucket``
    long.  Index tensors live at fixed addresses; each run copies the step's values into them
    from pinned host memory and replays."""

    RING = 4

    def __init__(self, runner: "Runner", bp: int, len_bucket: int):
        from .. import kernels
        self.runner, self.bp = runner, bp
        dev = runner.device
        self.n = 8 * bp + 1
        self.meta = torch.zeros(self.n, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(self.n, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0
        m, o = self.meta, 0

        def take(n):
            nonlocal o
            v = m[o:o + n]
            o += n
            return v

        self.d_tokens, self.d_pos, self.d_seq = take(bp), take(bp), take(bp)
        self.d_slot, self.d_start, self.d_len, self.d_cu, self.d_rows = take(bp), take(bp), take(bp), take(bp + 1), take(bp)
        pad_slot = runner.cache.n_slots
        fixed = torch.zeros(self.n, dtype=torch.int32)
        fixed[2 * bp:3 * bp] = torch.arange(bp)            # tok_seq
        fixed[3 * bp:4 * bp] = pad_slot                     # seq_slot of padding rows
        fixed[5 * bp:6 * bp] = 1                            # seq_len
        fixed[6 * bp:7 * bp + 1] = torch.arange(bp + 1)     # cu_seqlens
        fixed[7 * bp + 1:8 * bp + 1] = torch.arange(bp)     # wanted rows
        self.fixed = fixed
        self.meta.copy_(fixed)
        model = runner.model
        self.ctx = StepContext(
            compute=model.compute, act_dtype=model.act_dtype, device=dev, n_tokens=bp, n_seqs=bp,
            tok_pos=self.d_pos, tok_seq=self.d_seq, seq_slot=self.d_slot, seq_start=self.d_start, seq_len=self.d_len,
            cu_seqlens=self.d_cu, is_decode=True, max_new=1, max_total=len_bucket, cache=runner.cache,
            page_size=runner.cache.page_size)
        # once eagerly (loads the kernels, warms the allocator), then captured
        torch.cuda.synchronize(dev)
        self._forward()
        torch.cuda.synchronize(dev)
        before = kernels.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=runner._graph_pool()):
            self.logits = self._forward()
        self.launches = kernels.launch_count() - before

    def _forward(self):
        model = self.runner.model
        x = model.forward(self.ctx, self.d_tokens)
        return model.logits(self.ctx, x, self.d_rows)

    def run(self, tokens, tok_pos, seq_slot, seq_start):
        from .. import kernels
        b, bp = len(tokens), self.bp
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()       # the copy that last read this host buffer is done
        h = self.host[i]
        h.copy_(self.fixed)
        h[0:b] = torch.tensor(tokens, dtype=torch.int32)
        h[bp:bp + b] = torch.tensor(tok_pos, dtype=torch.int32)
        h[3 * bp:3 * bp + b] = torch.tensor(seq_slot, dtype=torch.int32)
        h[4 * bp:4 * bp + b] = torch.tensor(seq_start, dtype=torch.int32)
        self.meta.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        self.graph.replay()
        kernels.count_launches(self.launches)
        return self.logits
