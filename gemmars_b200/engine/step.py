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
        self.steps_run = 0
        self.launch_count = 0

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
