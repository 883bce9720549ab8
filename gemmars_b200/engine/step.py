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
import gc
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.pool import CacheError, SequenceCache
from ..csrc import build
from ..parts.base import StepContext
from .model import DecoderModel


class StepError(ValueError):
    pass


@dataclasses.dataclass
class StepItem:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are asked for


class _PinnedRing:
    """A few pinned host buffers used in turn for the step's index block; a buffer is written
    again only after the copy that last read it has finished.  They are allocated once, for the
    largest step, since pinning memory takes about a millisecond."""

    def __init__(self, capacity: int, n: int = 4):
        self.bufs = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(n)]
        self.views = [b.numpy() for b in self.bufs]
        self.events = [None] * n
        self.turn = 0

    def stage(self, values: np.ndarray, device) -> torch.Tensor:
        i = self.turn
        self.turn = (i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i].numel() < values.size:
            self.bufs[i] = torch.empty(2 * values.size, dtype=torch.int32).pin_memory()
            self.views[i] = self.bufs[i].numpy()
        self.views[i][:values.size] = values
        dev = self.bufs[i][:values.size].to(device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


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
        self._length_matters = model.capture_depends_on_length
        self._broken = set()      # slots a failed step left in a state that cannot be restored
        self._ring = _PinnedRing(4 * self.max_step_tokens + 8 * self.cache.n_slots + 64) if self.device.type == "cuda" else None
        self.steps_run = 0
        self.tokens_run = 0

    def _graph_pool(self):
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        return self._pool

    # ---- sequences
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)
        self._broken.discard(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # ---- the step
    def step(self, items: Sequence[StepItem]) -> Optional[torch.Tensor]:
        """Runs the items' tokens; returns float32 logits [wanted, vocab] in the order of the
        items and of each item's ``want`` (None when nothing is wanted)."""
        items = list(items)
        seen = set()
        toks = []
        for it in items:
            if it.slot in seen:
                raise StepError(f"slot {it.slot} appears twice in one step")
            seen.add(it.slot)
            if it.slot not in self.cache.lengths:
                raise StepError(f"slot {it.slot} is not open")
            if it.slot in self._broken:
                raise StepError(f"slot {it.slot} was left unfinished by a step that failed and can only be closed")
            t = np.asarray(it.tokens, dtype=np.int64).reshape(-1)
            if t.size == 0:
                raise StepError(f"slot {it.slot} brings no token")
            if t.min() < 0 or t.max() >= self.vocab_size:
                bad = int(t[(t < 0) | (t >= self.vocab_size)][0])
                raise StepError(f"token id {bad} is outside the vocabulary (0..{self.vocab_size - 1})")
            for w in it.want:
                if not 0 <= int(w) < t.size:
                    raise StepError(f"wanted place {w} is outside the {t.size} tokens of slot {it.slot}")
            toks.append(t)
        if not self.cache.can_extend([(it.slot, t.size) for it, t in zip(items, toks)]):
            raise CacheError("the step does not fit in the cache "
                             f"({sum(t.size for t in toks)} new tokens; "
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
        before = {it.slot: self.cache.lengths[it.slot] for it in items}
        try:
            while True:
                # one sub-step: up to prefill_chunk tokens of each unfinished sequence, within the budget
                budget, part = self.max_step_tokens, []
                for i, t in enumerate(toks):
                    left = t.size - done[i]
                    if left <= 0 or budget <= 0:
                        continue
                    n = min(left, self.prefill_chunk, budget)
                    part.append((i, done[i], n))
                    budget -= n
                if not part:
                    break
                self._run(items, toks, part, out, out_base)
                for i, _, n in part:
                    done[i] += n
        except BaseException:
            # The step is all or nothing: the lengths go back to what they were, so that they never
            # name positions no kernel wrote.  What cannot be taken back (a window's ring written
            # over, a state advanced) leaves the slot fit only for closing.
            for slot, old in before.items():
                if slot in self.cache.lengths and not self.cache.rollback(slot, old):
                    self._broken.add(slot)
            raise
        self.steps_run += 1
        self.tokens_run += sum(t.size for t in toks)
        return out

    def _run(self, items, toks, part, out, out_base):
        cache = self.cache
        b = len(part)
        slots = np.empty(b, dtype=np.int64)
        starts = np.empty(b, dtype=np.int64)
        lens = np.empty(b, dtype=np.int64)
        rows, dest = [], []
        base = 0
        for k, (i, off, n) in enumerate(part):
            it = items[i]
            slots[k], starts[k], lens[k] = it.slot, cache.extend(it.slot, n), n
            for j, w in enumerate(it.want):
                if off <= w < off + n:
                    rows.append(base + (w - off))
                    dest.append(out_base[i] + j)
            base += n
        cache.sync()
        t = base
        max_total = int((starts + lens).max())
        contiguous = bool(dest) and dest == list(range(dest[0], dest[0] + len(dest)))
        if self.use_graphs and t == b and len(rows) == b and rows == list(range(b)):
            # every sequence brings one token and wants its logits: replay the captured step
            tokens = np.fromiter((toks[i][off] for i, off, _ in part), dtype=np.int64, count=b)
            logits = self._decode_graph(tokens, starts, slots, max_total)
            if contiguous:
                out[dest[0]:dest[0] + b].copy_(logits)
            else:
                out[torch.tensor(dest, device=self.device)] = logits
            return
        cu = np.zeros(b + 1, dtype=np.int64)
        np.cumsum(lens, out=cu[1:])
        tok_seq = np.repeat(np.arange(b), lens)
        tok_pos = np.arange(t) - cu[tok_seq] + starts[tok_seq]
        tokens = np.concatenate([toks[i][off:off + n] for i, off, n in part])
        block = np.concatenate([tokens, tok_pos, tok_seq, slots, starts, lens, cu,
                                np.asarray(rows, dtype=np.int64)]).astype(np.int32)
        dev = self._ring.stage(block, self.device)
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
            is_decode=bool((lens == 1).all()), max_new=int(lens.max()), max_total=max_total, cache=cache,
            page_size=cache.page_size,
            host={"seq_slot": slots.tolist(), "seq_start": starts.tolist(), "seq_len": lens.tolist()})
        # the builds whose kernels start under the tail of the kernel before them
        build.set_pdl(True)
        try:
            x = self.model.forward(ctx, d_tokens)
            logits = self.model.logits(ctx, x, d_rows) if rows else None
        finally:
            build.set_pdl(False)
        if rows:
            if contiguous:
                out[dest[0]:dest[0] + len(dest)].copy_(logits)
            else:
                out[torch.tensor(dest, device=self.device)] = logits

    def decode_from_device(self, slots: Sequence[int], tokens: torch.Tensor) -> Optional[torch.Tensor]:
        """One more token for each sequence in ``slots``, the tokens being an int32 tensor on the
        device (what the sampler has just drawn and the host has not read yet): the step is
        launched without waiting for them, so that the device goes on while the host reads and
        judges the tokens of the step before.  Returns float32 logits [len(slots), vocab], or None
        when the step cannot be run this way (no captured steps, or the cache cannot take it):
        the caller then runs an ordinary step.  A token id outside the vocabulary cannot be
        refused here; the embedding reads the nearest row that exists."""
        slots = [int(s) for s in slots]
        b = len(slots)
        if (not self.use_graphs or b == 0 or tokens.device != self.device or tokens.dtype != torch.int32
                or tokens.numel() != b or len(set(slots)) != b):
            return None
        if any(s not in self.cache.lengths or s in self._broken for s in slots):
            return None
        if not self.cache.can_extend([(s, 1) for s in slots]):
            return None
        before = {s: self.cache.lengths[s] for s in slots}
        try:
            starts = np.fromiter((self.cache.extend(s, 1) for s in slots), dtype=np.int64, count=b)
            self.cache.sync()
            logits = self._decode_graph(tokens, starts, np.asarray(slots, dtype=np.int64), int(starts.max()) + 1)
            out = torch.empty((b, self.vocab_size), dtype=torch.float32, device=self.device)
            out.copy_(logits)
        except BaseException:
            for slot, old in before.items():
                if slot in self.cache.lengths and not self.cache.rollback(slot, old):
                    self._broken.add(slot)
            raise
        self.steps_run += 1
        self.tokens_run += b
        return out

    # ---- decode steps replayed from CUDA graphs
    def _decode_graph(self, tokens, starts, slots, max_total):
        """One token per sequence through a captured graph.  The batch is padded to a power of
        two with rows that belong to no sequence: their slot is the spare one (``ctx.pad_slot``:
        the last row of every page table, all page 0, and of every state tensor), so what they
        write lands where no sequence reads and they change no result."""
        b = len(tokens)
        bp = 1
        while bp < b:
            bp *= 2
        # one graph per padded batch size; per length bucket as well only when some part's launches
        # depend on the longest sequence (then ``ctx.max_total`` of the captured step is the bucket)
        len_bucket = 256 if self._length_matters else self.cache.max_seq_len
        while len_bucket < max_total:
            len_bucket *= 2
        key = (bp, len_bucket)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = _DecodeGraph(self, bp, len_bucket)
        return g.run(tokens, starts, slots)[:b]


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
        self.host_np = [h.numpy() for h in self.host]
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
        fixed = np.zeros(self.n, dtype=np.int32)
        fixed[2 * bp:3 * bp] = np.arange(bp)               # tok_seq
        fixed[3 * bp:4 * bp] = pad_slot                     # seq_slot of padding rows
        fixed[5 * bp:6 * bp] = 1                            # seq_len
        fixed[6 * bp:7 * bp + 1] = np.arange(bp + 1)        # cu_seqlens
        fixed[7 * bp + 1:8 * bp + 1] = np.arange(bp)        # wanted rows
        self.fixed = fixed
        self.meta.copy_(torch.from_numpy(fixed))
        model = runner.model
        self.ctx = StepContext(
            compute=model.compute, act_dtype=model.act_dtype, device=dev, n_tokens=bp, n_seqs=bp,
            tok_pos=self.d_pos, tok_seq=self.d_seq, seq_slot=self.d_slot, seq_start=self.d_start, seq_len=self.d_len,
            cu_seqlens=self.d_cu, is_decode=True, max_new=1, max_total=len_bucket, cache=runner.cache,
            page_size=runner.cache.page_size, pad_slot=pad_slot)
        # once eagerly (loads the kernels, warms the allocator), then captured
        build.set_pdl(True)
        try:
            torch.cuda.synchronize(dev)
            self._forward()
            torch.cuda.synchronize(dev)
            before = kernels.launch_count()
            self.graph = torch.cuda.CUDAGraph()
            # No graph of an earlier runner may be destroyed while this one is being captured (its
            # destructor frees device memory, which ends the capture with an error): collect what
            # is garbage now, and keep the collector from running inside the capture.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(self.graph, pool=runner._graph_pool()):
                    self.logits = self._forward()
            finally:
                if gc_was_on:
                    gc.enable()
            self.launches = kernels.launch_count() - before
        finally:
            build.set_pdl(False)

    def _forward(self):
        model = self.runner.model
        x = model.forward(self.ctx, self.d_tokens)
        return model.logits(self.ctx, x, self.d_rows)

    def run(self, tokens, starts, slots):
        from .. import kernels
        b, bp = len(tokens), self.bp
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()       # the copy that last read this host buffer is done
        h = self.host_np[i]
        h[:] = self.fixed
        on_device = isinstance(tokens, torch.Tensor)
        if not on_device:
            h[0:b] = tokens
        h[bp:bp + b] = starts                  # the token's position is the length before the step
        h[3 * bp:3 * bp + b] = slots
        h[4 * bp:4 * bp + b] = starts
        self.meta.copy_(self.host[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        if on_device:
            self.d_tokens[:b].copy_(tokens)    # in stream order after the block above and after the sampler
        self.graph.replay()
        kernels.count_launches(self.launches)
        return self.logits
