"""The generation loop: batches of prompts of unequal length, one batch after another.

For a batch: every prompt runs in one step, then each live sequence samples a token and runs
it, one token a step.  A sequence ends after a stop token (kept in its output, not run), after
its token limit, at the context limit, or when the callback says so; its slot is given back
at once and the batch goes on with the rest.  When the batch is empty the next requests start,
in slots that were used before.

The loop decides; it computes nothing.  It talks to the model through three callables
(``open``, ``close``, ``step``) and a sampler, so its decisions are tested without a GPU.

Reference: ``generate::decode`` (src/generate.rs:134-170) for one sequence: sample from the
current logits, push, stop check (the stop token is not run), callback, forward one token;
``StopReason`` {Stop, Length, Cancelled} (src/generate.rs:97-128); the limit of the context
(src/engine.rs:1046-1053, 1123-1126).  Batches are this engine's own.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable, List, Optional, Sequence

STOP, LENGTH, CANCELLED = "stop", "length", "cancelled"


@dataclasses.dataclass
class Request:
    prompt: Sequence[int]
    max_tokens: int = 1024            # src/main.rs:181
    stop_ids: Sequence[int] = ()
    sampling: object = None           # a SamplingParams; None: greedy defaults


@dataclasses.dataclass
class Generated:
    tokens: List[int]                 # generated tokens, the stop token included when one ended it
    reason: str                       # "stop", "length" or "cancelled"
    prompt_tokens: int
    forwards: int = 0                 # decode steps this sequence took part in
    #: the last generated token when it was not run and is no stop token: a later turn of the
    #: same sequence must feed it first (src/generate.rs:122-127)
    unfed: Optional[int] = None


def tokens_held(prompt_len: int, max_tokens: int, max_context: Optional[int]) -> int:
    """Most positions a request can come to hold in the cache: its prompt and every generated
    token that is run (the last generated token never is)."""
    n = prompt_len + max(0, max_tokens - 1)
    return min(n, max_context) if max_context else n


def plan_batches(requests: Sequence[Request], max_batch: int, cache_pages: int, page_size: int,
                 max_context: Optional[int] = None) -> List[List[int]]:
    """Splits the requests, in order, into batches of at most ``max_batch`` whose worst-case
    cache use fits ``cache_pages`` pages.  Raises if one request alone does not fit."""
    batches, cur, used = [], [], 0
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise ValueError(f"request {i}: empty prompt")
        if max_context and len(r.prompt) > max_context:
            raise ValueError(f"request {i}: prompt of {len(r.prompt)} tokens exceeds the context limit {max_context}")
        pages = -(-tokens_held(len(r.prompt), r.max_tokens, max_context) // page_size)
        if pages > cache_pages:
            raise ValueError(f"request {i}: needs {pages} cache pages of {page_size} tokens, the cache has {cache_pages}")
        if cur and (len(cur) >= max_batch or used + pages > cache_pages):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += pages
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    """``open() -> slot``, ``close(slot)``, ``step(list of (slot, tokens)) -> logits rows`` (one
    row per item: the logits after its last token) and ``make_sampler(list of sampling params)
    -> object with sample(logits, seq indices) -> token ids``."""

    def __init__(self, open_slot: Callable, close_slot: Callable, step: Callable, make_sampler: Callable,
                 max_batch: int, cache_pages: int, page_size: int, max_context: Optional[int] = None,
                 step_ahead: Optional[Callable] = None):
        """``step_ahead(slots, drawn) -> logits rows or None`` (optional): runs one token for each
        slot, the tokens being what the sampler's ``draw`` returned and nobody has read yet, so
        that the next step is on its way while this one's tokens are read and judged.  With it the
        sampler must have ``draw(logits, seq indices) -> drawn`` and ``read(drawn) -> token ids``."""
        self.open_slot, self.close_slot, self.step, self.make_sampler = open_slot, close_slot, step, make_sampler
        self.step_ahead = step_ahead
        self.ahead_steps = 0
        self.max_batch, self.cache_pages, self.page_size, self.max_context = max_batch, cache_pages, page_size, max_context
        self.decode_steps = 0
        self.prefill_steps = 0
        # wall time up to the first sampled tokens of each batch, and after (sampling reads the
        # tokens back to the host, so both include the device work they wait for)
        self.prefill_secs = 0.0
        self.decode_secs = 0.0
        self.decode_tokens = 0

    def run(self, requests: Sequence[Request],
            on_token: Optional[Callable[[int, List[int]], bool]] = None) -> List[Generated]:
        """Generates for every request; results in request order.  ``on_token(request index,
        tokens so far)`` is called for every token except a stop token; returning False ends
        that sequence (reason "cancelled")."""
        results: List[Optional[Generated]] = [None] * len(requests)
        for batch in plan_batches(requests, self.max_batch, self.cache_pages, self.page_size, self.max_context):
            self._run_batch(requests, batch, results, on_token)
        return results

    def run_in_slot(self, slot: int, held: int, request: Request,
                    on_token: Optional[Callable[[int, List[int]], bool]] = None) -> Generated:
        """One more turn of a sequence that lives on in ``slot``, which already holds ``held``
        positions: ``request.prompt`` is what the turn brings.  The slot stays open afterwards,
        whatever happens; the same decisions as for a batch apply."""
        if len(request.prompt) == 0:
            raise ValueError("the turn brings no token")
        if self.max_context and held + len(request.prompt) > self.max_context:
            raise ValueError(f"the conversation would exceed the context limit {self.max_context}")
        results: List[Optional[Generated]] = [None]
        self._run_batch([request], [0], results, on_token, kept={0: (slot, held)})
        return results[0]

    def _run_batch(self, requests, batch, results, on_token, kept=None):
        """``kept``: {request index: (slot, positions it holds)} for sequences whose slot is the
        caller's: it is neither opened nor closed here."""
        kept = kept or {}
        sampler = self.make_sampler([requests[i].sampling for i in batch])
        slots = {}
        try:
            for i in batch:
                slots[i] = kept[i][0] if i in kept else self.open_slot()
            out = {i: [] for i in batch}
            forwards = {i: 0 for i in batch}
            # positions in the cache
            held = {i: (kept[i][1] if i in kept else 0) + len(requests[i].prompt) for i in batch}
            live = [i for i in batch]
            fin = (requests, out, forwards, results, slots, live, kept)
            # requests that may generate nothing still get a result
            for i in list(live):
                if requests[i].max_tokens <= 0 and i not in kept:
                    self._finish(i, LENGTH, *fin)
            t_mark, first = time.perf_counter(), True
            if live:
                logits = self.step([(slots[i], list(requests[i].prompt)) for i in live])
                self.prefill_steps += 1
            for i in list(live):
                if requests[i].max_tokens <= 0:     # a kept sequence: its tokens are run, nothing is drawn
                    self._finish(i, LENGTH, *fin)
            while live:
                rows = [batch.index(i) for i in live]
                ahead = None
                # (not for a sequence whose slot lives on: its last token must stay unrun, to be fed
                # first by the turn after)
                if self.step_ahead is not None and not kept and self._may_run_ahead(live, requests, out, held):
                    # The next step is launched from the tokens as the sampler left them, before
                    # anyone has read them: rows are independent, so a sequence that turns out to
                    # have ended only wastes its row, and the others' logits are there already
                    # when the host has judged this step's tokens.
                    drawn = sampler.draw(logits, rows)
                    ahead = self.step_ahead([slots[i] for i in live], drawn)
                    toks = sampler.read(drawn)
                else:
                    toks = sampler.sample(logits, rows)
                before = list(live)
                now = time.perf_counter()
                if first:
                    self.prefill_secs += now - t_mark
                else:
                    self.decode_secs += now - t_mark
                    self.decode_tokens += len(toks)
                t_mark, first = now, False
                nxt = []
                for i, tok in zip(list(live), toks):
                    r = requests[i]
                    out[i].append(int(tok))
                    if int(tok) in r.stop_ids:
                        self._finish(i, STOP, *fin)
                    elif on_token is not None and on_token(i, out[i]) is False:
                        self._finish(i, CANCELLED, *fin)
                    elif len(out[i]) >= r.max_tokens:
                        self._finish(i, LENGTH, *fin)
                    elif self.max_context and held[i] + 1 > self.max_context:
                        self._finish(i, LENGTH, *fin)
                    else:
                        nxt.append((i, int(tok)))
                if not nxt:
                    break
                if ahead is not None:
                    going = {i for i, _ in nxt}
                    keep = [k for k, i in enumerate(before) if i in going]
                    logits = ahead if len(keep) == len(before) else ahead[keep]
                    self.ahead_steps += 1
                else:
                    logits = self.step([(slots[i], [tok]) for i, tok in nxt])
                self.decode_steps += 1
                for i, _ in nxt:
                    forwards[i] += 1
                    held[i] += 1
        finally:
            for i, s in list(slots.items()):
                if i not in kept:
                    self.close_slot(s)
                del slots[i]

    def _may_run_ahead(self, live, requests, out, held) -> bool:
        """Whether the next step may be launched before this step's tokens are known: some
        sequence must be able to go on after this token, and every sequence must still fit its
        context with one more position (a sequence at its limit ends with this token; its row of
        the step ahead would have nowhere to write)."""
        if self.max_context and any(held[i] + 1 > self.max_context for i in live):
            return False
        return any(len(out[i]) + 1 < requests[i].max_tokens for i in live)

    def _finish(self, i, reason, requests, out, forwards, results, slots, live, kept):
        unfed = out[i][-1] if out[i] and reason != STOP else None
        results[i] = Generated(out[i], reason, len(requests[i].prompt), forwards[i], unfed)
        live.remove(i)
        slot = slots.pop(i)
        if i not in kept:
            self.close_slot(slot)
