"""The generation loop's decisions, with a fake model (no GPU)."""
import pytest

from gemmars_b200.cache import CacheError, SlotAllocator
from gemmars_b200.engine.generate import CANCELLED, LENGTH, STOP, GenerationLoop, Request, plan_batches, tokens_held


class FakeModel:
    """Next token = (sum of the sequence so far) % 50; records every call."""

    def __init__(self, n_slots):
        self.slots = SlotAllocator(n_slots)
        self.seqs, self.calls, self.opened = {}, [], []

    def open(self):
        s = self.slots.take()
        self.seqs[s] = []
        self.opened.append(s)
        return s

    def close(self, s):
        self.slots.give_back(s)
        del self.seqs[s]

    def step(self, items):
        self.calls.append([(s, list(t)) for s, t in items])
        rows = []
        for s, toks in items:
            self.seqs[s].extend(toks)
            rows.append(sum(self.seqs[s]) % 50)
        return rows

    class Sampler:
        def __init__(self, params):
            self.params = params

        def sample(self, logits, seqs):
            assert len(logits) == len(seqs)
            return list(logits)

    def loop(self, max_batch=4, pages=100, max_context=None):
        return GenerationLoop(self.open, self.close, self.step, self.Sampler, max_batch, pages, 64, max_context)


def _expected(prompt, n, stop=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = sum(seq) % 50
        out.append(t)
        if t in stop:
            return out, STOP
        seq.append(t)
    return out, LENGTH


def test_unequal_prompts_end_at_different_times_and_free_their_slots():
    m = FakeModel(4)
    reqs = [Request([1, 2, 3], 6), Request([9], 2), Request([4, 4, 4, 4, 4], 4), Request([7, 1], 1)]
    res = m.loop().run(reqs)
    for r, q in zip(res, reqs):
        assert (r.tokens, r.reason) == _expected(q.prompt, q.max_tokens) and r.prompt_tokens == len(q.prompt)
    # one step for all prompts, then one token per live sequence; sequences leave the batch when they end
    assert [len(c) for c in m.calls] == [4, 3, 2, 2, 1, 1]
    assert all(len(t) == 1 for c in m.calls[1:] for _, t in c)
    assert m.slots.free_count == 4 and not m.seqs
    assert [r.forwards for r in res] == [5, 1, 3, 0]      # the last generated token is never run


def test_stop_token_is_kept_and_not_run():
    m = FakeModel(2)
    prompt = [10, 5]                       # 15 -> 30 -> 10 -> ...
    res = m.loop().run([Request(prompt, 10, stop_ids=(10,))])
    assert res[0].tokens == [15, 30, 10] and res[0].reason == STOP
    assert m.calls[-1] == [(0, [30])]      # the stop token 10 never ran


def test_batches_follow_one_another_and_reuse_slots():
    m = FakeModel(2)
    reqs = [Request([i + 1], 3) for i in range(5)]
    res = m.loop(max_batch=2).run(reqs)
    assert [r.tokens for r in res] == [_expected(q.prompt, 3)[0] for q in reqs]
    assert m.opened == [0, 1, 0, 1, 0]
    assert plan_batches(reqs, 2, 100, 64) == [[0, 1], [2, 3], [4]]


def test_batches_respect_the_cache():
    reqs = [Request([1] * 100, 30), Request([1] * 10, 10), Request([1] * 200, 57), Request([1], 1)]
    assert tokens_held(100, 30, None) == 129 and tokens_held(100, 30, 110) == 110
    assert plan_batches(reqs, 8, 6, 64) == [[0, 1], [2, 3]]          # 3 + 1 pages, then 4 + 1
    with pytest.raises(ValueError, match="cache pages"):
        plan_batches(reqs, 8, 3, 64)
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([Request([], 3)], 8, 6, 64)
    with pytest.raises(ValueError, match="context limit"):
        plan_batches(reqs, 8, 60, 64, max_context=150)


def test_cancel_and_context_limit_and_zero_tokens():
    m = FakeModel(3)
    seen = []

    def on_token(i, toks):
        seen.append((i, list(toks)))
        return not (i == 0 and len(toks) == 2)

    reqs = [Request([1, 2], 5), Request([3], 5), Request([4], 0)]
    res = m.loop(max_context=3).run(reqs, on_token)
    assert res[0].reason == CANCELLED and len(res[0].tokens) == 2
    # request 1: prompt of 1, context 3 -> runs tokens until 3 positions are held, then "length"
    assert res[1].reason == LENGTH and len(res[1].tokens) == 3 and res[1].forwards == 2
    assert res[2].tokens == [] and res[2].reason == LENGTH
    assert (0, res[0].tokens) in seen and m.slots.free_count == 3


def test_slots_are_given_back_when_a_step_fails():
    m = FakeModel(2)

    def bad_step(items):
        raise CacheError("boom")

    loop = GenerationLoop(m.open, m.close, bad_step, m.Sampler, 2, 100, 64)
    with pytest.raises(CacheError):
        loop.run([Request([1], 2), Request([2], 2)])
    assert m.slots.free_count == 2


def test_a_turn_in_a_kept_slot_uses_the_same_decisions_and_leaves_the_slot_open():
    """The conversation of ``send``: the loop runs one request in a slot the caller keeps, returns
    the token that was generated but not run, and the next turn feeds it first."""
    m = FakeModel(2)
    slot = m.open()
    loop = m.loop(max_context=40)
    first = loop.run_in_slot(slot, 0, Request([3, 4], 3))
    want, _ = _expected([3, 4], 3)
    assert first.tokens == want and first.reason == LENGTH and first.unfed == want[-1]
    assert slot in m.seqs and m.seqs[slot] == [3, 4] + want[:-1]          # the last token was not run
    # next turn: the unfed token first, then the new ones; a stop token ends it and is not run
    held = len(m.seqs[slot])
    feed = [first.unfed, 11]
    seq = list(m.seqs[slot]) + feed
    stop_at = sum(seq) % 50
    second = loop.run_in_slot(slot, held, Request(feed, 5, stop_ids=(stop_at,)))
    assert second.tokens == [stop_at] and second.reason == STOP and second.unfed is None
    assert m.seqs[slot] == seq and m.slots.free_count == 1
    # cancelled: the token the callback saw last is unfed
    third = loop.run_in_slot(slot, len(seq), Request([1], 9), on_token=lambda i, toks: len(toks) < 2)
    assert third.reason == CANCELLED and len(third.tokens) == 2 and third.unfed == third.tokens[-1]
    assert len(m.seqs[slot]) == len(seq) + 1 + 1
    # the context limit counts what the slot holds already
    with pytest.raises(ValueError, match="context limit"):
        loop.run_in_slot(slot, 39, Request([1, 2], 4))
    m.close(slot)
    assert m.slots.free_count == 2


def test_steps_launched_ahead_change_no_decision():
    """With ``step_ahead`` the next step runs from the drawn tokens before they are read.  The
    tokens, reasons and what each sequence holds must be what the plain loop gives: a sequence
    that ends only wastes its row of the step that was already on its way, and the rows of those
    that go on are picked out of it."""
    import numpy as np

    class AheadModel(FakeModel):
        def __init__(self, n):
            super().__init__(n)
            self.ahead_calls = 0

        def step(self, items):
            return np.asarray(super().step(items))

        def step_ahead(self, slots, drawn):
            self.ahead_calls += 1
            return self.step([(s, [int(t)]) for s, t in zip(slots, drawn)])

        class Sampler(FakeModel.Sampler):
            def draw(self, logits, seqs):
                return list(logits)

            def read(self, drawn):
                return [int(t) for t in drawn]

    reqs = [Request([1, 2, 3], 6), Request([9], 2), Request([4, 4, 4, 4, 4], 4, stop_ids=(_expected([4] * 5, 4)[0][1],)),
            Request([7, 1], 1), Request([5, 5], 7)]
    plain_model = FakeModel(5)
    want = plain_model.loop(max_batch=5).run(reqs)
    m = AheadModel(5)
    loop = GenerationLoop(m.open, m.close, m.step, m.Sampler, 5, 100, 64, None, step_ahead=m.step_ahead)
    got = loop.run(reqs)
    assert [(r.tokens, r.reason, r.forwards) for r in got] == [(r.tokens, r.reason, r.forwards) for r in want]
    assert m.ahead_calls > 0 and loop.ahead_steps > 0 and m.slots.free_count == 5
    # the last step of a batch is never launched ahead when no sequence can go on after it
    assert loop.decode_steps == plain_model_steps(reqs, want)
    # a turn in a kept slot never runs ahead: its last token must stay unrun
    slot = m.open()
    before = m.ahead_calls
    turn = loop.run_in_slot(slot, 0, Request([3, 4], 3))
    assert m.ahead_calls == before and m.seqs[slot] == [3, 4] + turn.tokens[:-1]


def plain_model_steps(reqs, results):
    """Decode steps a batch needs when none is wasted: as many as its longest-running sequence."""
    return max(r.forwards for r in results)


def test_random_request_sets_give_each_request_its_own_answer():
    """Whatever the prompts, limits, stop tokens, batch size and cache size: every request gets the
    tokens it would get alone, in request order; every slot is given back; with and without steps
    launched ahead."""
    import numpy as np
    from hypothesis import given, settings, strategies as st

    class AheadModel(FakeModel):
        def step(self, items):
            return np.asarray(super().step(items))

        def step_ahead(self, slots, drawn):
            return self.step([(s, [int(t)]) for s, t in zip(slots, drawn)])

        class Sampler(FakeModel.Sampler):
            def draw(self, logits, seqs):
                return list(logits)

            def read(self, drawn):
                return [int(t) for t in drawn]

    request = st.tuples(st.lists(st.integers(0, 49), min_size=1, max_size=12), st.integers(0, 9),
                        st.lists(st.integers(0, 49), max_size=3))

    @settings(max_examples=120, deadline=None)
    @given(st.lists(request, min_size=1, max_size=9), st.integers(1, 4), st.booleans())
    def run(specs, max_batch, ahead):
        reqs = [Request(p, n, stop_ids=tuple(stop)) for p, n, stop in specs]
        m = AheadModel(max_batch)
        loop = GenerationLoop(m.open, m.close, m.step, m.Sampler, max_batch, 50, 64, None,
                              step_ahead=m.step_ahead if ahead else None)
        got = loop.run(reqs)
        assert m.slots.free_count == max_batch and not m.seqs
        for r, (p, n, stop) in zip(got, specs):
            want, reason = _expected(p, n, stop)
            assert (r.tokens, r.reason, r.prompt_tokens) == (want, reason if n > 0 else LENGTH, len(p))
            assert r.unfed == (want[-1] if want and r.reason != STOP else None)

    run()
