"""Sampling settings, the reference's random generator, and the batched sampler that calls the
device kernel.

Reference: src/sampler.rs.  ``Sampler::new(temperature, top_k, top_p, seed)`` (:11-18; a zero
seed becomes 1); greedy iff temperature <= 0 (:37-39); the generator is xorshift64* whose top 24
bits make a float in [0, 1) (:20-30).  Defaults are the command line's: temperature 0, top-k 64,
top-p 0.95, seed 42 (src/main.rs:182-185, src/engine.rs:341-351).

Each sequence has a generator of its own, so what a sequence draws does not depend on the
batch it is in.  The uniform numbers are drawn on the host; selection, softmax, the top-p cut
and the walk run in the ``sampling`` CUDA unit.
"""
from __future__ import annotations

import dataclasses
from typing import List, Sequence

import torch

from .. import kernels

_MASK = (1 << 64) - 1


class Xorshift64Star:
    def __init__(self, seed: int):
        self.state = max(int(seed) & _MASK, 1)

    def next_f32(self) -> float:
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & _MASK
        x ^= x >> 27
        self.state = x
        r = (x * 0x2545F4914F6CDD1D) & _MASK
        return (r >> 40) / float(1 << 24)   # exact in float32


@dataclasses.dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 64
    top_p: float = 0.95
    seed: int = 42

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def wide(self) -> bool:
        """More candidates than the device sampler keeps in shared memory (top_k = 0: all tokens,
        src/sampler.rs:43-47): such rows are sorted in global memory, which is slower."""
        return not self.greedy and not 1 <= self.top_k <= kernels.MAX_TOP_K

    def check(self) -> None:
        if self.greedy:
            return
        if self.top_k < 0:
            raise ValueError(f"top_k must be 0 (all tokens) or positive, got {self.top_k}")
        if not 0.0 < self.top_p:
            raise ValueError(f"top_p must be positive, got {self.top_p}")


class BatchSampler:
    """One generator per sequence; ``sample`` draws one token for each given sequence."""

    RING = 4     # pinned host buffers used in turn; one is written again only after its copy is done

    def __init__(self, params: Sequence[SamplingParams], device):
        for p in params:
            p.check()
        self.params = list(params)
        self.rngs = [Xorshift64Star(p.seed) for p in params]
        self.device = device
        self.all_greedy = all(p.greedy for p in params)
        self.any_wide = any(p.wide for p in params)
        # the most candidates a row served from shared memory can have: the device kernels do less
        # work for a smaller bound
        self.cap = max([p.top_k for p in params if not p.greedy and not p.wide] + [1])
        self._host, self._events, self._turn = None, [None] * self.RING, 0
        self._copy_stream, self._host_tokens, self._drawn_at = None, None, None

    def sample(self, logits: torch.Tensor, seqs: Sequence[int]) -> List[int]:
        """``logits``: float32 [len(seqs), vocab] on the device; ``seqs``: which sequence each
        row belongs to.  Returns one token id per row."""
        return self.sample_device(logits, seqs).tolist()

    def _stage(self, seqs):
        """The rows' settings and uniform draws, through pinned host memory that is allocated
        once for the whole batch (pinning takes about a millisecond, a decode step a few):
        float32 [3, n] (temperature, top_p, uniform) and int32 [n] (top_k) on the device."""
        n, cap = len(seqs), len(self.params)
        if self._host is None:
            self._host = [(torch.empty(3 * cap, dtype=torch.float32).pin_memory(),
                           torch.empty(cap, dtype=torch.int32).pin_memory()) for _ in range(self.RING)]
        i = self._turn
        self._turn = (i + 1) % self.RING
        if self._events[i] is not None:
            self._events[i].synchronize()
        hf, hk = self._host[i]
        f, k = hf.numpy(), hk.numpy()
        for j, s in enumerate(seqs):                 # three runs of n values: each copy is one contiguous piece
            p = self.params[s]
            f[j], f[n + j] = p.temperature, p.top_p
            f[2 * n + j] = 0.0 if p.greedy else self.rngs[s].next_f32()
            k[j] = p.top_k
        dev_f = hf[:3 * n].to(self.device, non_blocking=True).view(3, n)
        dev_k = hk[:n].to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        return dev_f, dev_k

    def draw(self, logits: torch.Tensor, seqs: Sequence[int]) -> torch.Tensor:
        """As ``sample``, but the tokens stay on the device (int32 [len(seqs)]) until ``read``."""
        drawn = self.sample_device(logits, seqs)
        if drawn.is_cuda:
            self._drawn_at = torch.cuda.Event()
            self._drawn_at.record()
        return drawn

    def read(self, drawn: torch.Tensor) -> List[int]:
        """The tokens of the last ``draw`` on the host.  They are fetched on a stream of their own
        that waits for the sampler alone: on the stream the step runs on, the copy would queue up
        behind whatever was launched since (the next step, when it was launched ahead) and the
        host would learn the tokens a whole step late."""
        if not drawn.is_cuda:
            return drawn.tolist()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=drawn.device)
            self._host_tokens = torch.empty(max(len(self.params), drawn.numel()), dtype=torch.int32).pin_memory()
        n = drawn.numel()
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._drawn_at)
            self._host_tokens[:n].copy_(drawn, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self._copy_stream)
        done.synchronize()
        return self._host_tokens[:n].tolist()

    def sample_device(self, logits: torch.Tensor, seqs: Sequence[int]) -> torch.Tensor:
        n = len(seqs)
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if self.all_greedy:
            kernels.sample(logits, out)
            return out
        f, k = self._stage(seqs)
        kernels.sample(logits, out, f[0], k, f[1], f[2], wide=self.any_wide, cap=self.cap)
        return out
