"""What a part is, what it sees of a step, and the registry parts are chosen from.

A *part* is one piece of a layer: a norm, a position encoding, a mixer (attention here), a
feed-forward, or the arrangement of those in a block; the embedding and the output head are
parts too.  A part is built from a ``PartSpec`` alone (its sizes and constants) and the compute
precision; it never learns which model it is in.  The plan's ``kind`` strings are looked up in
the registry below, so a new kind of part is added by registering a class, from anywhere.

Interfaces (all tensors on the device; ``ctx`` is the ``StepContext`` of the running step):

* every part: ``wants()`` -> {short name: ``TensorWant``}; ``load(tensors)`` with
  {short name: tensor}, matrices in the compute precision and vectors in float32;
  ``kernel_units()`` -> the CUDA units it launches, for building ahead.
* norm: ``forward(ctx, x, rows_index=None)`` -> normed activations of the float32 rows ``x``.
* position encoding: ``apply(ctx, q, k)`` rotates/encodes ``[T, heads, head_dim]`` views in place.
* mixer: ``cache_need()`` -> ``KVNeed`` | ``StateNeed`` | None;
  ``forward(ctx, h, residual, cache, writes_cache)`` adds its output into the float32 ``residual``.
* feed-forward: ``forward(ctx, h, residual)`` adds its output into ``residual``.
* block: ``forward(ctx, x, cache, writes_cache)`` runs its mixer and feed-forward on ``x`` in place.
* embedding: ``forward(ctx, tokens, out)``; head: ``forward(ctx, h)`` -> float32 logits.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .plan import PartSpec


@dataclasses.dataclass(frozen=True)
class TensorWant:
    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix": held in the compute precision; "vector": held in float32
    optional: bool = False


@dataclasses.dataclass
class StepContext:
    """The batch of one step as the parts see it.  Tokens of all sequences are packed in order;
    index tensors are int32 on the device."""
    compute: str                       # "float32" or "bfloat16"
    act_dtype: torch.dtype
    device: torch.device
    n_tokens: int
    n_seqs: int
    tok_pos: torch.Tensor              # [T] absolute position of each token
    tok_seq: torch.Tensor              # [T] index of its sequence in this batch
    seq_slot: torch.Tensor             # [B] slot of each sequence
    seq_start: torch.Tensor            # [B] length of the sequence before this step
    seq_len: torch.Tensor              # [B] tokens the sequence brings in this step
    cu_seqlens: torch.Tensor           # [B + 1] offsets of the sequences in the packed tokens
    is_decode: bool                    # every sequence brings exactly one token
    max_new: int                       # most tokens one sequence brings
    max_total: int                     # longest sequence after this step (host upper bound)
    cache: object                      # the SequenceCache
    page_size: int
    extras: dict = dataclasses.field(default_factory=dict)
    pad_slot: Optional[int] = None     # slot of rows that belong to no sequence (a padded captured step)

    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.act_dtype, device=self.device)


class Part:
    category = "part"

    def __init__(self, spec: PartSpec, compute: str):
        self.spec, self.compute = spec, compute
        self.act_dtype = torch.float32 if compute == "float32" else torch.bfloat16

    def wants(self) -> Dict[str, TensorWant]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def kernel_units(self) -> List[Tuple[str, tuple]]:
        return []

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part."""
        return 0


_REGISTRY: Dict[Tuple[str, str], Callable] = {}
CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")


def register_part(category: str, kind: str, factory: Callable) -> None:
    """Makes ``kind`` available to plans as a part of ``category``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r} (known: {', '.join(CATEGORIES)})")
    _REGISTRY[(category, kind)] = factory


def build_part(category: str, spec: PartSpec, compute: str):
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ValueError(f"unknown {category} kind {spec.kind!r} (known: {', '.join(known)})") from None
    return factory(spec, compute)


def build_block(layer_spec, compute: str):
    """The block of a ``LayerSpec``: its ``block`` kind arranges the layer's parts."""
    try:
        factory = _REGISTRY[("block", layer_spec.block)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == "block")
        raise ValueError(f"unknown block kind {layer_spec.block!r} (known: {', '.join(known)})") from None
    return factory(layer_spec, compute)


def compute_dtype(compute: str) -> torch.dtype:
    if compute == "float32":
        return torch.float32
    if compute == "bfloat16":
        return torch.bfloat16
    raise ValueError(f"dtype must be float32 or bfloat16, got {compute!r}")
