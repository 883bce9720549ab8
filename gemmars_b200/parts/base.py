"""What a part is, what it sees of a step, and the registry parts are chosen from.

A *part* is one piece of a layer: a norm, a position encoding, a mixer (attention here), a
feed-forward, or the arrangement of those in a block; the embedding and the output head are
parts too.  A part is built from a ``PartSpec`` alone (its sizes and constants) and the compute
precision; it never learns which model it is in.  The plan's ``kind`` strings are looked up in
the registry below, so a new kind of part is added by registering a class, from anywhere.

Interfaces (all tensors on the device; ``ctx`` is the ``StepContext`` of the running step):

* every part: ``wants()`` -> {short name: ``TensorWant``}; ``load(tensors)`` with
  {short name: tensor}, matrices in the compute precision and vectors in float32;
  ``kernel_units()`` -> the CUDA units it launches, for building ahead; ``weight_bytes()`` ->
  the bytes of weights one decode step reads from it; ``cache_needs()`` -> a list of
  ``KVNeed`` | ``StateNeed`` (empty for most parts): what it keeps per sequence between steps.
  A part may ask for several (two states of different shapes, or keys and a state).
* norm: ``forward(ctx, x, rows_index=None)`` -> normed activations of the float32 rows ``x``.
* position encoding: ``apply(ctx, q, k)`` rotates/encodes ``[T, heads, head_dim]`` views in place.
* mixer: ``forward(ctx, h, residual, caches, writes_cache)`` adds its output into the float32
  ``residual``.  ``caches`` lists one view per entry of ``cache_needs()``, in that order:
  ``(KVGroup, k, v)`` for a ``KVNeed``, the state tensor ``[slots + 1, *shape]`` for a
  ``StateNeed``.  A mixer that keeps nothing itself but runs on another entry's cache
  (``ScheduleEntry.cache_of``) gets that entry's views, with ``writes_cache`` False.
* feed-forward: ``forward(ctx, h, residual)`` adds its output into ``residual``.
* block: built from a ``LayerSpec`` (it reads ``layer_spec.parts`` by the names of its own
  kind); ``parts()`` -> {name: part}, every part it built; ``forward(ctx, x, caches,
  writes_cache)`` runs them on ``x`` in place, ``caches`` being the views of all its parts'
  needs in the order of ``parts()`` (``Block.split_caches`` deals them out).
* embedding: ``forward(ctx, tokens, out)``; head: ``forward(ctx, h)`` -> float32 logits.

Optional, for decode steps: a norm taken into the products around it.  A mixer or feed-forward
whose class says ``links_norms = True`` takes one more argument, ``then_norm`` (the norm part that
reads the residual after it, or None), may be given ``kernels.UnscaledRows`` instead of a tensor
for ``h``, and returns what its last product left for ``then_norm`` (``UnscaledRows``) or None.  A
norm that says ``linkable = True`` can be taken in this way; a block that says ``chains_norms =
True`` takes ``h_in`` and ``next_norm`` and has ``first_norm()``.  Parts and blocks that say
nothing are given plain tensors and called as listed above.

Rows that belong to no sequence.  A decode step that is replayed from a captured graph is padded
to a fixed number of rows.  The padding rows are sequences of one token whose slot is
``ctx.pad_slot``: the spare last row of every page table (all page 0) and of every state tensor.
Several rows of a step may carry that slot.  A part may compute anything for them (their outputs
are dropped) as long as whatever it writes for them lands in that spare row or in page 0, which
no sequence ever reads; it must not let them touch another row's keys, values or state, and it
cannot ask the host about them (a captured step runs without the host).  In steps that are not
captured there are no such rows and ``ctx.pad_slot`` is None; those steps also carry the batch's
shape on the host (``ctx.host``), so a part that has to walk each sequence's tokens in order can
do so without reading device memory back.
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
    #: what parts keep for the length of one run of the model over this context; emptied when a run starts
    extras: dict = dataclasses.field(default_factory=dict)
    pad_slot: Optional[int] = None     # slot of rows that belong to no sequence (a padded captured step)
    #: the batch's shape on the host, for steps that are not captured (None in a captured step):
    #: {"seq_slot": [...], "seq_start": [...], "seq_len": [...]}, one entry per sequence
    host: Optional[dict] = None

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
        """Bytes of weights one decode step reads from this part (a table of which a step gathers
        a few rows counts as nothing)."""
        return 0

    def cache_needs(self) -> list:
        """What this part keeps per sequence between steps: a list of KVNeed | StateNeed."""
        return []

    #: True when what the part launches in a decode step depends on ``ctx.max_total``: captured
    #: decode steps are then kept per length bucket instead of one per batch size
    capture_depends_on_length = False


class Block(Part):
    """Base of the block kinds: builds nothing itself, deals the caches out to its parts."""
    category = "block"

    def __init__(self, layer_spec, compute: str):
        self.spec, self.compute = layer_spec, compute
        self.act_dtype = torch.float32 if compute == "float32" else torch.bfloat16

    def need(self, name: str, category: str):
        """Builds the part the layer's spec lists under ``name``."""
        try:
            spec = self.spec.parts[name]
        except KeyError:
            raise ValueError(f"block {self.spec.block!r} needs a part named {name!r}; the layer lists "
                             f"{', '.join(sorted(self.spec.parts)) or 'none'}") from None
        return build_part(category, spec, self.compute)

    def parts(self) -> Dict[str, "Part"]:
        raise NotImplementedError

    def cache_needs(self) -> list:
        return [n for part in self.parts().values() for n in part.cache_needs()]

    def split_caches(self, caches) -> Dict[str, list]:
        """{part name: its share of ``caches``} for views listed in the order of cache_needs().
        A block none of whose parts keeps anything passes foreign views (``cache_of``) to the
        part named ``mixer``."""
        out, at = {}, 0
        caches = list(caches or [])
        for name, part in self.parts().items():
            n = len(part.cache_needs())
            out[name] = caches[at:at + n]
            at += n
        if at == 0 and caches and "mixer" in out:
            out["mixer"] = caches
        return out


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
