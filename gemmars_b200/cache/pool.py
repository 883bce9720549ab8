"""Slots, pages and per-sequence state: the memory one batch of sequences lives in.

* A **slot** belongs to one sequence from its first token to its end.  ``SlotAllocator`` hands
  slots out and takes them back; a slot that is given back is used again by a later sequence.
* Keys and values are kept in **pages** of ``page_size`` positions.  Layers with the same needs
  form a **group** (``KVGroup``) with storage and a page table of its own: a group that keeps
  all keys maps every page of a sequence; a group that keeps a window maps a ring of pages and
  writes over the oldest.
* Parts with a fixed-size state per sequence (a recurrent mixer) get a ``StateGroup``: one
  tensor per layer with a row per slot, cleared when the slot is taken.

Everything here is host bookkeeping over ``torch`` tensors; it runs on the CPU as well, which is
how its tests run.

Reference: the reference keeps one growing ``LayerCache`` per layer and one session per engine
(src/model.rs:693-735, src/qwen.rs:287-294, 605-630), with a fixed-size recurrent state beside
it for other mixers (src/qwen.rs:170-175, 616-619); slots and pages have no counterpart there.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import torch

PAGE_SIZE = 64


class CacheError(RuntimeError):
    pass


class SlotAllocator:
    """Slots 0..n-1; lowest free slot first."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(range(n - 1, -1, -1))
        self._held = set()

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free slot: all {self.n} are held")
        s = self._free.pop()
        self._held.add(s)
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held (freed twice, or never taken)")
        self._held.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    @property
    def held(self) -> set:
        return set(self._held)

    @property
    def free_count(self) -> int:
        return len(self._free)


class PageAllocator:
    """Pages 1..n (page 0 is never handed out: padded rows of a batch write there)."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(range(n, 0, -1))
        self._held = set()

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"the cache is full: all {self.n} pages are held")
        p = self._free.pop()
        self._held.add(p)
        return p

    def give_back(self, page: int) -> None:
        if page not in self._held:
            raise CacheError(f"page {page} is not held (freed twice, or never taken)")
        self._held.remove(page)
        self._free.append(page)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)


@dataclasses.dataclass(frozen=True)
class KVNeed:
    """What a caching part asks of the cache: heads and width of its keys and values, and the
    window it reads (None: all keys)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per sequence: shape and dtype of one sequence's state."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class KVGroup:
    """Storage of the layers that share one ``KVNeed``.

    ``k``: ``[layers, pages + 1, kv_heads, page_size, head_dim]``; ``v`` is kept transposed inside
    a page, ``[layers, pages + 1, kv_heads, head_dim, page_size]``, so that attention's second
    product also contracts over the contiguous axis.
    ``page_table``: ``[slots + 1, table_width]`` int32; position ``p`` of the sequence in slot ``s``
    lives in page ``page_table[s, (p // page_size) % table_width]`` at offset ``p % page_size``.
    For a group that keeps all keys the table is as wide as the longest sequence; for a window it
    is a ring just wide enough for the window plus the tokens of one step.
    """

    def __init__(self, need: KVNeed, n_layers: int, n_slots: int, n_pages: int, max_seq_pages: int,
                 max_step_tokens: int, dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        self.need, self.n_layers, self.page_size = need, n_layers, page_size
        if need.window is None:
            self.table_width = max(1, max_seq_pages)
        else:
            ring = (need.window - 1 + max_step_tokens + page_size - 1) // page_size + 1
            self.table_width = max(1, min(max_seq_pages, ring))
            n_pages = min(n_pages, n_slots * self.table_width)
        self.pages = PageAllocator(n_pages)
        shape = (n_layers, n_pages + 1, need.num_kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape[:3] + (need.head_dim, page_size), dtype=dtype, device=device)
        # row n_slots stays all zero: padded rows of a batch use it and land in page 0
        self.table_host = torch.zeros((n_slots + 1, self.table_width), dtype=torch.int32)
        self.page_table = torch.zeros((n_slots + 1, self.table_width), dtype=torch.int32, device=device)
        self._dirty = set()
        self._mapped: Dict[int, int] = {}   # slot -> logical pages mapped so far

    def reserve(self, slot: int, new_len: int) -> None:
        """Maps the pages that positions ``< new_len`` of ``slot`` need."""
        need_pages = (new_len + self.page_size - 1) // self.page_size
        have = self._mapped.get(slot, 0)
        for lp in range(have, need_pages):
            col = lp % self.table_width
            if lp >= self.table_width:
                continue  # a ring: the page of logical page lp - width is written over
            self.table_host[slot, col] = self.pages.take()
            self._dirty.add(slot)
        self._mapped[slot] = max(have, need_pages)

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = min(self._mapped.get(slot, 0), self.table_width)
        want = min((new_len + self.page_size - 1) // self.page_size, self.table_width)
        return max(0, want - have)

    def release(self, slot: int) -> None:
        for col in range(min(self._mapped.pop(slot, 0), self.table_width)):
            self.pages.give_back(int(self.table_host[slot, col]))
            self.table_host[slot, col] = 0
        self._dirty.add(slot)

    def truncate(self, slot: int, new_len: int) -> None:
        """Forgets positions ``>= new_len``; only for groups that keep all keys."""
        if self.need.window is not None:
            raise CacheError("a windowed group cannot be truncated")
        keep = (new_len + self.page_size - 1) // self.page_size
        for lp in range(keep, self._mapped.get(slot, 0)):
            self.pages.give_back(int(self.table_host[slot, lp]))
            self.table_host[slot, lp] = 0
            self._dirty.add(slot)
        self._mapped[slot] = min(self._mapped.get(slot, 0), keep)

    def sync(self) -> None:
        """Copies the rows of the page table that changed to the device."""
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        # The host table is ordinary (pageable) memory on purpose: a copy from it is staged when it
        # is asked for, so later changes of the host table (the next step's pages, a slot given
        # back) cannot reach a copy that the device has not run yet.
        if len(rows) > 4:
            self.page_table.copy_(self.table_host)
        else:
            for r in rows:
                self.page_table[r].copy_(self.table_host[r])

    def layer(self, i: int):
        """(k, v) storage of the group's ``i``-th layer: k ``[pages + 1, kv_heads, page_size, head_dim]``,
        v ``[pages + 1, kv_heads, head_dim, page_size]``."""
        return self.k[i], self.v[i]


class StateGroup:
    """One fixed-size state per (layer, slot): ``[layers, slots + 1, *shape]``.  Row ``slots`` is
    the padding row."""

    def __init__(self, need: StateNeed, n_layers: int, n_slots: int, device):
        self.need = need
        self.data = torch.zeros((n_layers, n_slots + 1) + tuple(need.shape), dtype=need.dtype, device=device)

    def clear(self, slot: int) -> None:
        self.data[:, slot].zero_()

    def layer(self, i: int) -> torch.Tensor:
        return self.data[i]


@dataclasses.dataclass
class CacheBinding:
    """Where one schedule entry's cache lives: its group and its layer index in that group."""
    kind: str            # "kv" or "state"
    group: int
    index: int


class SequenceCache:
    """All groups of a model, the slots, and each sequence's length.

    ``needs``: for each schedule entry that keeps a cache, ``(entry index, needs)``, ``needs``
    being one ``KVNeed | StateNeed`` or a list of them (a layer may keep keys and a state, or two
    states of different shapes).  Equal needs share a group, whichever entry they come from.
    ``bindings[entry]`` lists, in the order of the entry's needs, where each one lives.
    """

    def __init__(self, needs: Sequence[Tuple[int, object]], max_tokens: int, n_slots: int, max_positions: int,
                 max_step_tokens: int, dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        self.page_size = page_size
        self.device = device
        self.n_pages = max(1, (max_tokens + page_size - 1) // page_size)
        self.n_slots = max(1, min(n_slots, self.n_pages))
        self.max_seq_len = self.n_pages * page_size
        if max_positions:
            self.max_seq_len = min(self.max_seq_len, max_positions)
        max_seq_pages = (self.max_seq_len + page_size - 1) // page_size
        self.slots = SlotAllocator(self.n_slots)
        self.lengths: Dict[int, int] = {}
        kv_keys: List[KVNeed] = []
        st_keys: List[StateNeed] = []
        members: Dict[Tuple[str, int], List[int]] = {}
        self.bindings: Dict[int, List[CacheBinding]] = {}
        for entry, entry_needs in needs:
            if isinstance(entry_needs, (KVNeed, StateNeed)):
                entry_needs = [entry_needs]
            for need in entry_needs:
                if isinstance(need, KVNeed):
                    if need not in kv_keys:
                        kv_keys.append(need)
                    g, kind = kv_keys.index(need), "kv"
                elif isinstance(need, StateNeed):
                    if need not in st_keys:
                        st_keys.append(need)
                    g, kind = st_keys.index(need), "state"
                else:
                    raise TypeError(f"schedule entry {entry}: unknown cache need {need!r}")
                lst = members.setdefault((kind, g), [])
                self.bindings.setdefault(entry, []).append(CacheBinding(kind, g, len(lst)))
                lst.append(entry)
        self.kv_groups = [KVGroup(n, len(members[("kv", i)]), self.n_slots, self.n_pages, max_seq_pages,
                                  max_step_tokens, dtype, device, page_size) for i, n in enumerate(kv_keys)]
        self.state_groups = [StateGroup(n, len(members[("state", i)]), self.n_slots, device)
                             for i, n in enumerate(st_keys)]

    # ---- sequences
    def open(self) -> int:
        """Takes a slot for a new, empty sequence."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.state_groups:
            g.clear(slot)
        return slot

    def close(self, slot: int) -> None:
        """Gives back the slot and every page it holds."""
        self.slots.give_back(slot)
        for g in self.kv_groups:
            g.release(slot)
        del self.lengths[slot]

    def can_extend(self, extensions: Sequence[Tuple[int, int]]) -> bool:
        """Whether every ``(slot, tokens to append)`` fits, taken together."""
        for g in self.kv_groups:
            want = sum(g.pages_needed(s, self.lengths[s] + n) for s, n in extensions)
            if want > g.pages.free_count:
                return False
        return all(self.lengths[s] + n <= self.max_seq_len for s, n in extensions)

    def extend(self, slot: int, n: int) -> int:
        """Reserves room for ``n`` more positions of ``slot``; returns the length before."""
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not open")
        start = self.lengths[slot]
        if start + n > self.max_seq_len:
            raise CacheError(f"sequence of {start + n} tokens exceeds the longest the cache holds ({self.max_seq_len})")
        for g in self.kv_groups:        # all or nothing: no group takes a page unless every group has enough
            if g.pages_needed(slot, start + n) > g.pages.free_count:
                raise CacheError(f"the cache is full: {g.pages.free_count} pages are free, slot {slot} needs "
                                 f"{g.pages_needed(slot, start + n)} more to hold {start + n} tokens")
        for g in self.kv_groups:
            g.reserve(slot, start + n)
        self.lengths[slot] = start + n
        return start

    def truncate(self, slot: int, new_len: int) -> None:
        if new_len < self.lengths[slot]:
            for g in self.kv_groups:
                g.truncate(slot, new_len)
            self.lengths[slot] = new_len

    def sync(self) -> None:
        for g in self.kv_groups:
            g.sync()

    def rollback(self, slot: int, old_len: int) -> bool:
        """After a step that failed: takes back the positions from ``old_len`` on that were
        reserved for it, so that the slot's length again names only positions that were written
        by steps that succeeded.  Returns whether the slot then holds exactly what it held before
        the step: true when every group keeps all keys (their pages beyond ``old_len`` are given
        back); false when a window's ring may have been written over or a state may have
        advanced, which cannot be undone: such a slot can only be closed."""
        if slot not in self.lengths or old_len >= self.lengths[slot]:
            return True
        for g in self.kv_groups:
            if g.need.window is None:
                g.truncate(slot, old_len)
        self.lengths[slot] = old_len
        return not self.state_groups and all(g.need.window is None for g in self.kv_groups)

    def views(self, entry: int) -> list:
        """The storage of every need of ``entry``, in the order of its needs: ``(KVGroup, k, v)``
        for keys and values, the state tensor ``[slots + 1, *shape]`` for a state."""
        out = []
        for b in self.bindings.get(entry, []):
            if b.kind == "kv":
                g = self.kv_groups[b.group]
                out.append((g,) + tuple(g.layer(b.index)))
            else:
                out.append(self.state_groups[b.group].layer(b.index))
        return out

    def kv(self, entry: int, which: int = 0):
        """(group, k, v) of the ``which``-th need of ``entry``, which must be a KVNeed."""
        assert self.bindings[entry][which].kind == "kv"
        return self.views(entry)[which]

    def state(self, entry: int, which: int = 0) -> torch.Tensor:
        assert self.bindings[entry][which].kind == "state"
        return self.views(entry)[which]

    def pages_held(self) -> int:
        return sum(g.pages.held_count for g in self.kv_groups)
