"""The cache on the device: paged keys and values per layer group, and beside them the
fixed-size per-sequence state (lengths, last tokens, any state a mixer keeps).

Layout of one layer group (all run steps whose mixers asked for the same ``KVNeed``):

    K, V        [entries, pages, kv_heads, page_size, head_dim]   engine dtype, zero-initialised
    page_table  [max_slots, max_pages_per_slot] int32             physical page of each logical page

so the ``page_size`` keys of one (page, kv head) are one contiguous ``[page_size, head_dim]`` tile,
which is what both attention kernels stream.  The reference keeps one dense
``[layers, b_cap, kv_heads, l_cap, head_dim]`` tensor per K and V, zero-initialised so that a masked
entry can never hold NaN (``engine/dryft_qwen3/cache.py:43-47``), and per-row ``seq_lens`` / ``ids``
(``cache.py:48-50``); a sequence's row index is its batch index.  Here a sequence takes any free
slot, holds only the pages its tokens need, and gives both back when it ends.

``seq_len[slot]`` is both "number of cached tokens" and "position of the next token"
(``cache.py:8-10``).  The device copy is what the kernels read (so one captured decode graph serves
every position); the host copy is what reservations are decided from.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .slots import CacheError, FreeList, PageLedger, pages_for


@dataclass(frozen=True)
class KVNeed:
    """What an attention-like mixer asks of the cache: keys and values of this shape, all of
    them (``window=None``) or the last ``window``."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence, zeroed when a sequence starts.  A mixer that keeps several kinds of
    state (a short convolution's tail and a recurrent state, say) asks with a mapping ``{name: StateNeed}``
    and is handed ``{name: tensor}``."""

    shape: Tuple[int, ...]
    dtype: torch.dtype


@dataclass
class CacheEntry:
    """What one run step's mixer gets: its K and V pages and its group's page table."""

    k: torch.Tensor  # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor  # [max_slots, max_pages_per_slot] int32
    page_size: int
    window: Optional[int]


class _KVGroup:
    def __init__(self, need: KVNeed, run_steps: List[int], n_pages: int, page_size: int, max_slots: int,
                 max_pages_per_slot: int, dtype: torch.dtype, device: torch.device):
        self.need = need
        self.run_steps = run_steps
        self.ledger = PageLedger(n_pages, page_size, max_pages_per_slot, need.window)
        shape = (len(run_steps), n_pages, need.kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.page_table_host = torch.zeros((max_slots, max_pages_per_slot), dtype=torch.int32)
        self.page_table = torch.zeros((max_slots, max_pages_per_slot), dtype=torch.int32, device=device)
        self.dirty: set = set()
        # pinned copy of the rows on their way to the device (one asynchronous copy per flush), and the
        # event after which it may be rewritten
        self.staging: Optional[torch.Tensor] = None
        self.staged: Optional[torch.cuda.Event] = None

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class SequenceCache:
    """Slots, pages and per-sequence state for one model on one device.

    ``needs[i]`` is what run step ``i`` asked for: ``(KVNeed | None, StateNeed | None)``; a run
    step that borrows another's cache is given ``borrow[i] = j`` and owns nothing.
    """

    def __init__(
        self,
        needs: Sequence[Tuple[Optional[KVNeed], Optional[StateNeed]]],
        borrow: Sequence[Optional[int]],
        *,
        max_tokens: int,
        max_slots: int,
        max_seq_len: int,
        page_size: int,
        dtype: torch.dtype,
        device: torch.device,
    ):
        if page_size <= 0 or page_size % 16:
            raise CacheError(f"page_size must be a positive multiple of 16, got {page_size}")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_seq_len = max_seq_len
        self.max_tokens = max_tokens
        self.dtype = dtype
        self.device = device
        n_pages = pages_for(max_tokens, page_size)
        max_pages_per_slot = min(pages_for(max_seq_len, page_size), n_pages)
        self.slots = FreeList(max_slots, "slot")
        self.len_host: List[int] = [0] * max_slots
        # per-sequence state of fixed size, indexed by slot
        self.seq_len = torch.zeros(max_slots, dtype=torch.int32, device=device)
        self.last_token = torch.zeros(max_slots, dtype=torch.int32, device=device)

        self._groups: List[_KVGroup] = []
        self._entry_of: Dict[int, Tuple[int, int]] = {}  # run step -> (group index, index in group)
        self._states: Dict[int, torch.Tensor] = {}
        by_need: Dict[KVNeed, List[int]] = {}
        for i, (kv, st) in enumerate(needs):
            if borrow[i] is not None:
                continue
            if kv is not None:
                by_need.setdefault(kv, []).append(i)
            if st is not None:
                make = lambda need: torch.zeros((max_slots, *need.shape), dtype=need.dtype, device=device)
                if isinstance(st, StateNeed):
                    self._states[i] = make(st)
                elif isinstance(st, Mapping) and st and all(isinstance(v, StateNeed) for v in st.values()):
                    self._states[i] = {name: make(need) for name, need in st.items()}
                else:
                    raise CacheError(f"run step {i}: state_need() must give a StateNeed or a mapping of names to StateNeed, "
                                     f"got {st!r}")
        for need, steps in by_need.items():
            g = _KVGroup(need, steps, n_pages, page_size, max_slots, max_pages_per_slot, dtype, device)
            for j, s in enumerate(steps):
                self._entry_of[s] = (len(self._groups), j)
            self._groups.append(g)
        for i, src in enumerate(borrow):
            if src is not None:
                if src in self._entry_of:
                    self._entry_of[i] = self._entry_of[src]
                if src in self._states:
                    self._states[i] = self._states[src]

    # ------------------------------------------------------------------ views for the parts
    def entry(self, run_step: int) -> Optional[CacheEntry]:
        loc = self._entry_of.get(run_step)
        if loc is None:
            return None
        g = self._groups[loc[0]]
        return CacheEntry(g.k[loc[1]], g.v[loc[1]], g.page_table, self.page_size, g.need.window)

    def state(self, run_step: int):
        """The run step's state ``[slots, *shape]`` (a mapping of such tensors if it asked with a mapping), or None."""
        return self._states.get(run_step)

    def _state_tensors(self) -> List[torch.Tensor]:
        seen: Dict[int, torch.Tensor] = {}
        for st in self._states.values():
            for t in (st.values() if isinstance(st, dict) else (st,)):
                seen[id(t)] = t
        return list(seen.values())

    def n_groups(self) -> int:
        return len(self._groups)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self._groups)

    def free_tokens(self) -> int:
        """Tokens the scarcest group could still take."""
        if not self._groups:
            return self.max_tokens
        return min(g.ledger.pool.n_free for g in self._groups) * self.page_size

    # ------------------------------------------------------------------ sequences
    def open_sequences(self, n: int) -> List[int]:
        """Take ``n`` slots; their lengths and states start at zero."""
        slots = self.slots.take(n)
        for s in slots:
            self.len_host[s] = 0
            for g in self._groups:
                g.ledger.open(s)
        if slots:
            idx = torch.tensor(slots, dtype=torch.int64).to(self.device, non_blocking=True)
            self.seq_len.index_fill_(0, idx, 0)
            self.last_token.index_fill_(0, idx, 0)
            for st in self._state_tensors():
                st.index_fill_(0, idx, 0)
        return slots

    def close_sequences(self, slots: Sequence[int]) -> None:
        """Give slots and their pages back.  What the pages hold stays; it is never read again
        because every read is bounded by the new holder's own length."""
        slots = list(slots)
        for s in slots:
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} freed twice (or never taken)")
        for s in slots:
            for g in self._groups:
                g.ledger.close(s)
            self.len_host[s] = 0
        self.slots.give_back(slots)

    def can_hold(self, lengths: Sequence[int]) -> bool:
        """Whether sequences of these final lengths fit at once beside what is held now."""
        if len(lengths) > self.slots.n_free:
            return False
        if any(n > self.max_seq_len for n in lengths):
            return False
        need = sum(pages_for(n, self.page_size) for n in lengths)
        return all(need <= g.ledger.pool.n_free for g in self._groups)

    def reserve(self, slot: int, n_new: int) -> None:
        """Make room for ``n_new`` more tokens of ``slot`` in every group (host side; the page
        tables reach the device at the next ``flush``)."""
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")
        cur = self.len_host[slot]
        new = cur + n_new
        if new > self.max_seq_len:
            raise CacheError(f"sequence would reach {new} tokens; the cache was built for at most {self.max_seq_len}")
        # all-or-nothing over the groups: check before taking
        for g in self._groups:
            held = g.ledger.held(slot)
            want = [lp for lp in range(pages_for(cur, self.page_size), pages_for(new, self.page_size)) if lp not in held]
            if len(want) > g.ledger.pool.n_free:
                raise CacheError(
                    f"cache full: {len(want)} more page(s) of {self.page_size} tokens wanted, "
                    f"{g.ledger.pool.n_free} free (built for {self.max_tokens} tokens)"
                )
        for g in self._groups:
            added = g.ledger.grow(slot, cur, new)
            if added:
                row = g.page_table_host[slot]
                for lp, pp in added.items():
                    row[lp] = pp
                g.dirty.add(slot)

    def flush(self) -> None:
        """Copy page-table rows that changed to the device (stream-ordered, before the step): the span
        of rows from the first to the last changed one, through a pinned snapshot, as one asynchronous
        copy per group.  Rows in between that did not change are rewritten with the values they have."""
        for g in self._groups:
            if not g.dirty:
                continue
            lo, hi = min(g.dirty), max(g.dirty) + 1
            g.dirty.clear()
            if self.device.type != "cuda":
                g.page_table[lo:hi].copy_(g.page_table_host[lo:hi])
                continue
            if g.staging is None:
                g.staging = torch.empty_like(g.page_table_host).pin_memory()
            if g.staged is not None:
                g.staged.synchronize()   # the copy before this one has read the snapshot
            g.staging[lo:hi].copy_(g.page_table_host[lo:hi])
            g.page_table[lo:hi].copy_(g.staging[lo:hi], non_blocking=True)
            g.staged = torch.cuda.Event()
            g.staged.record()

    def advanced(self, slot: int, n: int) -> None:
        """Record on the host that ``slot`` grew by ``n`` tokens (the device copy is advanced by
        the step itself) and let windowed groups drop pages that fell out of sight."""
        self.len_host[slot] += n
        for g in self._groups:
            if g.need.window is not None:
                g.ledger.trim(slot, self.len_host[slot])

    def check(self) -> None:
        self.slots.check()
        for g in self._groups:
            g.ledger.check()
