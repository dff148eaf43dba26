"""The cache: a slot per sequence, paged keys and values per cache unit, fixed-size state.

Layout. A *unit* is the storage of one entry of the model's run order (a layer that runs
twice has two units; a layer that reads another entry's cache has none). Units whose mixers
ask for the same thing (KV heads, head size, window) form a *group* with storage of its own:

    k, v          [units, pages + 1, kv_heads, page_size, head_dim]   keys are stored rotated
    block_table   [slots + 1, max_pages_per_seq] int32                logical page -> page

Pages hold `page_size` (64) consecutive positions of one sequence; a sequence holds only the
pages it has reached, so memory follows the tokens held, not slots x longest length. A group
with a window gives pages back once no later token can read them. Fixed-size per-sequence state
(for mixers that carry a recurrent state) lives beside it as [units, slots + 1, *shape] and is
zeroed when a slot is taken; this architecture asks for none. A unit may hold several requests of
either kind, told apart by name (a layer with two mixers). Slot `n_slots` and page
`n_pages` are scratch: padding lanes of a captured decode step write there.

Each sequence's length lives on the device (`seq_lens`) so that a captured decode step reads
positions without host rewrites; the host keeps a mirror for page allocation and limits.
The reference's cache is two dense tensors [L, Bmax, Hkv, Smax, hd] with the batch row as the
slot and one shared position (src/kv_cache.py:4-57).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .allocator import CacheError, FreeList, PageTableHost

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequest:
    """A mixer asks for keys and values of every earlier position (window 0) or of the last
    `window` positions. `name` tells several such requests of one unit apart."""
    n_kv_heads: int
    head_dim: int
    window: int = 0
    name: str = "kv"

    def geometry(self) -> Tuple[int, int, int]:
        """What decides which group's storage serves the request."""
        return (self.n_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateRequest:
    """A mixer asks for a fixed-size state per sequence (float32 unless `dtype` says otherwise),
    zeroed when a slot is taken."""
    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVUnit:
    """What an attention kernel needs of one unit."""
    k: torch.Tensor              # [pages + 1, kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor    # [slots + 1, max_pages_per_seq] int32
    page_size: int
    window: int


class CacheUnit:
    """The view of one schedule entry's storage that its layer gets: `kvs` and `state` by request name;
    `kv` is the keys and values named "kv", or the only ones there are."""

    def __init__(self, kvs: Dict[str, KVUnit], state: Dict[str, torch.Tensor]):
        self.kvs = kvs
        self.state = state       # name -> [slots + 1, *shape]
        self.kv = kvs.get("kv") or (next(iter(kvs.values())) if len(kvs) == 1 else None)

    def scoped(self, role: str) -> "CacheUnit":
        """The requests that a block prefixed with `role.` (a layer with several mixers), under the names the
        mixer gave them."""
        cut = len(role) + 1
        return CacheUnit({n[cut:]: u for n, u in self.kvs.items() if n.startswith(role + ".")},
                         {n[cut:]: t for n, t in self.state.items() if n.startswith(role + ".")})


class _KVGroup:
    def __init__(self, req: KVRequest, units: List[Tuple[int, str]], n_pages: int, n_slots: int, max_pages_per_seq: int,
                 dtype: torch.dtype, device):
        self.req = req
        self.units = units
        self.table = PageTableHost(n_pages, PAGE_SIZE, max_pages_per_seq, req.window)
        shape = (len(units), n_pages + 1, req.n_kv_heads, PAGE_SIZE, req.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.block_table = torch.full((n_slots + 1, max_pages_per_seq), n_pages, dtype=torch.int32, device=device)

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class Cache:
    def __init__(self, unit_requests: Sequence[Sequence[object]], n_slots: int, max_tokens: int,
                 max_seq_len: int, dtype: torch.dtype, device):
        """unit_requests[u] lists what unit u's mixer asked for. `max_tokens` is the number of
        positions all live sequences may hold together, each rounded up to whole pages."""
        if n_slots <= 0 or max_tokens <= 0 or max_seq_len <= 0:
            raise ValueError("n_slots, max_tokens and max_seq_len must be positive")
        self.page_size = PAGE_SIZE
        self.n_slots = n_slots
        self.scratch_slot = n_slots
        self.n_pages = (max_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        self.max_seq_len = max_seq_len
        self.max_pages_per_seq = min(self.n_pages, (max_seq_len + PAGE_SIZE - 1) // PAGE_SIZE)
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = FreeList(n_slots, "slot")
        self.lengths: List[int] = [0] * (n_slots + 1)          # host mirror of seq_lens
        self._mapped_upto: List[int] = [0] * (n_slots + 1)     # positions below this are writable without a new page
        self.seq_lens = torch.zeros(n_slots + 1, dtype=torch.int32, device=device)

        # groups by geometry (kv heads, head size, window); a member is (unit, request name)
        self._groups: Dict[Tuple[int, int, int], _KVGroup] = {}
        by_geometry: Dict[Tuple[int, int, int], List[Tuple[int, str]]] = {}
        first_request: Dict[Tuple[int, int, int], KVRequest] = {}
        state_specs: Dict[Tuple[str, Tuple[int, ...], torch.dtype], List[int]] = {}
        for u, reqs in enumerate(unit_requests):
            names = set()
            for r in reqs:
                if not isinstance(r, (KVRequest, StateRequest)):
                    raise TypeError(f"cache unit {u}: unknown request {r!r}")
                if (type(r), r.name) in names:
                    raise ValueError(f"cache unit {u}: two {type(r).__name__}s are named {r.name!r}; give them "
                                     "different names")
                names.add((type(r), r.name))
                if isinstance(r, KVRequest):
                    by_geometry.setdefault(r.geometry(), []).append((u, r.name))
                    first_request.setdefault(r.geometry(), r)
                else:
                    state_specs.setdefault((r.name, tuple(r.shape), r.dtype), []).append(u)
        for geo, members in by_geometry.items():
            self._groups[geo] = _KVGroup(first_request[geo], members, self.n_pages, n_slots, self.max_pages_per_seq,
                                         dtype, device)
        self._state: Dict[Tuple[str, Tuple[int, ...], torch.dtype], Tuple[List[int], torch.Tensor]] = {}
        for (name, shape, sdtype), units in state_specs.items():
            self._state[(name, shape, sdtype)] = (units, torch.zeros((len(units), n_slots + 1) + shape,
                                                                     dtype=sdtype, device=device))
        self._units: List[CacheUnit] = []
        for u, reqs in enumerate(unit_requests):
            kvs, state = {}, {}
            for r in reqs:
                if isinstance(r, KVRequest):
                    g = self._groups[r.geometry()]
                    i = g.units.index((u, r.name))
                    kvs[r.name] = KVUnit(g.k[i], g.v[i], g.block_table, PAGE_SIZE, r.window)
                else:
                    units, store = self._state[(r.name, tuple(r.shape), r.dtype)]
                    state[r.name] = store[units.index(u)]
            self._units.append(CacheUnit(kvs, state))

    # ---------------------------------------------------------------- views
    def unit(self, u: int) -> CacheUnit:
        return self._units[u]

    @property
    def n_units(self) -> int:
        return len(self._units)

    def groups(self) -> List[KVRequest]:
        """One request per group of units with storage of its own."""
        return [g.req for g in self._groups.values()]

    def bytes(self) -> int:
        return sum(g.bytes() for g in self._groups.values()) + \
            sum(s.numel() * s.element_size() for _, s in self._state.values())

    def free_pages(self) -> int:
        return min((g.table.pages.n_free for g in self._groups.values()), default=self.n_pages)

    def free_slots(self) -> int:
        return self.slots.n_free

    # ---------------------------------------------------------------- slots
    def take_slot(self) -> int:
        slot = self.slots.take()
        for g in self._groups.values():
            g.table.open_slot(slot)
        for units, store in self._state.values():
            store[:, slot].zero_()
        if self.lengths[slot] != 0:
            self.lengths[slot] = 0
        self._mapped_upto[slot] = 0
        self.seq_lens[slot:slot + 1].zero_()
        return slot

    def give_back_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is given back but is not held (freed twice?)")
        for g in self._groups.values():
            g.table.close_slot(slot)
            # The row names the scratch page again: whatever a later step addresses behind a sequence's last mapped
            # page must never lead to a page that has since been given to another sequence.
            g.block_table[slot].fill_(self.n_pages)
        self.slots.give_back(slot)
        self.lengths[slot] = 0
        self._mapped_upto[slot] = 0

    # ---------------------------------------------------------------- growth
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Free pages (of the tightest group) that appending n_new tokens to `slot` takes."""
        old = self.lengths[slot]
        return max((g.table.pages_needed(slot, old, old + n_new) for g in self._groups.values()), default=0)

    def can_hold(self, total_tokens: int) -> int:
        """Pages a fresh sequence of that many tokens would take."""
        return (total_tokens + PAGE_SIZE - 1) // PAGE_SIZE

    def reserve(self, slot: int, new_len: int) -> None:
        """Maps pages so that positions < new_len of `slot` can be written; updates the device
        block tables. Does not change the length."""
        if new_len <= self._mapped_upto[slot]:
            return                       # the common case of a one-token step inside a mapped page
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is not held")
        if new_len > self.max_seq_len:
            raise CacheError(f"slot {slot}: {new_len} tokens exceed max_seq_len {self.max_seq_len}")
        old = self.lengths[slot]
        for g in self._groups.values():
            need = g.table.pages_needed(slot, old, new_len)
            if need > g.table.pages.n_free:
                raise CacheError(f"cache is full: slot {slot} needs {need} more pages of {PAGE_SIZE} tokens, "
                                 f"{g.table.pages.n_free} are free (sized for {self.n_pages * PAGE_SIZE} tokens)")
        for g in self._groups.values():
            mapped = g.table.grow(slot, old, new_len)
            if mapped:
                lo = mapped[0][0]
                hi = mapped[-1][0] + 1
                if [lp for lp, _ in mapped] == list(range(lo, hi)):
                    row = torch.tensor([pp for _, pp in mapped], dtype=torch.int32)
                    g.block_table[slot, lo:hi].copy_(row)
                else:
                    for lp, pp in mapped:
                        g.block_table[slot, lp:lp + 1].copy_(torch.tensor([pp], dtype=torch.int32))
        if new_len > 0:
            self._mapped_upto[slot] = ((new_len - 1) // PAGE_SIZE + 1) * PAGE_SIZE

    def note_appended(self, slot: int, new_len: int, device_updated: bool) -> None:
        """Records that `slot` now holds new_len tokens. `device_updated` says whether a kernel
        has already written the device copy of the length."""
        self.lengths[slot] = new_len
        if not device_updated:
            self.seq_lens[slot:slot + 1].fill_(new_len)
        for g in self._groups.values():
            g.table.trim(slot, new_len)

    def check(self) -> None:
        self.slots.check()
        for g in self._groups.values():
            g.table.check()
