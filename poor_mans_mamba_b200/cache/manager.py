"""The cache manager: pages with a block table per request for state that grows with the
sequence, slots for per-request state of fixed size.

Layers declare what they keep (StateSpec).  Paged states with the same row layout and
window form a *group*: the group has pages of its own ([member, page, plane, page_size,
width] on the device, one member per layer state) and one block table per request, shared
by the group's layers.  A group that only ever reads a window of the sequence gives pages
back as soon as the window has passed them.  Fixed states live in slots ([slot, *shape]
per layer state; the states of one shape and dtype are slices of one tensor, so that admitting a
request zeroes its slot in all layers with one fill per kind: 72 fills of the 36-layer model cost
the host 0.5 ms per admitted request).  Everything a request holds is given back when it
ends, and is used again.

The reference keeps one contiguous slot per request sized for max_seq tokens
(src/runtime/cache/cache_layout.cpp:103-139, cache_pool.cpp:86-126); only the zero-filled
fixed part and the take/give-back discipline carry over.

Index ``num_pages`` of every pool and index ``num_slots`` of every slot tensor are spare
entries that no request ever owns; padded rows of a fixed-shape batch point there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Tuple

import torch

from ..parts.base import LayerCache, PagedView, StateSpec
from .pages import OutOfPages, PageAccountingError, PagePool

Tensor = torch.Tensor


def _dtype_of(spec_dtype: str, compute: torch.dtype) -> torch.dtype:
    if spec_dtype == "compute":
        return compute
    if spec_dtype == "float32":
        return torch.float32
    raise ValueError(f"unknown state dtype {spec_dtype!r}")


@dataclass
class _Member:
    layer: int
    name: str


class PagedGroup:
    """Pages and block tables of the layer states that share one row layout and window."""

    def __init__(self, key: Tuple, planes: int, width: int, window: int, page_size: int, num_pages: int):
        self.key = key
        self.planes, self.width, self.window = planes, width, window
        self.page_size, self.num_pages = page_size, num_pages
        self.members: List[_Member] = []
        self.pool = PagePool(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}  # logical block -> page, -1 once given back
        self.storage: Optional[Tensor] = None

    def blocks_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def first_needed_block(self, next_pos: int) -> int:
        """The first logical block that a token at position >= next_pos can still read."""
        if self.window <= 0:
            return 0
        return max(0, next_pos - self.window + 1) // self.page_size

    def pages_to_grow(self, req: Hashable, new_len: int) -> int:
        return max(0, self.blocks_for(new_len) - len(self.tables.get(req, [])))


class CacheManager:
    def __init__(self, state_specs: Dict[int, List[Tuple[str, StateSpec]]], page_size: int, num_pages: int,
                 num_slots: int, dtype: torch.dtype, device, pages_per_group: Optional[Dict[Tuple, int]] = None):
        if page_size <= 0 or num_slots <= 0:
            raise ValueError("page_size and num_slots must be positive")
        self.page_size, self.num_slots = int(page_size), int(num_slots)
        self.dtype, self.device = dtype, torch.device(device)
        self.groups: Dict[Tuple, PagedGroup] = {}
        self._paged_of: Dict[Tuple[int, str], Tuple[PagedGroup, int]] = {}
        self._fixed: Dict[Tuple[int, str], Tensor] = {}
        fixed_kinds: Dict[Tuple, List[Tuple[int, str]]] = {}
        for layer, specs in sorted(state_specs.items()):
            for name, spec in specs:
                if spec.kind == "paged":
                    key = (spec.planes, spec.width, spec.window)
                    if key not in self.groups:
                        n = (pages_per_group or {}).get(key, num_pages)
                        self.groups[key] = PagedGroup(key, spec.planes, spec.width, spec.window,
                                                      self.page_size, int(n))
                    g = self.groups[key]
                    self._paged_of[(layer, name)] = (g, len(g.members))
                    g.members.append(_Member(layer, name))
                elif spec.kind == "fixed":
                    kind = (tuple(int(d) for d in spec.shape), _dtype_of(spec.dtype, dtype))
                    fixed_kinds.setdefault(kind, []).append((layer, name))
                else:
                    raise ValueError(f"unknown state kind {spec.kind!r}")
        # Fixed states of one shape and dtype share a tensor [member, slot, *shape]: a layer's state
        # is the contiguous [slot, *shape] it always was, and a request's slot is zeroed in all
        # layers with one fill per kind instead of one per layer state.
        self._fixed_stores: List[Tensor] = []
        for (shape, dt), members in fixed_kinds.items():
            store = torch.zeros((len(members), self.num_slots + 1, *shape), dtype=dt, device=self.device)
            self._fixed_stores.append(store)
            for m, member in enumerate(members):
                self._fixed[member] = store[m]
        for g in self.groups.values():
            g.storage = torch.zeros((len(g.members), g.num_pages + 1, g.planes, g.page_size, g.width),
                                    dtype=dtype, device=self.device)
        self._free_slots: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}
        self.lengths: Dict[Hashable, int] = {}  # tokens whose state each live request holds
        self.admissions: Dict[Hashable, int] = {}  # a number that changes every time a request is admitted
        self._admission_counter = 0
        self.layers = sorted(state_specs)

    # ------------------------------------------------------------------ requests
    def admit(self, req: Hashable) -> int:
        """Take a slot for a new request; its fixed state starts at zero."""
        if req in self._slot_of:
            raise ValueError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise OutOfPages("no free state slot")
        slot = self._free_slots.pop()
        self._slot_of[req] = slot
        self.lengths[req] = 0
        self._admission_counter += 1
        self.admissions[req] = self._admission_counter
        for store in self._fixed_stores:
            store[:, slot].zero_()
        for g in self.groups.values():
            g.tables[req] = []
        return slot

    def has(self, req: Hashable) -> bool:
        return req in self._slot_of

    def slot(self, req: Hashable) -> int:
        return self._slot_of[req]

    def pages_needed(self, req: Hashable, new_len: int) -> Dict[Tuple, int]:
        """Pages each group must still take so that ``req`` can hold ``new_len`` tokens."""
        return {k: g.pages_to_grow(req, new_len) for k, g in self.groups.items()}

    def can_grow(self, req: Hashable, new_len: int, reserved: Optional[Dict[Tuple, int]] = None) -> bool:
        reserved = reserved or {}
        return all(g.pages_to_grow(req, new_len) + reserved.get(k, 0) <= g.pool.n_free
                   for k, g in self.groups.items())

    def grow(self, req: Hashable, new_len: int) -> None:
        """Give ``req`` pages for positions up to new_len-1 in every group, or none at all."""
        if req not in self._slot_of:
            raise KeyError(f"request {req!r} is not admitted")
        if not self.can_grow(req, new_len):
            raise OutOfPages(f"not enough free pages for request {req!r} to reach {new_len} tokens")
        for g in self.groups.values():
            table = g.tables[req]
            while len(table) < g.blocks_for(new_len):  # every new position is written, windowed or not
                table.append(g.pool.alloc(req))

    def trim(self, req: Hashable, cur_len: int) -> int:
        """Give back the pages that no later token of ``req`` (position >= cur_len) can read."""
        n = 0
        for g in self.groups.values():
            if g.window <= 0:
                continue
            table = g.tables[req]
            for b in range(min(g.first_needed_block(cur_len), len(table))):
                if table[b] >= 0:
                    g.pool.free(table[b], req)
                    table[b] = -1
                    n += 1
        return n

    def release(self, req: Hashable) -> None:
        """The request has ended: everything it holds is given back."""
        if req not in self._slot_of:
            raise KeyError(f"request {req!r} is not admitted (released twice?)")
        for g in self.groups.values():
            for page in g.tables.pop(req):
                if page >= 0:
                    g.pool.free(page, req)
        self._free_slots.append(self._slot_of.pop(req))
        del self.lengths[req]
        del self.admissions[req]

    def advance(self, req: Hashable, n_tokens: int) -> int:
        """A step has written ``n_tokens`` more tokens of ``req``; pages that a window has
        passed are given back.  Returns the new length."""
        self.lengths[req] += int(n_tokens)
        self.trim(req, self.lengths[req])
        return self.lengths[req]

    # ------------------------------------------------------------------ queries
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> Dict[Tuple, int]:
        return {k: g.pool.n_free for k, g in self.groups.items()}

    def min_free_pages(self) -> int:
        return min((g.pool.n_free for g in self.groups.values()), default=1 << 30)

    def block_table(self, req: Hashable, key: Tuple) -> List[int]:
        return self.groups[key].tables[req]

    def live_requests(self) -> List[Hashable]:
        return list(self._slot_of)

    def check(self) -> None:
        """Raises unless no page or slot is lost, held twice or both free and held."""
        for g in self.groups.values():
            g.pool.check()
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(held) != len(set(held)):
                raise PageAccountingError("a page is in two block tables")
            if len(held) != g.pool.n_held:
                raise PageAccountingError("pages are held that no block table names")
            for req, t in g.tables.items():
                for p in t:
                    if p >= 0 and g.pool.owner(p) != req:
                        raise PageAccountingError(f"page {p} in the table of {req!r} belongs to someone else")
        slots = list(self._slot_of.values()) + self._free_slots
        if sorted(slots) != list(range(self.num_slots)):
            raise PageAccountingError("a state slot is lost or held twice")

    # ------------------------------------------------------------------ views for a step
    def spare_page(self, key: Tuple) -> int:
        return self.groups[key].num_pages

    @property
    def spare_slot(self) -> int:
        return self.num_slots

    def layer_caches(self, block_tables: Dict[Tuple, Tensor]) -> Dict[int, LayerCache]:
        """Per layer, the views its mixers use during a step; ``block_tables`` holds the step's
        device table [n_seq, max_blocks] of every group."""
        paged: Dict[int, Dict[str, PagedView]] = {l: {} for l in self.layers}
        fixed: Dict[int, Dict[str, Tensor]] = {l: {} for l in self.layers}
        for (layer, name), (g, m) in self._paged_of.items():
            paged[layer][name] = PagedView(g.storage[m], block_tables[g.key], g.page_size, g.window)
        for (layer, name), t in self._fixed.items():
            fixed[layer][name] = t
        return {l: LayerCache(paged[l], fixed[l]) for l in self.layers}

    def bytes_per_token(self) -> int:
        return sum(len(g.members) * g.planes * g.width * g.storage.element_size() for g in self.groups.values())

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self._fixed.values())
