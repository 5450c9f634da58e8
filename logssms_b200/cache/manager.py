"""The cache manager: paged keys/values per layer group, state slots per request.

What a model needs is collected from its mixers (`CacheNeeds` per cache layer):
  * `PagedNeed`: tensors of a fixed shape per token, in pages (`KVNeed(heads, head size, window)` writes the
    common one: keys and values of one shape; a cache of latents has one tensor, keys and values of different
    head sizes two of different shapes).  Cache layers whose needs are equal form one *group*; each group has its
    own page pool, its own storage and, per request, its own block table.  A group with a window gives pages back
    as soon as the window has passed them.
  * `StateNeed`: a tensor of fixed size per request (a conv window, an SSM
    state).  One slot per live request; the slot index is the request's row.

Lifetime of a request: `admit` (takes a row/slot; optionally reserves pages for
its whole life so that later steps cannot run dry) -> `extend` before every step
that appends tokens -> `release`.  With `poison_on_free` freed pages and slots
are filled with NaN on the device, so a stale read shows up in the logits.

The reference's counterpart is its naive cache manager plus the two pools
(python/logssms/cache/naive/manager.py:38-335, python/logssms/cache/radix/mha_pool.py:13-68,
python/logssms/cache/radix/state_pool.py:12-42).  Differences: block tables hold page ids
(not a token index per position), one state slot per request (no slot per page: there is no
prefix reuse here), and the SSM state is 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .pools import FreeList, OutOfPages


@dataclass(frozen=True)
class PagedTensor:
    name: str
    shape: tuple[int, ...]                # per token
    dtype: torch.dtype | None = None      # None: the engine's activation dtype


@dataclass(frozen=True)
class PagedNeed:
    """What a cache layer keeps per token, in pages: named tensors; `window`: only the last so many tokens are read."""
    tensors: tuple[PagedTensor, ...]
    window: int | None = None


def KVNeed(num_kv_heads: int, head_dim: int, window: int | None = None, value_head_dim: int | None = None) -> PagedNeed:
    """Keys "k" and values "v" of [num_kv_heads, head_dim] per token (values of another head size if given)."""
    return PagedNeed((PagedTensor("k", (num_kv_heads, head_dim)),
                      PagedTensor("v", (num_kv_heads, value_head_dim or head_dim))), window)


@dataclass(frozen=True)
class StateNeed:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype | None = None      # None: the engine's activation dtype


@dataclass(frozen=True)
class CacheNeeds:
    kv: PagedNeed | None = None           # the layer's paged tensors (keys and values, mostly)
    states: tuple[StateNeed, ...] = ()


class PageGroup:
    """Cache layers with equal paged needs: one page pool, one storage, one block table per request."""

    def __init__(self, need: PagedNeed, layers: list[int], num_pages: int, page_size: int, max_requests: int,
                 max_pages_per_request: int, dtype, device):
        self.need = need
        self.layers = layers
        self.page_size = page_size
        self.pool = FreeList(num_pages, "page")
        self.layer_index = {layer: i for i, layer in enumerate(layers)}
        # per tensor of the need: [layers, pages, page_size, *shape per token]
        # one page more than the pool hands out: the dummy page (index `num_pages`), where the dummy requests of a
        # padded step keep their keys and values; its block-table row is the last one
        self.storage = {t.name: torch.zeros((len(layers), num_pages + 1, page_size, *t.shape), dtype=t.dtype or dtype,
                                            device=device) for t in need.tensors}
        self.block_table = np.full((max_requests + 1, max_pages_per_request), -1, dtype=np.int32)
        self.block_table[max_requests, :] = num_pages
        self.first_page = np.zeros(max_requests, dtype=np.int64)     # pages below are given back (window)
        self.num_pages_of = np.zeros(max_requests, dtype=np.int64)    # logical pages handed out so far

    def tensor(self, name: str, layer: int) -> torch.Tensor:
        """[pages, page_size, *shape per token] of one cache layer."""
        return self.storage[name][self.layer_index[layer]]

    def k_cache(self, layer: int) -> torch.Tensor:
        return self.tensor("k", layer)

    def v_cache(self, layer: int) -> torch.Tensor:
        return self.tensor("v", layer)

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def lifetime_pages(self, total_len: int, max_step_tokens: int) -> int:
        """Most pages a request of `total_len` tokens holds at any time."""
        full = self.pages_for(total_len)
        if self.need.window is None:
            return full
        # live span while a step of `max_step_tokens` runs: window - 1 earlier keys + the step's tokens
        return min(full, self.pages_for(self.need.window - 1 + max_step_tokens) + 1)


@dataclass
class RequestCache:
    """What the cache manager knows about a live request."""
    row: int                       # state slot and block-table row
    length: int = 0                # tokens whose keys/values have room
    reserved: dict = field(default_factory=dict)   # group index -> pages reserved for the whole life


class CacheManager:
    def __init__(self, needs: list[CacheNeeds], *, page_size: int, num_pages: int, max_requests: int,
                 max_seq_len: int, dtype, device, poison_on_free: bool = False, max_step_tokens: int = 1 << 30):
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.device = torch.device(device)
        self.dtype = dtype
        self.poison_on_free = poison_on_free
        self.max_step_tokens = max_step_tokens
        self.max_pages_per_request = -(-max_seq_len // page_size)
        self.rows = FreeList(max_requests, "request slot")
        self.live: dict[int, RequestCache] = {}
        # Row, state slot and (per group) page that no request ever gets: a step that is filled up to fixed sizes
        # (`engine.plan.Bucket`) lets its dummy requests read and write there.
        self.dummy_row = max_requests

        by_need: dict[PagedNeed, list[int]] = {}
        for layer, need in enumerate(needs):
            if need.kv is not None:
                by_need.setdefault(need.kv, []).append(layer)
        self.groups = [PageGroup(need, layers, num_pages, page_size, max_requests, self.max_pages_per_request,
                                 dtype, self.device) for need, layers in by_need.items()]
        self.group_of_layer = {layer: gi for gi, g in enumerate(self.groups) for layer in g.layers}
        self._unclaimed = [0] * len(self.groups)     # reserved but not yet handed out, per group

        self.states: list[dict[str, torch.Tensor]] = []
        for need in needs:
            per_layer = {}
            for s in need.states:
                per_layer[s.name] = torch.zeros((max_requests + 1, *s.shape), dtype=s.dtype or dtype, device=self.device)
            self.states.append(per_layer)

    # ------------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(needs: list[CacheNeeds], page_size: int, dtype) -> int:
        size = lambda t: int(np.prod(t.shape)) * torch.empty((), dtype=t.dtype or dtype).element_size()
        return sum(page_size * size(t) for n in needs if n.kv is not None for t in n.kv.tensors)

    @staticmethod
    def bytes_per_request_state(needs: list[CacheNeeds], dtype) -> int:
        total = 0
        for n in needs:
            for s in n.states:
                total += int(np.prod(s.shape)) * torch.empty((), dtype=s.dtype or dtype).element_size()
        return total

    # ------------------------------------------------------------------ admission
    def available_pages(self, gi: int) -> int:
        return self.groups[gi].pool.num_free - self._unclaimed[gi]

    def can_admit(self, reserve_tokens: int = 0) -> bool:
        if self.rows.num_free == 0:
            return False
        return all(self.available_pages(gi) >= g.lifetime_pages(reserve_tokens, self.max_step_tokens)
                   for gi, g in enumerate(self.groups))

    def fits_at_all(self, total_tokens: int) -> bool:
        """Could a request of this length ever run, with the pools empty?"""
        if total_tokens > self.max_seq_len:
            return False
        return all(g.pool.count >= g.lifetime_pages(total_tokens, self.max_step_tokens) for g in self.groups)

    def admit(self, reserve_tokens: int = 0) -> RequestCache:
        """Take a request row.  `reserve_tokens` > 0 sets aside the pages the request needs over its
        whole life (prompt + generated tokens); 0 leaves every `extend` to find free pages itself."""
        if reserve_tokens > self.max_seq_len:
            raise OutOfPages(f"request of {reserve_tokens} tokens exceeds max_seq_len {self.max_seq_len}")
        if not self.can_admit(reserve_tokens):
            raise OutOfPages("no room to admit the request")
        (row,) = self.rows.alloc(1)
        rc = RequestCache(row=row)
        if reserve_tokens > 0:
            for gi, g in enumerate(self.groups):
                n = g.lifetime_pages(reserve_tokens, self.max_step_tokens)
                rc.reserved[gi] = n
                self._unclaimed[gi] += n
        for g in self.groups:
            g.block_table[row, :] = -1
            g.first_page[row] = 0
            g.num_pages_of[row] = 0
        self.live[row] = rc
        return rc

    # ------------------------------------------------------------------ growth
    def extend(self, rc: RequestCache, new_length: int, first_pos: int | None = None) -> None:
        """Make room for positions [rc.length, new_length) in every group; for a group with a window,
        first give back the pages that no token of this step can still see.  `first_pos`: the position of the
        step's first token where that is not rc.length (a step planned once more after the cache has grown)."""
        if new_length < rc.length:
            raise ValueError("a request's cache never shrinks")
        if new_length > self.max_seq_len:
            raise OutOfPages(f"request grows to {new_length} tokens, beyond max_seq_len {self.max_seq_len}")
        for gi, g in enumerate(self.groups):
            if g.need.window is not None:
                self._drop_behind(gi, rc, rc.length if first_pos is None else min(first_pos, rc.length))   # the step's first token
            want = g.pages_for(new_length)
            have = int(g.num_pages_of[rc.row])
            if want > have:
                beyond_reservation = (want - have) - rc.reserved.get(gi, 0)
                if beyond_reservation > self.available_pages(gi):      # never eat what others were promised
                    raise OutOfPages(f"group {gi}: request row {rc.row} needs {want - have} more pages, "
                                     f"{self.available_pages(gi)} are free and unpromised")
                pages = g.pool.alloc(want - have)
                g.block_table[rc.row, have:want] = pages
                g.num_pages_of[rc.row] = want
                if gi in rc.reserved:
                    self._claim(gi, rc, want - have)
        rc.length = new_length

    def check_room(self, growth: list[tuple[RequestCache, int]]) -> None:
        """Raise `OutOfPages` unless `extend(rc, new_length)` will succeed for ALL the given pairs, one after the
        other; nothing is changed.  A step extends several requests: without this check a later one could run dry
        after earlier ones had already grown, although none of the step's tokens ever ran."""
        for gi, g in enumerate(self.groups):
            available = self.available_pages(gi)
            for rc, new_length in growth:
                if new_length < rc.length:
                    raise ValueError("a request's cache never shrinks")
                if new_length > self.max_seq_len:
                    raise OutOfPages(f"request grows to {new_length} tokens, beyond max_seq_len {self.max_seq_len}")
                have, reserved = int(g.num_pages_of[rc.row]), rc.reserved.get(gi, 0)
                if g.need.window is not None:
                    # pages the window has passed go back first; a request with a reservation may claim them again
                    oldest_needed = max(0, rc.length - g.need.window + 1)
                    given_back = max(0, min(oldest_needed // g.page_size, have) - int(g.first_page[rc.row]))
                    if gi in rc.reserved:
                        reserved += given_back
                    else:
                        available += given_back
                beyond = max(0, g.pages_for(new_length) - have) - reserved
                if beyond > available:
                    raise OutOfPages(f"group {gi}: request row {rc.row} needs {beyond} more pages than it reserved, "
                                     f"{max(available, 0)} are free and unpromised")
                available -= max(beyond, 0)

    def _claim(self, gi: int, rc: RequestCache, n: int) -> None:
        take = min(n, rc.reserved[gi])
        rc.reserved[gi] -= take
        self._unclaimed[gi] -= take

    def _drop_behind(self, gi: int, rc: RequestCache, first_query_pos: int) -> None:
        g = self.groups[gi]
        oldest_needed = max(0, first_query_pos - g.need.window + 1)
        keep_from = min(oldest_needed // g.page_size, int(g.num_pages_of[rc.row]))
        lo = int(g.first_page[rc.row])
        if keep_from > lo:
            pages = [int(p) for p in g.block_table[rc.row, lo:keep_from]]
            self._free_pages(gi, pages)
            g.block_table[rc.row, lo:keep_from] = -1
            g.first_page[rc.row] = keep_from
            if gi in rc.reserved:            # a returned page may be claimed again by this request
                rc.reserved[gi] += len(pages)
                self._unclaimed[gi] += len(pages)

    def _free_pages(self, gi: int, pages: list[int]) -> None:
        g = self.groups[gi]
        if self.poison_on_free and pages:
            idx = torch.tensor(pages, device=self.device, dtype=torch.long)
            for t in g.storage.values():
                t[:, idx] = float("nan") if t.is_floating_point() else -1
        g.pool.free(pages)

    # ------------------------------------------------------------------ end of life
    def release(self, rc: RequestCache) -> None:
        if self.live.get(rc.row) is not rc:
            raise ValueError(f"request row {rc.row} released twice (or never admitted)")
        for gi, g in enumerate(self.groups):
            lo, hi = int(g.first_page[rc.row]), int(g.num_pages_of[rc.row])
            self._free_pages(gi, [int(p) for p in g.block_table[rc.row, lo:hi]])
            g.block_table[rc.row, :] = -1
            g.first_page[rc.row] = 0
            g.num_pages_of[rc.row] = 0
            if gi in rc.reserved:
                self._unclaimed[gi] -= rc.reserved[gi]
        rc.reserved.clear()
        if self.poison_on_free:
            for per_layer in self.states:
                for t in per_layer.values():
                    t[rc.row] = float("nan") if t.is_floating_point() else -1
        del self.live[rc.row]
        self.rows.free([rc.row])

    # ------------------------------------------------------------------ views for the step function
    def kv(self, layer: int) -> tuple[torch.Tensor, torch.Tensor, int]:
        gi = self.group_of_layer[layer]
        g = self.groups[gi]
        return g.k_cache(layer), g.v_cache(layer), gi

    def slot_of(self, gi: int, rc: RequestCache, position: int) -> int:
        g = self.groups[gi]
        page = int(g.block_table[rc.row, position // g.page_size])
        if page < 0:
            raise AssertionError(f"position {position} of request row {rc.row} has no page in group {gi}")
        return page * g.page_size + position % g.page_size

    # ------------------------------------------------------------------ checks
    def check_integrity(self) -> None:
        """No page lost, held twice or freed twice; reservations add up; rows consistent."""
        self.rows.check()
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen: set[int] = set()
            for row, rc in self.live.items():
                lo, hi = int(g.first_page[row]), int(g.num_pages_of[row])
                pages = [int(p) for p in g.block_table[row, lo:hi]]
                for p in pages:
                    if p < 0 or not g.pool.is_held(p):
                        raise AssertionError(f"group {gi}: row {row} lists page {p} that it does not hold")
                    if p in seen:
                        raise AssertionError(f"group {gi}: page {p} is held twice")
                    seen.add(p)
                if (g.block_table[row, :lo] != -1).any() or (g.block_table[row, hi:] != -1).any():
                    raise AssertionError(f"group {gi}: row {row} has entries outside its live pages")
            if len(seen) != g.pool.num_held:
                raise AssertionError(f"group {gi}: {g.pool.num_held - len(seen)} pages are held by nobody")
            if sum(rc.reserved.get(gi, 0) for rc in self.live.values()) != self._unclaimed[gi]:
                raise AssertionError(f"group {gi}: reservations do not add up")
            if self._unclaimed[gi] > g.pool.num_free:
                raise AssertionError(f"group {gi}: more pages promised than free")
        if set(self.live) != {i for i in range(self.max_requests) if self.rows.is_held(i)}:
            raise AssertionError("live requests and held rows differ")
