"""The cache manager: paged keys/values with a block table per request, one page pool per
group of layers with equal needs, and slots of fixed-size per-request state.

Layers are grouped by their `KVCacheSpec` (kv heads, head size, window). Each group has
pages of its own: a group that keeps every key grows with the request, a group with a
window gives pages back as soon as the window has passed them, and the pages of a request
that ends return at once and are handed out again. State layers (`StateSpec`) get one slot
per live request from a slot pool, zeroed when the request opens; Llama has none, the pool
then has no tensors.

Tensor layout per KV layer: K and V each [pages, kv_heads, page_size, head_dim], so that
one (page, head) is a contiguous [page_size, head_dim] tile.
Parity: src/model/kv_cache.rs:725-947 (pool), 949-1091 (per-sequence table) of the
reference; the grouping replaces its `kv_layer_map` (src/model/config.rs:1293-1335).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import KVCacheSpec, LayerCache, StateSpec
from .pages import CacheError, OutOfPages, PagePool


@dataclass
class CacheGroup:
    spec: KVCacheSpec
    layers: list[int]
    pool: PagePool
    k: dict[int, torch.Tensor] = field(default_factory=dict)
    v: dict[int, torch.Tensor] = field(default_factory=dict)


@dataclass
class RequestCache:
    """What one live request holds. `pages[g][i]` is the page of positions
    [i*page_size, (i+1)*page_size) in group g, or -1 once a window has passed it."""
    request_id: object
    num_tokens: int = 0
    pages: list[list[int]] = field(default_factory=list)
    state_slot: int = -1
    # `serial` tells two holdings apart even when a request id comes back (a preempted request is
    # opened again); `epoch` counts the changes to `pages` other than appending a page (a window
    # gave pages back, a step that did not run was trimmed). A copy of a block-table row is up to
    # date when serial, epoch and the page counts are what they were when it was made.
    serial: int = 0
    epoch: int = 0


def pages_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


class CacheManager:
    def __init__(self, specs: list, page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.dtype, self.device = page_size, dtype, device
        self.max_requests = max_requests
        self.groups: list[CacheGroup] = []
        self.layer_group: dict[int, int] = {}
        self.state_layers: dict[int, StateSpec] = {}
        self.state: dict[int, dict[str, torch.Tensor]] = {}
        for layer, spec in enumerate(specs):
            if isinstance(spec, KVCacheSpec):
                for gi, g in enumerate(self.groups):
                    if g.spec == spec:
                        g.layers.append(layer)
                        self.layer_group[layer] = gi
                        break
                else:
                    self.layer_group[layer] = len(self.groups)
                    self.groups.append(CacheGroup(spec, [layer], PagePool(num_pages)))
            elif isinstance(spec, StateSpec):
                self.state_layers[layer] = spec
            elif spec is not None:
                raise TypeError(f"cache layer {layer}: unknown spec {spec!r}")
        self.slots = PagePool(max_requests)
        if allocate:
            for g in self.groups:
                shape = (num_pages, g.spec.kv_heads, page_size, g.spec.head_dim)
                for layer in g.layers:
                    g.k[layer] = torch.zeros(shape, dtype=dtype, device=device)
                    g.v[layer] = torch.zeros(shape, dtype=dtype, device=device)
            for layer, spec in self.state_layers.items():
                self.state[layer] = {name: torch.zeros((max_requests,) + tuple(shape), dtype=dt, device=device)
                                     for name, shape, dt in spec.tensors}
        self.live: dict[object, RequestCache] = {}

    # ------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(specs: list, page_size: int, dtype: torch.dtype) -> int:
        per = torch.empty((), dtype=dtype).element_size()
        return sum(2 * s.kv_heads * s.head_dim * page_size * per for s in specs if isinstance(s, KVCacheSpec))

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    # ------------------------------------------------------------ request life cycle
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already open")
        slot = self.slots.alloc(request_id)          # OutOfPages when all slots are taken
        self._serial = getattr(self, "_serial", 0) + 1
        rc = RequestCache(request_id, 0, [[] for _ in self.groups], slot, serial=self._serial)
        for tensors in self.state.values():
            for t in tensors.values():
                t[slot].zero_()
        self.live[request_id] = rc
        return rc

    def first_needed_page(self, group: CacheGroup, num_tokens: int) -> int:
        """Pages below this index hold only keys that no later query can see."""
        if group.spec.window is None:
            return 0
        first_key = num_tokens - group.spec.window + 1   # oldest key the next query sees
        return max(0, first_key // self.page_size)

    def pages_needed(self, rc: RequestCache, new_total: int) -> list[int]:
        """Additional pages per group to hold positions [0, new_total)."""
        return [max(0, pages_for(new_total, self.page_size) - len(rc.pages[gi]))
                for gi in range(len(self.groups))]

    def can_reserve(self, rc: RequestCache | None, new_total: int) -> bool:
        have = [len(p) for p in rc.pages] if rc is not None else [0] * len(self.groups)
        need = pages_for(new_total, self.page_size)
        return all(need - have[gi] <= g.pool.num_free for gi, g in enumerate(self.groups))

    def reserve(self, rc: RequestCache, new_total: int) -> None:
        """Hold pages for positions [num_tokens, new_total) in every group, or none at all."""
        if new_total < rc.num_tokens:
            raise CacheError("a request cannot shrink")
        total = pages_for(new_total, self.page_size)
        if all(len(p) >= total for p in rc.pages):       # the common decode step: the last page has room
            return
        need = self.pages_needed(rc, new_total)
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.num_free:
                raise OutOfPages(f"group {gi} needs {need[gi]} pages, {g.pool.num_free} free")
        for gi, g in enumerate(self.groups):
            for _ in range(need[gi]):
                rc.pages[gi].append(g.pool.alloc(rc.request_id))

    def trim(self, rc: RequestCache) -> None:
        """Give back pages reserved beyond what the stored positions need (a step that
        did not run)."""
        keep = pages_for(rc.num_tokens, self.page_size)
        for gi, g in enumerate(self.groups):
            while len(rc.pages[gi]) > keep:
                rc.epoch += 1
                page = rc.pages[gi].pop()
                if page >= 0:
                    g.pool.free(page, rc.request_id)

    def commit(self, rc: RequestCache, new_total: int) -> None:
        """The step stored positions up to new_total; give back what a window has passed."""
        if pages_for(new_total, self.page_size) > min((len(p) for p in rc.pages), default=10 ** 9):
            raise CacheError("commit beyond the reserved pages")
        rc.num_tokens = new_total
        for gi, g in enumerate(self.groups):
            if g.spec.window is None:                     # every key is kept: nothing to give back
                continue
            last = min(self.first_needed_page(g, new_total), len(rc.pages[gi]))
            for i in range(last):
                if rc.pages[gi][i] >= 0:
                    g.pool.free(rc.pages[gi][i], rc.request_id)
                    rc.pages[gi][i] = -1
                    rc.epoch += 1

    def close(self, request_id) -> None:
        rc = self.live.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is not open")
        for gi, g in enumerate(self.groups):
            for page in rc.pages[gi]:
                if page >= 0:
                    g.pool.free(page, request_id)
            rc.pages[gi] = []
        self.slots.free(rc.state_slot, request_id)
        rc.state_slot = -1

    # ------------------------------------------------------------ for the step function
    def slot_of(self, rc: RequestCache, gi: int, position: int) -> int:
        page = rc.pages[gi][position // self.page_size]
        if page < 0:
            raise CacheError(f"position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def layer_view(self, cache_layer: int, ctx, writes: bool = True) -> LayerCache:
        if cache_layer in self.state_layers:
            return LayerCache(self.state_layers[cache_layer], state=self.state[cache_layer], writes=writes)
        gi = self.layer_group[cache_layer]
        g, view = self.groups[gi], ctx.groups[gi]
        return LayerCache(g.spec, self.page_size, g.k[cache_layer], g.v[cache_layer], view.slots,
                          view.block_table, writes)

    # ------------------------------------------------------------ checks (tests, debug)
    def check(self) -> None:
        """No page lost, held twice or freed twice; holders are live requests."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = {}
            for rc in self.live.values():
                for page in rc.pages[gi]:
                    if page < 0:
                        continue
                    if page in held:
                        raise CacheError(f"group {gi}: page {page} held by {held[page]!r} and {rc.request_id!r}")
                    held[page] = rc.request_id
                    if g.pool.owner(page) != rc.request_id:
                        raise CacheError(f"group {gi}: page {page} in a table but not held")
            if len(held) + g.pool.num_free != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.num_pages - len(held) - g.pool.num_free} pages lost")
        self.slots.check()
