"""The cache manager: paged keys/values with a block table per request, one page pool per
group of layers with equal needs, and slots of fixed-size per-request state.

How a layer's need is served is looked up by the class of its spec (`parts.base.CacheKind`,
`register_cache_kind`); the manager knows no spec class by name. Layers of a paged kind are
grouped by equal specs (`KVCacheSpec`: kv heads, head size, window). Each group has pages of its
own, and a pool of its own size: a group that keeps every key grows with the request, a group
with a window gives pages back as soon as the window has passed them, and the pages of a request
that ends return at once and are handed out again. Layers of a slot kind (`StateSpec`) get one
slot per live request from a slot pool, zeroed when the request opens; Llama has none, the pool
then has no tensors.

The bookkeeping (pools, tables, state slots) is native: csrc/host_runtime.cpp.

Tensor layout per KV layer: K and V each [pages, kv_heads, page_size, head_dim], so that
one (page, head) is a contiguous [page_size, head_dim] tile.
Parity: src/model/kv_cache.rs:725-947 (pool), 949-1091 (per-sequence table) of the
reference; the grouping replaces its `kv_layer_map` (src/model/config.rs:1293-1335).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import LayerCache, cache_kind_of
from .native import lib
from .pages import CacheError, Holders, OutOfPages, PagePool


@dataclass
class CacheGroup:
    spec: object
    layers: list[int]
    pool: PagePool
    tensors: dict[int, dict[str, torch.Tensor]] = field(default_factory=dict)    # layer -> name -> tensor

    @property
    def k(self) -> dict[int, torch.Tensor]:
        return {layer: t["k"] for layer, t in self.tensors.items() if "k" in t}

    @property
    def v(self) -> dict[int, torch.Tensor]:
        return {layer: t["v"] for layer, t in self.tensors.items() if "v" in t}


class RequestCache:
    """What one live request holds; the numbers live in the native tables, this object names
    them. `pages[g][i]` is the page of positions [i*page_size, (i+1)*page_size) in group g, or
    -1 once a window has passed it. `serial` tells two holdings apart even when a request id
    comes back (a preempted request is opened again); `epoch` counts the changes to the tables
    other than appending a page."""
    __slots__ = ("_m", "request_id", "handle")

    def __init__(self, manager, request_id, handle: int):
        self._m, self.request_id, self.handle = manager, request_id, handle

    @property
    def state_slot(self) -> int:
        return self.handle

    @property
    def num_tokens(self) -> int:
        return self._m._L.cache_num_tokens(self._m._ptr, self.handle) if self.handle >= 0 else 0

    @property
    def serial(self) -> int:
        return self._m._L.cache_serial(self._m._ptr, self.handle)

    @property
    def epoch(self) -> int:
        return self._m._L.cache_epoch(self._m._ptr, self.handle)

    def num_held(self, group: int) -> int:
        """Entries of the block table of `group` (given-back pages included)."""
        return self._m._L.cache_num_held(self._m._ptr, self.handle, group) if self.handle >= 0 else 0

    def pages_array(self, group: int) -> np.ndarray:
        if self.handle < 0:
            return np.empty(0, dtype=np.int32)
        n = self.num_held(group)
        out = np.empty(max(n, 1), dtype=np.int32)
        self._m._L.cache_pages(self._m._ptr, self.handle, group, out.ctypes.data, n)
        return out[:n]

    @property
    def pages(self) -> list[list[int]]:
        return [self.pages_array(g).tolist() for g in range(len(self._m.groups))]


def pages_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


class CacheManager:
    def __init__(self, specs: list, page_size: int, num_pages, max_requests: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        """`num_pages`: pages of every group's pool, or a mapping spec -> pages for groups that
        differ (a spec it does not name gets what its kind's `num_pages` makes of the largest)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size, self.dtype, self.device = page_size, dtype, device
        self.max_requests = max_requests
        self.groups: list[CacheGroup] = []
        self.layer_group: dict[int, int] = {}
        self.state_layers: dict[int, object] = {}
        self.state: dict[int, dict[str, torch.Tensor]] = {}
        group_specs: list = []
        group_layers: list[list[int]] = []
        for layer, spec in enumerate(specs):
            if spec is None:
                continue
            try:
                kind = cache_kind_of(spec)
            except TypeError as e:
                raise TypeError(f"cache layer {layer}: {e}") from None
            if kind.paged:
                for gi, gs in enumerate(group_specs):
                    if type(gs) is type(spec) and gs == spec:
                        group_layers[gi].append(layer)
                        self.layer_group[layer] = gi
                        break
                else:
                    self.layer_group[layer] = len(group_specs)
                    group_specs.append(spec)
                    group_layers.append([layer])
            else:
                self.state_layers[layer] = spec
        by_spec = num_pages if isinstance(num_pages, dict) else {}
        default = max(by_spec.values(), default=0) if isinstance(num_pages, dict) else int(num_pages)
        pages_of = [int(by_spec[gs]) if gs in by_spec else int(cache_kind_of(gs).num_pages(gs, default))
                    for gs in group_specs]
        # the native tables: one pool per group, the state slots, every holding
        self._L = lib()
        G = len(group_specs)
        counts = (ctypes.c_int * max(G, 1))(*pages_of)
        windows = (ctypes.c_int * max(G, 1))(*[(-1 if cache_kind_of(gs).window(gs) is None else cache_kind_of(gs).window(gs))
                                               for gs in group_specs])
        self._ptr = self._L.cache_new(G, counts, windows, page_size, max_requests)
        if not self._ptr:
            raise ValueError("the native cache tables could not be made")
        self.holders = Holders()
        for gi, (gs, layers) in enumerate(zip(group_specs, group_layers)):
            pool = PagePool(pages_of[gi], _ptr=self._L.cache_pool(self._ptr, gi), _holders=self.holders, _owner=self)
            self.groups.append(CacheGroup(gs, layers, pool))
        self.slots = PagePool(max_requests, _ptr=self._L.cache_slots(self._ptr), _holders=self.holders, _owner=self)
        if allocate:
            for g in self.groups:
                kind = cache_kind_of(g.spec)
                for layer in g.layers:
                    g.tensors[layer] = kind.allocate(g.spec, g.pool.num_pages, page_size, dtype, device)
            for layer, spec in self.state_layers.items():
                self.state[layer] = cache_kind_of(spec).allocate(spec, max_requests, None, dtype, device)
        self.live: dict[object, RequestCache] = {}

    def __del__(self):
        if getattr(self, "_ptr", None):
            self._L.cache_delete(self._ptr)
            self._ptr = None

    # ------------------------------------------------------------ sizes
    @staticmethod
    def bytes_per_page(specs: list, page_size: int, dtype: torch.dtype) -> int:
        """Bytes one page costs over all paged layers (each layer has the page in its own tensors)."""
        return sum(cache_kind_of(s).page_bytes(s, page_size, dtype) for s in specs
                   if s is not None and cache_kind_of(s).paged)

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    @staticmethod
    def _raise(rc: int, what: str):
        if rc <= -10:
            raise CacheError(f"{what}: the pool refused a release (code {rc + 10}): a page was freed twice "
                             f"or is held by another request")
        raise CacheError(f"{what}: no such holding" if rc == -9 else f"{what}: code {rc}")

    # ------------------------------------------------------------ request life cycle
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already open")
        handle = self._L.cache_open(self._ptr, self.holders.key(request_id))
        if handle == -1:
            raise OutOfPages("no free state slot")          # all slots are taken
        if handle < 0:
            self._raise(handle, "open")
        rc = RequestCache(self, request_id, handle)
        for tensors in self.state.values():
            for t in tensors.values():
                t[handle].zero_()
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
        total = pages_for(new_total, self.page_size)
        return [max(0, total - rc.num_held(gi)) for gi in range(len(self.groups))]

    def held_pages(self, rc: RequestCache) -> list[int]:
        """Pages per group the request really holds (given-back entries not counted)."""
        return [int((rc.pages_array(gi) >= 0).sum()) for gi in range(len(self.groups))]

    def can_reserve(self, rc: RequestCache | None, new_total: int) -> bool:
        return bool(self._L.cache_can_reserve(self._ptr, rc.handle if rc is not None else -1, new_total))

    def reserve(self, rc: RequestCache, new_total: int) -> None:
        """Hold pages for positions [num_tokens, new_total) in every group, or none at all."""
        code = self._L.cache_reserve(self._ptr, rc.handle, new_total)
        if code == 0:
            return
        if code == -1:
            raise OutOfPages(f"not enough free pages for {new_total} positions ({self.free_pages()} free)")
        if code == -2:
            raise CacheError("a request cannot shrink")
        self._raise(code, "reserve")

    def trim(self, rc: RequestCache) -> None:
        """Give back pages reserved beyond what the stored positions need (a step that
        did not run)."""
        code = self._L.cache_trim(self._ptr, rc.handle)
        if code:
            self._raise(code, "trim")

    def commit(self, rc: RequestCache, new_total: int) -> None:
        """The step stored positions up to new_total; give back what a window has passed."""
        code = self._L.cache_commit(self._ptr, rc.handle, new_total)
        if code == -2:
            raise CacheError("commit beyond the reserved pages")
        if code:
            self._raise(code, "commit")

    def close(self, request_id) -> None:
        rc = self.live.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is not open")
        code = self._L.cache_close(self._ptr, rc.handle)
        rc.handle = -1
        self.holders.forget(request_id)
        if code:
            self._raise(code, "close")

    # ------------------------------------------------------------ for the step function
    def slot_of(self, rc: RequestCache, gi: int, position: int) -> int:
        page = int(rc.pages_array(gi)[position // self.page_size])
        if page < 0:
            raise CacheError(f"position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def layer_view(self, cache_layer: int, ctx, writes: bool = True) -> LayerCache:
        if cache_layer in self.state_layers:
            return LayerCache(self.state_layers[cache_layer], state=self.state[cache_layer], writes=writes,
                              tensors=self.state[cache_layer])
        gi = self.layer_group[cache_layer]
        g, view = self.groups[gi], ctx.groups[gi]
        t = g.tensors[cache_layer]
        return LayerCache(g.spec, self.page_size, t.get("k"), t.get("v"), view.slots, view.block_table, writes,
                          tensors=t)

    # ------------------------------------------------------------ checks (tests, debug)
    def check(self) -> None:
        """No page lost, held twice or freed twice; holders are live requests."""
        code = self._L.cache_check(self._ptr)
        if code == 0:
            return
        if code >= 1000:
            raise CacheError("the state slots' free list and holders disagree")
        gi, what = code // 100 - 1, code % 100
        names = {4: "a table names a page that does not exist", 5: "a page is in two tables",
                 6: "a page is in a table but not held by that request", 7: "pages are lost"}
        raise CacheError(f"group {gi}: {names.get(what, 'the free list and the holders disagree')}")
