"""CUDA graphs for decode steps.

A step that brings one token per request launches some nine kernels per layer, each a few
microseconds long; issued one by one from the host they cost more than they run. Such a
step is therefore captured once per shape and replayed: the same kernels, on the same cache,
reading the step's metadata (token ids, positions, slots, block tables, key counts) from a
device buffer at a fixed address that is refilled before every replay.

A graph is keyed by (rows, block-table width). The width is the pages of the longest request
rounded up to a power of two, so that a request growing by a token a step meets a new graph
only when its length doubles. The rows are the number of requests rounded up to a size from a
short list (every size up to 8, then steps of 4, 8 and 16): a capture costs about thirty
replays, and a batch that shrinks request by request would otherwise meet a new graph at every
step. Rows beyond the requests are stand-ins: one token at position 0 that sees one key (the
first of page 0, whatever it holds) and writes none; their logits are not returned. Everything
a kernel's launch shape depends on (grid sizes, how many ranges the keys are cut into) follows
from the key; what differs from step to step is read on the device.

Only models whose parts all declare `graph_safe` (they read nothing of the step on the
host) are captured; any other model runs launch by launch.
"""
from __future__ import annotations

import gc
import weakref
from collections import OrderedDict

import numpy as np
import torch

from ..kernels import ops

MAX_GRAPH_BATCH = 256
MAX_GRAPHS = 48


def padded_rows(S: int) -> int:
    """The graph size that serves S requests."""
    if S <= 8:
        return S
    step = 4 if S <= 32 else 8 if S <= 64 else 16
    return (S + step - 1) // step * step


class _Slot:
    __slots__ = ("lay", "host", "dev", "ctx", "rows", "graph", "logits", "copied", "launches", "head", "handles", "tokens", "rows_state",
                 "live", "_lib")

    def __del__(self):
        rs, L = getattr(self, "rows_state", None), getattr(self, "_lib", None)
        if rs and L is not None:
            L.rows_delete(rs)


class DecodeGraphs:
    def __init__(self, engine):
        self._engine = weakref.ref(engine)      # the engine owns this object, not the reverse
        self.slots: OrderedDict[tuple[int, int], _Slot] = OrderedDict()
        self.pool = None
        self.captures = 0

    @property
    def engine(self):
        return self._engine()

    def _width(self, rcs) -> int:
        G = len(self.engine.cache.groups)
        need = max((rc.num_held(g) for rc in rcs for g in range(G)), default=1)
        p = 8
        while p < need:
            p *= 2
        return p

    def takes(self, entries, rcs) -> bool:
        return len(entries) <= MAX_GRAPH_BATCH and all(len(e.tokens) == 1 and len(e.want) <= 1
                                                       for e in entries)

    def _forward(self, slot: _Slot) -> torch.Tensor:
        eng = self.engine
        eng.check_meta(slot.ctx)
        h = eng.model.forward(slot.ctx, eng.cache)
        return eng.model.logits(h, slot.rows, slot.ctx)

    def _new_slot(self, S: int, P: int) -> _Slot:
        from .step import MetaLayout
        eng = self.engine
        slot = _Slot()
        slot.lay = lay = MetaLayout(S, S, P, S, len(eng.cache.groups))
        slot.host = torch.full((lay.total,), -1, dtype=torch.int32).pin_memory()
        slot.dev = torch.full((lay.total,), -1, dtype=torch.int32, device=eng.device)
        cap = P * eng.cache.page_size           # upper bound of every request's key count
        slot.ctx, slot.rows = eng.make_context(slot.dev, lay, [1] * S, [cap] * S, [cap - 1] * S, [-1] * S)
        slot.ctx.graph_safe = True
        slot.ctx.kv_lens_host = slot.ctx.state_slots_host = None     # not known when replayed
        slot.ctx.extras.pop("starts_host", None)
        slot.graph = slot.logits = None
        slot.copied = torch.cuda.Event()
        # the native writer remembers what the host buffer's block-table rows hold: a row is
        # rewritten only when another holding takes it or its pages changed other than by growing
        slot._lib = eng.cache._L
        slot.rows_state = slot._lib.rows_new(S, len(eng.cache.groups))
        slot.handles = np.zeros(S, dtype=np.int32)
        slot.tokens = np.zeros(S, dtype=np.int32)
        slot.head = int(lay.offs[8]) if len(eng.cache.groups) == 1 else lay.total   # ints before the first table
        slot.live = S                                                   # rows that held requests in the last step
        host = slot.host.numpy()
        lay.view(host, 2, S)[:] = np.arange(S, dtype=np.int32)          # token s belongs to sequence s
        lay.view(host, 3, S + 1)[:] = np.arange(S + 1, dtype=np.int32)  # one row each
        lay.view(host, 6, S)[:] = np.arange(S, dtype=np.int32)          # logits of every row
        return slot

    def _capture(self, slot: _Slot) -> None:
        # once launch by launch (this also sets every kernel's attributes), then captured
        cur = torch.cuda.current_stream(self.engine.device)
        side = torch.cuda.Stream(self.engine.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            self._forward(slot)
        cur.wait_stream(side)
        torch.cuda.synchronize(self.engine.device)
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        # Nothing may be destroyed while the capture runs: a dead cycle that holds another
        # engine's graphs or pinned buffers, collected in the middle of it, invalidates it.
        # So the collector is off meanwhile (a collection beforehand would cost as much as the
        # capture itself).
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, pool=self.pool):
                slot.logits = self._forward(slot)
        finally:
            if gc_was_on:
                gc.enable()
        slot.launches = ops.LAUNCHES - before    # kernels one replay launches
        ops.LAUNCHES = before                    # a capture launches nothing
        slot.graph = graph
        self.captures += 1

    def _fill(self, slot: _Slot, entries, rcs) -> bool:
        """The step's metadata into the slot's host buffer (the native writer: the vectors of S
        numbers each step, a block-table row only where it changed). Returns whether a table row
        was touched."""
        cache = self.engine.cache
        S, lay = len(entries), slot.lay
        slot.handles[:S] = [rc.handle for rc in rcs]
        slot.tokens[:S] = [e.tokens[0] for e in entries]
        rc = cache._L.fill_decode(cache._ptr, slot.rows_state, S, slot.handles.ctypes.data, slot.tokens.ctypes.data,
                                  lay.P, slot.host.data_ptr(), lay.offs.ctypes.data)
        if rc < 0:
            raise RuntimeError(f"decode metadata could not be written (code {rc})")
        dirty = rc > 0
        if S != slot.live:
            # rows S.. stand in for requests that are not there: token 0 at position 0, one key
            # (page 0, offset 0), nothing written, no state
            host = slot.host.numpy()
            for i, v in ((0, 0), (1, 0), (4, 1), (5, -1)):
                lay.view(host, i, lay.S)[S:] = v
            for g in range(lay.G):
                lay.view(host, 7 + 2 * g, lay.S)[S:] = -1
                table = lay.view(host, 8 + 2 * g, lay.S * lay.P).reshape(lay.S, lay.P)
                table[S:] = -1
                table[S:, 0] = 0
            cache._L.rows_forget(slot.rows_state, S)
            slot.live = S
            dirty = True
        return dirty

    def run(self, entries, rcs, keep: bool = True, feed: torch.Tensor | None = None) -> torch.Tensor | None:
        """Replay the graph of this shape. `feed`: int32 [S] on the device, the entries' token ids
        (those in `entries` are then placeholders): the step can be launched before the host has
        seen the tokens that the step before it drew."""
        eng = self.engine
        S = len(entries)
        key = (padded_rows(S), self._width(rcs))
        slot = self.slots.get(key)
        if slot is None:
            slot = self._new_slot(*key)
            self.slots[key] = slot
            while len(self.slots) > MAX_GRAPHS:
                self.slots.popitem(last=False)
        else:
            self.slots.move_to_end(key)
        slot.copied.synchronize()               # the last copy out of the host buffer is over
        dirty = self._fill(slot, entries, rcs)
        # one small kernel reads the words out of the pinned buffer (all of them if a block table
        # changed, else the vectors in front) and takes the token ids from `feed` if that is given
        n = slot.lay.total if dirty else slot.head
        ops.step_meta(slot.host, slot.dev, n, feed)
        eng.h2d_bytes += 4 * n
        slot.copied.record()
        if slot.graph is None:
            self._capture(slot)
        slot.graph.replay()
        ops.LAUNCHES += slot.launches
        wanted = [s for s, e in enumerate(entries) if e.want]
        if not wanted:
            return None
        if len(wanted) == S:
            return slot.logits[:S].clone() if keep else slot.logits[:S]
        idx = torch.tensor(wanted, dtype=torch.int32).to(eng.device)
        return ops.gather_rows(slot.logits, idx)
