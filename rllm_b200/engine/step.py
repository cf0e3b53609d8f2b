"""The step function: one batch of (request, its next tokens) through the model.

A step runs exactly the tokens it is given, as one batch, against what earlier steps
left in the cache, and returns float32 logits at the wanted places. Prompt portions of
any length stand beside single decoded tokens; a request may skip steps. Nothing here
samples or schedules: the scheduler, `generate()` and the trace replay all drive this
one function.

The reference runs one forward per prefilling sequence and a separate batched decode
(src/engine/mod.rs:485-714); here they are one call, and a later portion of a prompt
attends the keys of the earlier ones through the block table.

Steps that bring exactly one token per request (decoding) replay a CUDA graph of the
same launches (see `graphs.py`) when every part of the model allows it; the kernels and
the cache are the same either way.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from .context import GroupView, StepContext


_log = logging.getLogger("rllm_b200")


@dataclass
class Entry:
    """One request's share of a step: its next `tokens`, and `want`, the indices among
    these tokens whose logits are asked for (may be empty)."""
    request_id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class StepError(ValueError):
    pass


class MetaLayout:
    """Where each vector of a step's metadata lies in the one int32 buffer that is copied
    to the device: ids | positions | token_seq | cu_q | kv_lens | state_slots | rows |
    per cache group: slots[T], block_table[S * P]. Every vector starts on a 16-byte
    boundary."""

    def __init__(self, T: int, S: int, P: int, n_rows: int, G: int):
        self.T, self.S, self.P, self.n_rows, self.G = T, S, P, n_rows, G
        sizes = [T, T, T, S + 1, S, S, max(n_rows, 1)] + [T, S * P] * G
        self.offs = np.concatenate([[0], np.cumsum([(n + 3) // 4 * 4 for n in sizes])]).astype(np.int64)
        self.total = int(self.offs[-1])

    def view(self, buf, i: int, n: int):
        o = int(self.offs[i])
        return buf[o: o + n]


class Engine:
    def __init__(self, model, backend, cache: CacheManager, use_graphs: bool | None = None):
        self.model, self.backend, self.cache = model, backend, cache
        self.device = backend.device
        self.vocab = model.vocab_size
        # device words: [0] a kernel's bounded wait ran out, [1] a token id outside the table,
        # [2] checked runs: a page number or cache slot outside the pool, [3] spare
        if backend.fast:
            from ..kernels import sm100
            self.error_words = sm100.init(self.device).err
        else:
            self.error_words = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._err_flag = self.error_words[1:2]
        # RLLM_B200_CHECKED=1: every step's block tables and slots are tested on the device before
        # the model's kernels read them (one small kernel per cache group, also inside graphs)
        self.checked = os.environ.get("RLLM_B200_CHECKED") == "1"
        self.steps_run = 0
        self.graph_steps = 0
        self.h2d_bytes = 0            # bytes of step metadata copied to the device so far
        self._opened: list = []
        if use_graphs is None:
            use_graphs = os.environ.get("RLLM_B200_NO_GRAPHS") != "1"
        self.graphs = None
        if use_graphs and hasattr(model, "parts"):
            unsafe = sorted({type(p).__name__ for p in model.parts() if not getattr(p, "graph_safe", False)})
            if unsafe:
                # said once, when the engine is made: a part that reads the step on the host keeps the
                # whole model's decode steps out of CUDA graphs (they then run launch by launch)
                _log.warning("decode steps run without CUDA graphs: part(s) %s do not declare graph_safe",
                             ", ".join(unsafe))
            else:
                from .graphs import DecodeGraphs
                self.graphs = DecodeGraphs(self)

    # ------------------------------------------------------------------ requests
    def has(self, request_id) -> bool:
        return request_id in self.cache.live

    def num_tokens(self, request_id) -> int:
        return self.cache.live[request_id].num_tokens

    def end(self, request_ids) -> None:
        """The requests are finished: everything they hold is given back."""
        for rid in request_ids:
            if rid in self.cache.live:
                self.cache.close(rid)

    def check(self) -> None:
        """Read the device error words (one small copy): a token id outside the table, or a
        kernel whose bounded wait ran out. Callers that read results back anyway call this at
        the same time."""
        wait, token, page = self.error_words.tolist()[:3]
        if token:
            self._err_flag.zero_()
            raise StepError("a token id outside the embedding table reached the device")
        if page:
            self.error_words[2:3].zero_()
            what = f"slot of token {page & 0x3fffffff}" if page & 0x40000000 else f"block-table entry {page - 1}"
            raise StepError(f"checked run: a {what} named a page outside the pool (the access was skipped)")
        if wait and self.backend.fast:
            from ..kernels import sm100
            sm100.check_error(self.device)

    # ------------------------------------------------------------------ the step
    def _validate(self, entries: list[Entry]) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab:
                raise StepError(f"request {e.request_id!r}: token id outside [0, {self.vocab})")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} outside its "
                                    f"{len(e.tokens)} tokens")

    def prepare(self, entries: list[Entry]):
        """Reserve pages for every entry (all or nothing). Returns the requests' holdings; the ids
        of the requests this call opened are kept in `self._opened` until the step has run."""
        self._validate(entries)
        cache = self.cache
        opened, reserved = [], []
        try:
            rcs = []
            for e in entries:
                rc = cache.live.get(e.request_id)
                if rc is None:
                    rc = cache.open(e.request_id)
                    opened.append(e.request_id)
                cache.reserve(rc, rc.num_tokens + len(e.tokens))
                reserved.append(rc)
                rcs.append(rc)
        except OutOfPages:
            self._undo(reserved, opened)
            raise
        self._opened = opened
        return rcs

    def _undo(self, reserved, opened) -> None:
        """A step that did not run to its end leaves every request as it was: reservations are
        given back, requests it opened are closed."""
        for rc in reserved:
            if rc.handle >= 0:
                self.cache.trim(rc)
        for rid in opened:
            if rid in self.cache.live:
                self.cache.close(rid)

    def fill_meta(self, host: np.ndarray, lay: MetaLayout, entries: list[Entry], rcs) -> None:
        """Write the step's metadata into `host` (int32, `lay.total` long, preset to -1)."""
        ps = self.cache.page_size
        T, S, P, G = lay.T, lay.S, lay.P, lay.G
        ids, pos, tseq = lay.view(host, 0, T), lay.view(host, 1, T), lay.view(host, 2, T)
        cu, kvl, sslot = lay.view(host, 3, S + 1), lay.view(host, 4, S), lay.view(host, 5, S)
        rows = lay.view(host, 6, max(lay.n_rows, 1))
        r = q0 = 0
        cu[0] = 0
        for s, (e, rc) in enumerate(zip(entries, rcs)):
            q = len(e.tokens)
            start = rc.num_tokens
            ids[q0:q0 + q] = e.tokens
            pos[q0:q0 + q] = np.arange(start, start + q, dtype=np.int32)
            tseq[q0:q0 + q] = s
            cu[s + 1] = q0 + q
            kvl[s] = start + q
            sslot[s] = rc.state_slot
            for w in e.want:
                rows[r] = q0 + w
                r += 1
            for g in range(G):
                pages = rc.pages_array(g)
                o = int(lay.offs[8 + 2 * g]) + s * P
                host[o: o + len(pages)] = pages
                p = pos[q0:q0 + q]
                o = int(lay.offs[7 + 2 * g]) + q0
                host[o: o + q] = pages[p // ps] * ps + p % ps
            q0 += q
        if lay.n_rows == 0:
            rows[0] = 0

    def make_context(self, dev: torch.Tensor, lay: MetaLayout, q_lens, kv_lens, starts,
                     state_slots) -> tuple[StepContext, torch.Tensor]:
        """The step context over the device copy `dev` of a metadata buffer."""
        T, S, P = lay.T, lay.S, lay.P
        ps = self.cache.page_size
        groups = {g: GroupView(lay.view(dev, 7 + 2 * g, T), lay.view(dev, 8 + 2 * g, S * P).view(S, P), ps)
                  for g in range(lay.G)}
        ctx = StepContext(
            backend=self.backend, num_tokens=T, num_seqs=S, token_ids=lay.view(dev, 0, T),
            positions=lay.view(dev, 1, T), token_seq=lay.view(dev, 2, T), cu_q=lay.view(dev, 3, S + 1),
            kv_lens=lay.view(dev, 4, S), state_slots=lay.view(dev, 5, S), q_lens_host=list(q_lens),
            kv_lens_host=list(kv_lens), state_slots_host=list(state_slots), groups=groups,
            max_q_len=max(q_lens), max_kv_len=max(kv_lens))
        ctx.extras["err_flag"] = self._err_flag
        ctx.extras["starts_host"] = list(starts)
        return ctx, lay.view(dev, 6, lay.n_rows)

    def check_meta(self, ctx: StepContext) -> None:
        """Checked runs: test (and make harmless) the step's tables and slots, group by group."""
        if not self.checked:
            return
        from ..kernels import ops
        for gi, view in ctx.groups.items():
            ops.check_meta(view.block_table, view.slots, self.cache.groups[gi].pool.num_pages, view.page_size,
                           self.error_words[2:3])

    def build_context(self, entries: list[Entry], rcs) -> tuple[StepContext, torch.Tensor]:
        G = len(self.cache.groups)
        q_lens = [len(e.tokens) for e in entries]
        starts = [rc.num_tokens for rc in rcs]
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        P = max(1, max((rc.num_held(g) for rc in rcs for g in range(G)), default=1))
        lay = MetaLayout(sum(q_lens), len(entries), P, sum(len(e.want) for e in entries), G)
        host = torch.full((lay.total,), -1, dtype=torch.int32).pin_memory()
        self.fill_meta(host.numpy(), lay, entries, rcs)
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes += 4 * lay.total
        return self.make_context(dev, lay, q_lens, kv_lens, starts, [rc.state_slot for rc in rcs])

    def takes_feed(self, entries: list[Entry]) -> bool:
        """Can this batch take its token ids from the device (`step(..., feed=)`)? Only steps that
        replay a graph read their metadata from a buffer that outlives the call."""
        return self.graphs is not None and all(e.request_id in self.cache.live for e in entries) \
            and self.graphs.takes(entries, [self.cache.live[e.request_id] for e in entries])

    def step(self, entries: list[Entry], keep: bool = True, feed: torch.Tensor | None = None) -> torch.Tensor | None:
        """Run one batch; returns float32 logits [wanted places, vocab] on the device, in
        the order of the entries and of each `want` (None if nothing is wanted).
        Raises OutOfPages if the pages do not suffice; that, or any other error raised while the
        batch runs, leaves every request as it was (nothing committed, reservations given back).
        `keep=False`: the caller reads the logits before the next step, so they may live
        in a buffer that the next step overwrites (saves a copy).
        `feed`: the entries' token ids as an int32 tensor on the device, one per entry (see
        `takes_feed`); the ids in `entries` are placeholders then."""
        if feed is not None and not self.takes_feed(entries):
            raise StepError("token ids can be fed from the device only to a step that replays a graph")
        rcs = self.prepare(entries)
        logits = None
        try:
            if self.graphs is not None and self.graphs.takes(entries, rcs):
                logits = self.graphs.run(entries, rcs, keep, feed)
                self.graph_steps += 1
            else:
                ctx, rows = self.build_context(entries, rcs)
                self.check_meta(ctx)
                h = self.model.forward(ctx, self.cache)
                if rows.numel():
                    logits = self.model.logits(h, rows, ctx)
        except BaseException:
            # a refused size, a failed launch or capture: nothing is committed, the pages go back
            self._undo(rcs, self._opened)
            raise
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.num_tokens + len(e.tokens))
        self.steps_run += 1
        return logits
