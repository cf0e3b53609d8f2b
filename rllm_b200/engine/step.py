"""The step function: one batch of (request, its next tokens) through the model.

A step runs exactly the tokens it is given, as one batch, against what earlier steps
left in the cache, and returns float32 logits at the wanted places. Prompt portions of
any length stand beside single decoded tokens; a request may skip steps. Nothing here
samples or schedules: the scheduler, `generate()` and the trace replay all drive this
one function.

The reference runs one forward per prefilling sequence and a separate batched decode
(src/engine/mod.rs:485-714); here they are one call, and a later portion of a prompt
attends the keys of the earlier ones through the block table.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from .context import GroupView, StepContext


@dataclass
class Entry:
    """One request's share of a step: its next `tokens`, and `want`, the indices among
    these tokens whose logits are asked for (may be empty)."""
    request_id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class StepError(ValueError):
    pass


class Engine:
    def __init__(self, model, backend, cache: CacheManager):
        self.model, self.backend, self.cache = model, backend, cache
        self.device = backend.device
        self.vocab = model.vocab_size
        self._err_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps_run = 0

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
        if int(self._err_flag.item()):
            self._err_flag.zero_()
            raise StepError("a token id outside the embedding table reached the device")
        if self.backend.fast:
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
        """Reserve pages for every entry (all or nothing) and build the step's metadata."""
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
            for rc in reserved:
                cache.trim(rc)
            for rid in opened:
                cache.close(rid)
            raise
        return rcs

    def build_context(self, entries: list[Entry], rcs) -> tuple[StepContext, torch.Tensor]:
        cache, ps = self.cache, self.cache.page_size
        S = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        starts = [rc.num_tokens for rc in rcs]
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        G = len(cache.groups)
        P = max(1, max((len(rc.pages[g]) for rc in rcs for g in range(G)), default=1))
        n_rows = sum(len(e.want) for e in entries)

        # one int32 buffer: ids | positions | token_seq | cu_q | kv_lens | state_slots | rows |
        #                   per group: slots[T], block_table[S*P]
        sizes = [T, T, T, S + 1, S, S, max(n_rows, 1)] + [T, S * P] * G
        offs = np.concatenate([[0], np.cumsum([(n + 3) // 4 * 4 for n in sizes])]).astype(np.int64)
        host = np.full(int(offs[-1]), -1, dtype=np.int32)
        ids = host[offs[0]:offs[0] + T]
        pos = host[offs[1]:offs[1] + T]
        tseq = host[offs[2]:offs[2] + T]
        cu = host[offs[3]:offs[3] + S + 1]
        kvl = host[offs[4]:offs[4] + S]
        sslot = host[offs[5]:offs[5] + S]
        rows = host[offs[6]:offs[6] + max(n_rows, 1)]
        r = 0
        q0 = 0
        cu[0] = 0
        for s, (e, rc) in enumerate(zip(entries, rcs)):
            q = q_lens[s]
            ids[q0:q0 + q] = e.tokens
            pos[q0:q0 + q] = np.arange(starts[s], starts[s] + q, dtype=np.int32)
            tseq[q0:q0 + q] = s
            cu[s + 1] = q0 + q
            kvl[s] = kv_lens[s]
            sslot[s] = rc.state_slot
            for w in e.want:
                rows[r] = q0 + w
                r += 1
            for g in range(G):
                pages = np.asarray(rc.pages[g], dtype=np.int32)
                bt = host[offs[8 + 2 * g] + s * P: offs[8 + 2 * g] + s * P + len(pages)]
                bt[:] = pages
                p = pos[q0:q0 + q]
                host[offs[7 + 2 * g] + q0: offs[7 + 2 * g] + q0 + q] = pages[p // ps] * ps + p % ps
            q0 += q
        if n_rows == 0:
            rows[0] = 0
        dev = torch.from_numpy(host).pin_memory().to(self.device, non_blocking=True)

        def view(i, n):
            return dev[int(offs[i]): int(offs[i]) + n]

        groups = {g: GroupView(view(7 + 2 * g, T), view(8 + 2 * g, S * P).view(S, P), ps)
                  for g in range(G)}
        ctx = StepContext(
            backend=self.backend, num_tokens=T, num_seqs=S, token_ids=view(0, T),
            positions=view(1, T), token_seq=view(2, T), cu_q=view(3, S + 1), kv_lens=view(4, S),
            state_slots=view(5, S), q_lens_host=q_lens, kv_lens_host=kv_lens,
            state_slots_host=[rc.state_slot for rc in rcs], groups=groups,
            max_q_len=max(q_lens), max_kv_len=max(kv_lens))
        ctx.extras["err_flag"] = self._err_flag
        ctx.extras["starts_host"] = starts
        return ctx, view(6, n_rows)

    def step(self, entries: list[Entry]) -> torch.Tensor | None:
        """Run one batch; returns float32 logits [wanted places, vocab] on the device, in
        the order of the entries and of each `want` (None if nothing is wanted).
        Raises OutOfPages, leaving every request as it was, if the pages do not suffice."""
        rcs = self.prepare(entries)
        ctx, rows = self.build_context(entries, rcs)
        h = self.model.forward(ctx, self.cache)
        logits = self.model.logits(h, rows, ctx) if rows.numel() else None
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.num_tokens + len(e.tokens))
        self.steps_run += 1
        return logits
