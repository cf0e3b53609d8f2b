"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees; and decides what happens when pages run out.

Decisions per step, in this order:
  1. every request that is decoding gets its one token (oldest admission first);
  2. requests whose prompt is not yet stored get a portion of it, as large as the rest of
     the budget and `max_chunk` allow (a portion may be cut anywhere);
  3. waiting requests are admitted first-come-first-served while a place (`max_active`),
     budget and pages for their first portion are left; the head of the line is never
     overtaken (the reference's rule, src/engine/mod.rs:273-312).
Pages are counted per cache group before anything runs, so the step function never fails
half-way. When a running request cannot get the pages it needs, the most recently admitted
running request is preempted: its pages are given back, and it returns to the FRONT of the
waiting line with prompt + generated tokens as its new prompt (recompute), keeping its
generated tokens and its random-number counter, so its output is unchanged (the reference
preempts only when nothing could be admitted and drops the seed, src/engine/mod.rs:367-427).
A request that cannot fit even when it has the pool to itself finishes with reason
"out_of_pages" instead of blocking the line.

The scheduler needs only a `CacheManager` (for counting) and an `executor` with
`step(entries) -> logits` and `end(ids)`: tests drive it with a fake executor on the CPU.
"""
from __future__ import annotations

import itertools
import random
from collections import deque
from dataclasses import dataclass, field

from ..cache import CacheManager, pages_for
from ..sampling import SamplingParams
from .step import Entry


@dataclass
class Request:
    request_id: int
    prompt: list[int]
    params: SamplingParams
    seed: int
    output: list[int] = field(default_factory=list)
    # with params.logprobs: (ln p of the token, [(token, ln p) of the most probable ones]) per output token
    logprobs: list[tuple[float, list[tuple[int, float]]]] = field(default_factory=list)
    # tokens to store before the next sample: prompt (+ output after a preemption)
    pending: list[int] = field(default_factory=list)
    num_stored: int = 0          # tokens whose keys/values are in the cache
    admitted_at: int = -1
    finished: bool = False
    finish_reason: str | None = None
    preemptions: int = 0

    @property
    def decoding(self) -> bool:
        return not self.pending and bool(self.output)


@dataclass
class Planned:
    request: Request
    tokens: list[int]
    samples: bool       # the step's logits for this request's last token are sampled
    need: list[int] = field(default_factory=list)   # pages per group this step adds


@dataclass
class StepOutput:
    request_id: int
    token: int | None
    finished: bool
    finish_reason: str | None = None
    logprob: float | None = None                          # with params.logprobs
    top_logprobs: list[tuple[int, float]] | None = None


class Scheduler:
    def __init__(self, cache: CacheManager, max_active: int = 64, max_tokens_per_step: int = 2048,
                 max_chunk: int | None = None):
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be >= 1")
        self.cache = cache
        self.max_active = max_active
        self.max_tokens_per_step = max_tokens_per_step
        self.max_chunk = max_chunk or max_tokens_per_step
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in admission order
        self.requests: dict[int, Request] = {}
        self._ids = itertools.count()
        self._admissions = itertools.count()
        self.preempted_total = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: list[int], params: SamplingParams | None = None) -> int:
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        params = params or SamplingParams()
        rid = next(self._ids)
        seed = params.seed if params.seed is not None else random.getrandbits(63)
        req = Request(rid, list(prompt), params, seed, pending=list(prompt))
        self.requests[rid] = req
        self.waiting.append(req)
        return rid

    def abort(self, request_id: int, executor=None) -> bool:
        """Remove a request wherever it is; its pages return at once
        (src/engine/mod.rs:316-321)."""
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return False
        if req in self.running:
            self.running.remove(req)
            self._release(req, executor)
        else:
            self.waiting.remove(req)
        req.finished, req.finish_reason = True, "aborted"
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ page counting
    def _need(self, req: Request, n_new: int) -> list[int]:
        rc = self.cache.live.get(req.request_id)
        total = pages_for(req.num_stored + n_new, self.cache.page_size)
        return [max(0, total - (rc.num_held(g) if rc else 0)) for g in range(len(self.cache.groups))]

    def _held(self, req: Request) -> list[int]:
        rc = self.cache.live.get(req.request_id)
        if rc is None:
            return [0] * len(self.cache.groups)
        return self.cache.held_pages(rc)

    def _release(self, req: Request, executor) -> None:
        if req.request_id in self.cache.live:
            if executor is not None:
                executor.end([req.request_id])
            else:
                self.cache.close(req.request_id)

    def _preempt(self, victim: Request, executor) -> None:
        self.running.remove(victim)
        self._release(victim, executor)
        victim.pending = victim.prompt + victim.output
        victim.num_stored = 0
        victim.preemptions += 1
        self.preempted_total += 1
        self.waiting.appendleft(victim)

    def _finish(self, req: Request, reason: str, executor) -> None:
        req.finished, req.finish_reason = True, reason
        if req in self.running:
            self.running.remove(req)
        self._release(req, executor)

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self, executor=None) -> tuple[list[Planned], list[StepOutput]]:
        """What runs in the next step, and which requests ended without running."""
        plan: list[Planned] = []
        failed: list[StepOutput] = []
        budget = self.max_tokens_per_step
        free = list(self.cache.free_pages())
        # The steady state of serving: nobody waits, everybody decodes, and even if every request
        # needed a new page in every group the pools would have them. Same plan as the general
        # rules below give, without counting pages request by request.
        if not self.waiting and self.running and len(self.running) <= budget \
                and all(f >= len(self.running) for f in free) and all(r.decoding for r in self.running):
            return [Planned(r, [r.output[-1]], True) for r in self.running], failed
        pool = [g.pool.num_pages for g in self.cache.groups]

        def fits(need):
            return all(n <= f for n, f in zip(need, free))

        order = [r for r in self.running if r.decoding] + [r for r in self.running if not r.decoding]
        for req in order:
            if req not in self.running:        # preempted while placing an earlier one
                continue
            n = 1 if req.decoding else min(len(req.pending), budget, self.max_chunk)
            if n <= 0:
                continue
            if req.decoding and budget <= 0:
                continue
            need = self._need(req, n)
            while not fits(need):
                victim = self.running[-1]
                if victim is req and len(self.running) == 1:
                    break
                held = self._held(victim)
                self._preempt(victim, executor)
                free = [f + h for f, h in zip(free, held)]
                for i, p in enumerate(plan):
                    if p.request is victim:      # it was already placed in this step
                        budget += len(p.tokens)
                        free = [f + x for f, x in zip(free, p.need)]
                        del plan[i]
                        break
                if victim is req:
                    break
            if req not in self.running:
                continue
            if not fits(need):
                # alone and still too large for the whole pool
                self._finish(req, "out_of_pages", executor)
                failed.append(StepOutput(req.request_id, None, True, "out_of_pages"))
                free = list(self.cache.free_pages())
                continue
            toks = [req.output[-1]] if req.decoding else req.pending[:n]
            p = Planned(req, toks, req.decoding or n == len(req.pending), need)
            plan.append(p)
            free = [f - x for f, x in zip(free, need)]
            budget -= n

        while self.waiting and len(self.running) < self.max_active and budget > 0:
            req = self.waiting[0]
            total_pages = pages_for(len(req.pending) + 1, self.cache.page_size)
            if any(total_pages > p for p in pool):
                self.waiting.popleft()
                req.finished, req.finish_reason = True, "out_of_pages"
                failed.append(StepOutput(req.request_id, None, True, "out_of_pages"))
                continue
            if len(self.cache.live) >= self.cache.max_requests:
                break
            n = min(len(req.pending), budget, self.max_chunk)
            need = self._need(req, n)
            if not fits(need):
                break                           # the head of the line waits; nobody overtakes
            self.waiting.popleft()
            req.admitted_at = next(self._admissions)
            self.running.append(req)
            p = Planned(req, req.pending[:n], n == len(req.pending), need)
            plan.append(p)
            free = [f - x for f, x in zip(free, need)]
            budget -= n
        return plan, failed

    # ------------------------------------------------------------------ after the step ran
    def plan_ahead(self, plan: list[Planned]) -> list[Planned] | None:
        """The plan of the step after `plan`, made before `plan`'s tokens are known, or None if
        that cannot be told yet. It can when `plan` is the steady state (nobody waits, everybody
        decodes and is sampled), the next step is too unless a request meets its end-of-sequence
        token, and nothing about a request's next step hangs on the token it is about to get: no
        request reaches its token limit, none is penalised for tokens it has produced. The tokens
        of the returned plan are placeholders; a request that did end in `plan` is passed over
        when the step ahead is recorded (`advance`), its extra token dropped."""
        if self.waiting or not plan or len(plan) != len(self.running) or len(plan) > self.max_tokens_per_step:
            return None
        for p, r in zip(plan, self.running):
            if p.request is not r or not p.samples or len(p.tokens) != 1 or r.pending or r.finished:
                return None
            if len(r.output) + 2 > r.params.max_tokens or r.params.has_penalties:
                return None                      # it ends with the coming token, or its draw needs the history
        if not all(f >= len(plan) for f in self.cache.free_pages()):
            return None
        return [Planned(r, [0], True) for r in self.running]

    def advance(self, plan: list[Planned], tokens: list[int], executor=None,
                logprobs: dict | None = None) -> list[StepOutput]:
        """Record what the step stored and sampled; finish and free what is done. `tokens`
        are the sampled tokens of the planned requests with `samples`, in plan order;
        `logprobs` maps an index into `tokens` to (ln p, [(token, ln p), ...]) for the requests
        that asked for them."""
        outs, it = [], iter(tokens)
        nth = -1
        for p in plan:
            req = p.request
            nth += p.samples
            if req.finished:                     # ended (or aborted) while this step was under way
                if p.samples:
                    next(it)
                continue
            req.num_stored += len(p.tokens)
            if not req.decoding:
                req.pending = req.pending[len(p.tokens):]
            if not p.samples:
                continue
            tok = int(next(it))
            req.output.append(tok)
            reason = None
            if not req.params.ignore_eos and tok in req.params.eos_token_ids:
                reason = "eos"
            elif len(req.output) >= req.params.max_tokens:
                reason = "max_tokens"
            if reason:
                self._finish(req, reason, executor)
            lp = logprobs.get(nth) if logprobs else None
            if lp is not None:
                req.logprobs.append(lp)
            outs.append(StepOutput(req.request_id, tok, reason is not None, reason,
                                   lp[0] if lp else None, lp[1] if lp else None))
        return outs

    def entries(self, plan: list[Planned]) -> list[Entry]:
        return [Entry(p.request.request_id, p.tokens, [len(p.tokens) - 1] if p.samples else [])
                for p in plan]
