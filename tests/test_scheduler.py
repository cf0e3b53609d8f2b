"""The scheduler's decisions, on the CPU with a fake executor (in the manner of the
reference's MockDispatch tests, src/engine/mod.rs:1231-1310)."""
import pytest
import torch

from rllm_b200.cache import CacheManager
from rllm_b200.engine.scheduler import Scheduler
from rllm_b200.parts.base import KVCacheSpec
from rllm_b200.sampling import SamplingParams


class FakeExecutor:
    """Reserves and commits pages like the real step function; 'samples' a counter."""

    def __init__(self, cache):
        self.cache, self.batches = cache, []

    def step(self, entries):
        rcs = []
        for e in entries:
            rc = self.cache.live.get(e.request_id) or self.cache.open(e.request_id)
            self.cache.reserve(rc, rc.num_tokens + len(e.tokens))
            rcs.append(rc)
        for e, rc in zip(entries, rcs):
            self.cache.commit(rc, rc.num_tokens + len(e.tokens))
        self.batches.append([(e.request_id, list(e.tokens), list(e.want)) for e in entries])
        self.cache.check()

    def end(self, ids):
        for i in ids:
            self.cache.close(i)


def make(pages=64, page=4, **kw):
    cache = CacheManager([KVCacheSpec(1, 16)], page, pages, 16, torch.float32, "cpu", allocate=False)
    return Scheduler(cache, **kw), FakeExecutor(cache)


def run_step(s, ex, token_of=lambda req: 1000 + len(req.output)):
    plan, failed = s.schedule(ex)
    if plan:
        ex.step(s.entries(plan))
    toks = [token_of(p.request) for p in plan if p.samples]
    return plan, failed + s.advance(plan, toks, ex)


def test_fcfs_admission_and_max_active():
    s, ex = make(max_active=2, max_tokens_per_step=100)
    ids = [s.add_request([1, 2, 3], SamplingParams(max_tokens=2)) for _ in range(3)]
    plan, _ = run_step(s, ex)
    assert [p.request.request_id for p in plan] == ids[:2]
    assert len(s.waiting) == 1
    plan, outs = run_step(s, ex)       # both decode one token and finish (max_tokens 2)
    assert all(o.finished and o.finish_reason == "max_tokens" for o in outs)
    plan, _ = run_step(s, ex)
    assert [p.request.request_id for p in plan] == [ids[2]]


def test_budget_cuts_prompts_into_portions_and_decodes_first():
    s, ex = make(max_tokens_per_step=8)
    a = s.add_request(list(range(5)), SamplingParams(max_tokens=4))
    run_step(s, ex)                                   # a's prompt, first token
    b = s.add_request(list(range(20)), SamplingParams(max_tokens=4))
    plan, _ = run_step(s, ex)
    assert [(p.request.request_id, len(p.tokens), p.samples) for p in plan] == [(a, 1, True), (b, 7, False)]
    plan, _ = run_step(s, ex)
    assert [(p.request.request_id, len(p.tokens), p.samples) for p in plan] == [(a, 1, True), (b, 7, False)]
    plan, outs = run_step(s, ex)                      # a samples its 4th token and finishes
    assert [(p.request.request_id, len(p.tokens), p.samples) for p in plan] == [(a, 1, True), (b, 6, True)]
    assert [o.request_id for o in outs if o.finished] == [a]
    # only the last portion of a prompt asks for logits
    assert ex.batches[-1][1][2] == [5] and ex.batches[-2][1][2] == []
    plan, _ = run_step(s, ex)
    assert [(p.request.request_id, len(p.tokens)) for p in plan] == [(b, 1)]


def test_max_chunk_limits_a_portion():
    s, ex = make(max_tokens_per_step=64, max_chunk=5)
    s.add_request(list(range(12)), SamplingParams(max_tokens=1))
    sizes = []
    while s.has_work():
        plan, _ = run_step(s, ex)
        sizes += [len(p.tokens) for p in plan]
    assert sizes == [5, 5, 2]


def test_head_of_line_blocks_when_pages_lack():
    s, ex = make(pages=6, page=4, max_tokens_per_step=100)
    a = s.add_request(list(range(14)), SamplingParams(max_tokens=3))   # 4 pages
    b = s.add_request(list(range(12)), SamplingParams(max_tokens=3))   # 3 pages: does not fit beside a
    c = s.add_request([1], SamplingParams(max_tokens=3))               # would fit, but must not overtake
    plan, _ = run_step(s, ex)
    assert [p.request.request_id for p in plan] == [a]
    assert [r.request_id for r in s.waiting] == [b, c]
    while s.requests[a].finished is False:
        run_step(s, ex)
    plan, _ = run_step(s, ex)
    assert [p.request.request_id for p in plan] == [b, c]


def test_finish_frees_pages_and_eos_stops():
    s, ex = make(pages=8)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=50, eos_token_ids=(7,)))
    run_step(s, ex, token_of=lambda r: 5)
    assert ex.cache.free_pages() == [7]
    _, outs = run_step(s, ex, token_of=lambda r: 7)
    assert outs[0].finished and outs[0].finish_reason == "eos"
    assert ex.cache.free_pages() == [8] and not s.has_work()
    b = s.add_request([1, 2, 3], SamplingParams(max_tokens=3, eos_token_ids=(7,), ignore_eos=True))
    outs = []
    while s.has_work():
        outs += run_step(s, ex, token_of=lambda r: 7)[1]
    assert [o.finish_reason for o in outs] == [None, None, "max_tokens"]


def test_abort_waiting_and_running():
    s, ex = make(pages=8, max_active=1)
    a = s.add_request([1, 2, 3, 4, 5])
    b = s.add_request([1, 2, 3])
    run_step(s, ex)
    assert s.abort(b, ex) and not s.waiting
    assert s.abort(a, ex) and ex.cache.free_pages() == [8]
    assert not s.has_work() and not s.abort(a, ex)


def test_preemption_when_pages_run_out_recomputes_and_keeps_tokens():
    # 6 pages of 4: two requests of 8 prompt tokens take 2+2 pages (+1 each for the
    # first decoded tokens = 6); the next page either needs preempts the later one
    s, ex = make(pages=6, page=4, max_tokens_per_step=100)
    a = s.add_request(list(range(8)), SamplingParams(max_tokens=12))
    b = s.add_request(list(range(8)), SamplingParams(max_tokens=12))
    seen_preempt = False
    for _ in range(200):
        if not s.has_work():
            break
        run_step(s, ex)
        if s.preempted_total and not seen_preempt:
            seen_preempt = True
            # b (the later admission) went back to the FRONT of the line with prompt+output
            assert s.waiting[0].request_id == b
            assert s.waiting[0].pending == s.requests[b].prompt + s.requests[b].output
    assert seen_preempt and not s.has_work()
    for r in (a, b):
        # the counter 'sampler' depends on len(output) only: recompute changes nothing
        assert s.requests[r].output == [1000 + i for i in range(12)]
        assert s.requests[r].finish_reason == "max_tokens"
    assert ex.cache.free_pages() == [6]
    # after the preemption b's whole history ran again as one prompt portion
    assert any(rid == b and len(toks) > 8 for batch in ex.batches for rid, toks, _ in batch)


def test_request_too_large_for_the_pool_fails_with_a_status():
    s, ex = make(pages=3, page=4)
    a = s.add_request(list(range(40)))            # can never fit: 10 pages
    b = s.add_request([1, 2])
    plan, outs = run_step(s, ex)
    assert [(o.request_id, o.finish_reason) for o in outs if o.token is None] == [(a, "out_of_pages")]
    assert [p.request.request_id for p in plan] == [b]


def test_single_request_outgrowing_the_pool_fails_not_hangs():
    s, ex = make(pages=2, page=4)
    a = s.add_request(list(range(6)), SamplingParams(max_tokens=100))
    reasons = []
    for _ in range(50):
        if not s.has_work():
            break
        reasons += [o.finish_reason for o in run_step(s, ex)[1] if o.finished]
    assert reasons == ["out_of_pages"] and ex.cache.free_pages() == [2]
    assert len(s.requests[a].output) >= 2        # it produced what fitted


def test_seed_is_fixed_per_request():
    s, _ = make()
    a = s.add_request([1], SamplingParams(seed=42))
    b = s.add_request([1], SamplingParams())
    assert s.requests[a].seed == 42 and isinstance(s.requests[b].seed, int)


def test_a_step_is_planned_ahead_only_in_the_steady_state():
    """`plan_ahead` gives the next step's plan before this step's tokens are known: when nobody
    waits, everybody decodes, no request ends with the coming token by its limit, none is
    penalised for what it produced, and pages are left. A request that ends meanwhile is passed
    over when the step ahead is recorded."""
    s, ex = make(pages=64, page=4, max_tokens_per_step=100)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=6, eos_token_ids=(7,)))
    b = s.add_request([4, 5], SamplingParams(max_tokens=4))
    plan, _ = s.schedule(ex)
    assert s.plan_ahead(plan) is None                      # prompts: what follows hangs on their tokens
    ex.step(s.entries(plan))
    s.advance(plan, [10, 20], ex)
    plan, _ = s.schedule(ex)                               # both decode: a has 1 token, b has 1
    nxt = s.plan_ahead(plan)
    assert [p.request.request_id for p in nxt] == [a, b] and all(p.samples and len(p.tokens) == 1 for p in nxt)
    ex.step(s.entries(plan))
    ex.step(s.entries(nxt))                                # launched ahead
    s.advance(plan, [11, 21], ex)                          # outputs: a [10, 11], b [20, 21]
    # `nxt` brings b its third token, the step after it the fourth and last: that one may still be
    # planned ahead, none beyond it
    nxt2 = s.plan_ahead(nxt)
    assert nxt2 is not None
    ex.step(s.entries(nxt2))
    outs = s.advance(nxt, [7, 22], ex)                     # a meets its end token
    assert [(o.request_id, o.token, o.finished) for o in outs] == [(a, 7, True), (b, 22, False)]
    assert s.plan_ahead(nxt2) is None                      # a has gone; and b ends with the coming token
    # the step that was under way when a ended drops a's token
    outs = s.advance(nxt2, [99, 23], ex)
    assert [(o.request_id, o.token, o.finished, o.finish_reason) for o in outs] == [(b, 23, True, "max_tokens")]
    assert s.requests[a].output == [10, 11, 7] and s.requests[b].output == [20, 21, 22, 23]
    assert not s.has_work() and ex.cache.free_pages() == [64]
    # a request that is penalised for its tokens, or somebody waiting: not planned ahead
    c = s.add_request([1], SamplingParams(max_tokens=9, frequency_penalty=0.5))
    run_step(s, ex)
    plan, _ = s.schedule(ex)
    assert [p.request.request_id for p in plan] == [c] and s.plan_ahead(plan) is None
    s.abort(c, ex)
    d = s.add_request([1], SamplingParams(max_tokens=9))
    run_step(s, ex)
    plan, _ = s.schedule(ex)
    assert [p.request.request_id for p in plan] == [d] and s.plan_ahead(plan) is not None
    s.add_request([2], SamplingParams(max_tokens=9))
    assert s.plan_ahead(plan) is None
    ex.cache.check()


def test_logprobs_are_recorded_with_their_tokens():
    """`advance` hands each sampled request its entry of the step's log-probabilities (keyed by the
    request's place among the sampled ones), also when a request before it has ended meanwhile."""
    s, ex = make(max_active=4, max_tokens_per_step=64)
    a = s.add_request([1, 2, 3], SamplingParams(max_tokens=4, logprobs=True, top_logprobs=1))
    b = s.add_request([4, 5], SamplingParams(max_tokens=4))
    c = s.add_request([6], SamplingParams(max_tokens=4, logprobs=True))
    plan, _ = s.schedule(ex)
    ex.step(s.entries(plan))
    s.abort(b, ex)
    outs = s.advance(plan, [7, 8, 9], ex, {0: (-0.5, [(7, -0.5)]), 2: (-1.5, [])})
    assert [(o.request_id, o.token, o.logprob, o.top_logprobs) for o in outs] == \
        [(a, 7, -0.5, [(7, -0.5)]), (c, 9, -1.5, [])]
    assert s.requests[a].logprobs == [(-0.5, [(7, -0.5)])] and s.requests[c].logprobs == [(-1.5, [])]
    assert s.requests[b].logprobs == []


def test_sampling_params_check_bias_and_logprobs():
    sp = SamplingParams(logit_bias={9: -100.0, 3: 2})
    assert sp.logit_bias == ((3, 2.0), (9, -100.0)) and hash(sp) is not None
    assert SamplingParams(logit_bias=[(4, 1.0)]).logit_bias == ((4, 1.0),)
    for bad in (dict(logit_bias=[(1, 1.0), (1, 2.0)]), dict(logit_bias={-1: 1.0}), dict(top_logprobs=3),
                dict(logprobs=True, top_logprobs=21)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_keeps_the_budget_the_pages_and_the_order(seed):
    """Random arrivals, prompt lengths, token limits, end tokens and aborts on a pool so small that
    requests are preempted: every step stays within the token budget and the places, the pages
    always suffice (the fake executor reserves like the real one and the cache proves its books),
    nobody overtakes the head of the line, a preempted request goes on where it was, and
    everybody ends with the tokens it should have."""
    import random
    r = random.Random(seed)
    budget, chunk, places = r.choice([8, 17, 64]), r.choice([None, 5, 16]), r.choice([2, 3, 6])
    s, ex = make(pages=r.choice([6, 9, 14]), page=4, max_active=places, max_tokens_per_step=budget, max_chunk=chunk)
    pool = s.cache.groups[0].pool.num_pages
    want, admitted_order, aborted, idle = {}, [], set(), 0
    for step in range(5000):
        if step < 250 and r.random() < 0.35:
            n_prompt, n_new = r.randint(1, 30), r.randint(1, 12)
            eos = (1000 + r.randint(1, n_new),) if r.random() < 0.3 else ()
            rid = s.add_request(list(range(n_prompt)), SamplingParams(max_tokens=n_new, eos_token_ids=eos))
            want[rid] = (n_prompt, n_new, eos)
        if r.random() < 0.03 and want:
            rid = r.choice(list(want))
            if s.abort(rid, ex):
                aborted.add(rid)
        before = {q.request_id: len(q.output) for q in s.requests.values()}
        was_running = {q.request_id for q in s.running}
        plan, outs = run_step(s, ex)
        idle = idle + 1 if not plan and not outs and s.has_work() else 0
        assert idle < 3, "work is waiting and nothing runs"
        assert sum(len(p.tokens) for p in plan) <= budget and len(s.running) <= places
        assert len({p.request.request_id for p in plan}) == len(plan)
        for p in plan:
            rid = p.request.request_id
            if chunk:
                assert len(p.tokens) <= chunk
            if rid not in was_running and p.request.preemptions == 0:
                admitted_order.append(rid)
            assert len(p.request.output) - before[rid] == (1 if p.samples else 0)
        s.cache.check()
        if not s.has_work() and step >= 250:
            break
    assert not s.has_work(), "requests were left over: the scheduler stalled"
    assert admitted_order == sorted(admitted_order)          # first come, first admitted
    assert s.cache.free_pages() == [pool]
    for rid, (n_prompt, n_new, eos) in want.items():
        q = s.requests[rid]
        assert q.finished
        if rid in aborted:
            assert q.finish_reason == "aborted"
            continue
        if q.finish_reason == "out_of_pages":                # it could never fit, or outgrew the pool alone
            assert (n_prompt + len(q.output)) // 4 + 1 > pool - 1 or n_prompt + n_new > (pool - 1) * 4
            continue
        assert q.output == [1000 + i for i in range(len(q.output))]     # nothing lost or repeated over preemptions
        if eos and eos[0] < 1000 + n_new:
            assert q.finish_reason == "eos" and q.output[-1] == eos[0]
        else:
            assert q.finish_reason == "max_tokens" and len(q.output) == n_new
    assert s.preempted_total > 0 or pool > 9


def test_decode_graph_sizes_are_few_and_waste_little():
    """A batch that shrinks request by request meets a short list of graph sizes: every size up to
    8, then steps of 4, 8 and 16; a size serves itself, and the stand-in rows stay under a third."""
    from rllm_b200.engine.graphs import padded_rows
    sizes = sorted({padded_rows(s) for s in range(1, 257)})
    assert sizes[:8] == list(range(1, 9)) and len(sizes) <= 32
    for s in range(1, 257):
        p = padded_rows(s)
        assert p >= s and padded_rows(p) == p and (p - s) * 3 < p + 3
    assert [padded_rows(s) for s in (9, 12, 13, 33, 64, 65, 200)] == [12, 12, 16, 40, 64, 80, 208]


@pytest.mark.parametrize("seed", range(4))
def test_random_traffic_with_steps_planned_ahead_gives_the_same_outputs(seed):
    """The loop of `LLM.step` (a step planned and run ahead whenever `plan_ahead` allows it, its
    tokens recorded one call later) against the plain loop, on the same random traffic with end
    tokens, limits and aborts: the same outputs and reasons, pages that always suffice, an empty
    pool at the end. The token a request gets is a function of its id and its place, as with the
    counter-based random numbers."""
    import random

    def token_of(req, ahead=0):
        return (req.request_id * 7 + (len(req.output) + ahead) * 3) % 50

    def traffic(s, ex, ahead_allowed):
        r = random.Random(100 + seed)
        ahead, aborted, planned_ahead = None, set(), 0
        for step in range(3000):
            if step < 200 and r.random() < 0.15:
                sp = SamplingParams(max_tokens=r.randint(1, 25), eos_token_ids=(r.randrange(50),) if r.random() < 0.5 else ())
                s.add_request(list(range(r.randint(1, 20))), sp)
            if r.random() < 0.02 and s.requests:
                rid = r.choice(list(s.requests))
                if rid not in aborted and s.abort(rid, ex):
                    aborted.add(rid)
            if ahead is not None:
                plan, tokens = ahead
                ahead = None
            else:
                plan, _ = s.schedule(ex)
                if not plan:
                    if not s.has_work() and step >= 200:
                        break
                    continue
                ex.step(s.entries(plan))
                tokens = [token_of(p.request) for p in plan if p.samples]
            if ahead_allowed:
                nxt = s.plan_ahead(plan)
                if nxt is not None:
                    ex.step(s.entries(nxt))                 # runs before this step's tokens are recorded
                    ahead = (nxt, [token_of(p.request, 1) for p in nxt])
                    planned_ahead += 1
            s.advance(plan, tokens, ex)
            if ahead is not None and all(p.request.finished for p in ahead[0]):
                ahead = None
            s.cache.check()
        assert not s.has_work() and s.cache.free_pages() == [s.cache.groups[0].pool.num_pages]
        return {rid: (q.output, q.finish_reason) for rid, q in s.requests.items()}, planned_ahead

    a, n_ahead = traffic(*make(pages=200, page=4, max_active=6, max_tokens_per_step=32), ahead_allowed=True)
    b, _ = traffic(*make(pages=200, page=4, max_active=6, max_tokens_per_step=32), ahead_allowed=False)
    assert n_ahead > 20
    # an abort between a step ahead and its recording may cost the aborted request its last token;
    # everybody else has exactly the same output
    for rid in a:
        if a[rid][1] == "aborted":
            assert b[rid][1] == "aborted" and a[rid][0][: len(b[rid][0])] == b[rid][0][: len(a[rid][0])]
        else:
            assert a[rid] == b[rid], rid


def test_uniform_numbers_hang_on_seed_and_index_only():
    """The draw of a request's n-th token: in [0, 1), 24 bits, the same for the same (seed, index),
    spread evenly, and neighbouring seeds or indices give unrelated values."""
    from rllm_b200.sampling.rng import uniform
    us = [uniform(5, i) for i in range(4000)]
    assert all(0.0 <= u < 1.0 and u * (1 << 24) == int(u * (1 << 24)) for u in us)
    assert us == [uniform(5, i) for i in range(4000)] and len(set(us)) > 3990
    assert abs(sum(us) / len(us) - 0.5) < 0.02
    counts = [0] * 10
    for u in us:
        counts[int(u * 10)] += 1
    assert min(counts) > 330 and max(counts) < 470
    other = [uniform(6, i) for i in range(4000)]
    mean = lambda v: sum(v) / len(v)
    cov = mean([a * b for a, b in zip(us, other)]) - mean(us) * mean(other)
    lag = mean([a * b for a, b in zip(us, us[1:])]) - mean(us[:-1]) * mean(us[1:])
    assert abs(cov) < 0.01 and abs(lag) < 0.01
    assert uniform(2 ** 63 + 11, 0) == uniform(2 ** 63 + 11, 0) and 0 <= uniform(-3, 7) < 1
