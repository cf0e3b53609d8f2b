"""Generation through the entry point: greedy tokens equal the plain implementation's,
sampling follows the counter-based draws however the work is batched, long decoding stays
on the plain logits, the first tokens of a sequence are right, and pages that run out
preempt and recompute without changing the output."""
import numpy as np
import pytest
import torch

import plain_llama as P
import replay
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {n: tiny.make_model_dir(root, n) for n in tiny.TINY}


def llm(d, name, dtype, **kw):
    from rllm_b200.api import LLM
    kw.setdefault("page_size", tiny.TINY[name][4])
    return LLM(d, dtype=dtype, **kw)


@pytest.mark.parametrize("name,lens,steps", [("A", [5, 11, 17], 8), ("B", [3, 9, 24, 40], 12)])
def test_greedy_generation_equals_plain_float32(dirs, name, lens, steps):
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], 7 + n) for n in lens]
    want = [P.greedy(cfg, w, p, steps) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=steps)
    # all together; in portions of 7 mixed with decodes; one at a time
    assert llm(dirs[name], name, "float32", num_pages=64).generate(prompts, sp) == want
    assert llm(dirs[name], name, "float32", num_pages=64, max_tokens_per_step=9, max_chunk=7).generate(prompts, sp) == want
    one = llm(dirs[name], name, "float32", num_pages=64, max_active=1)
    assert one.generate(prompts, sp) == want


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_stays_on_the_plain_path(dirs, name):
    """In bfloat16 a near tie may flip a token, after which the texts differ; so each chosen
    token is checked against the plain logits for the engine's own history: it must be the
    plain argmax or within the bfloat16 tolerance of it."""
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], 70 + n) for n in (6, 21)]
    outs = llm(dirs[name], name, "bfloat16", num_pages=64).generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        lg = P.forward(cfg, w, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            assert float(lg[i].max() - lg[i, tok]) <= 3e-2 * float(lg.abs().max()), (i, tok)


def test_temperature_sampling_is_the_same_however_it_is_batched(dirs):
    from rllm_b200.sampling import SamplingParams, uniform
    name = "B"
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], 5 + n) for n in (3, 9, 24, 40)]
    sps = [SamplingParams(temperature=0.8, max_tokens=12, seed=100 + i) for i in range(4)]
    a = llm(dirs[name], name, "float32", num_pages=64).generate(prompts, sps)
    b = llm(dirs[name], name, "float32", num_pages=64, max_tokens_per_step=9, max_chunk=7).generate(prompts, sps)
    c = llm(dirs[name], name, "float32", num_pages=64, max_active=2).generate(prompts, sps)
    assert a == b == c
    # and each token is the one the plain pipeline picks for the same uniform number
    for p, o, sp in zip(prompts, a, sps):
        for i, tok in enumerate(o):
            probs = P.sample_probs(P.forward(cfg, w, p + o[:i])[-1], 0.8).double()
            cdf = torch.cumsum(probs, 0)
            u = uniform(sp.seed, i)
            lo = float(cdf[tok - 1]) if tok else 0.0
            assert lo - 1e-4 <= u <= float(cdf[tok]) + 1e-4, (i, tok, u)
    d = llm(dirs[name], name, "float32", num_pages=64).generate(
        prompts, [SamplingParams(temperature=0.8, max_tokens=12, seed=999)] * 4)
    assert d != a                                           # another seed, other draws


def test_pages_running_out_preempts_and_output_is_unchanged(dirs):
    from rllm_b200.sampling import SamplingParams
    name = "B"                                              # pages of 8
    cfg, _ = P.read_model_dir(dirs[name])
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], 31 + n) for n in (20, 22, 18)]
    sp = SamplingParams(temperature=0.0, max_tokens=30)
    roomy = llm(dirs[name], name, "float32", num_pages=64)
    want = roomy.generate(prompts, sp)
    tight = llm(dirs[name], name, "float32", num_pages=12)  # 96 positions for 3 x ~50
    got = tight.generate(prompts, sp)
    assert tight.scheduler.preempted_total > 0 and roomy.scheduler.preempted_total == 0
    assert got == want
    tight.engine.cache.check()
    assert tight.engine.cache.free_pages() == [12]


def test_preemption_and_temperature_in_bfloat16(dirs):
    """The two tests above once on the serving path. bfloat16 rounds differently from step shape to
    step shape, so outputs are not compared with each other but each with the plain implementation
    on its own history: a greedy token must be the plain argmax or within the bfloat16 tolerance of
    it, a drawn token's interval of the plain cumulative distribution must hold the request's
    uniform number to within what that tolerance moves the distribution."""
    from rllm_b200.sampling import SamplingParams, uniform
    name = "B"
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [tiny.random_prompt(n, cfg["vocab_size"], 31 + n) for n in (20, 22, 18)]
    tight = llm(dirs[name], name, "bfloat16", num_pages=12)          # 96 positions for 3 x ~50
    outs = tight.generate(prompts, SamplingParams(temperature=0.0, max_tokens=30))
    assert tight.scheduler.preempted_total > 0
    tight.engine.cache.check()
    assert tight.engine.cache.free_pages() == [12]
    for p, o in zip(prompts, outs):
        assert len(o) == 30
        lg = P.forward(cfg, w, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            assert float(lg[i].max() - lg[i, tok]) <= 3e-2 * float(lg[i].abs().max()), (i, tok)
    sps = [SamplingParams(temperature=0.8, max_tokens=12, seed=100 + i) for i in range(3)]
    outs = llm(dirs[name], name, "bfloat16", num_pages=64, max_tokens_per_step=9, max_chunk=7).generate(prompts, sps)
    for p, o, sp in zip(prompts, outs, sps):
        for i, tok in enumerate(o):
            cdf = torch.cumsum(P.sample_probs(P.forward(cfg, w, p + o[:i])[-1], 0.8).double(), 0)
            u = uniform(sp.seed, i)
            lo = float(cdf[tok - 1]) if tok else 0.0
            assert lo - 2e-2 <= u <= float(cdf[tok]) + 2e-2, (i, tok, u)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_long_decoding_and_first_tokens(dirs, dtype, tol):
    """250 tokens decoded one by one after a 3-token prompt (the window of model C passes
    many pages meanwhile), logits compared at every position; the first positions include
    position 0, where a key sees only itself."""
    from rllm_b200.engine import Entry, load_engine
    name = "C"
    cfg, w = P.read_model_dir(dirs[name])
    toks = tiny.random_prompt(253, cfg["vocab_size"], 77)
    eng = load_engine(dirs[name], dtype=dtype, page_size=4, max_tokens=256, max_requests=2)
    got = {}
    lg = eng.step([Entry("a", toks[:3], [0, 1, 2])]).float().cpu().numpy()
    got.update({("a", i): lg[i] for i in range(3)})
    for i in range(3, 253):
        got[("a", i)] = eng.step([Entry("a", [toks[i]], [0])]).float().cpu().numpy()[0]
    held = [sum(p >= 0 for p in pages) for pages in eng.cache.live["a"].pages]
    windowed = [g.spec.window is not None for g in eng.cache.groups]
    assert any(windowed) and all((h <= 8) == wnd for h, wnd in zip(held, windowed))
    replay.compare(got, replay.plain_logits(dirs[name], {"a": toks}), tol, f"long decode {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(dirs, dtype):
    """In the steady state of decoding a step is launched before the tokens of the step before
    it are read. The same requests with and without that: the same tokens, finish reasons and
    step-by-step outputs, also when requests meet an end token or their limit at different
    times, are drawn with a temperature, or are aborted half-way; and every page comes back."""
    from rllm_b200.sampling import SamplingParams
    name = "D"
    cfg, _ = P.read_model_dir(dirs[name])
    V = cfg["vocab_size"]
    prompts = [tiny.random_prompt(n, V, 900 + n) for n in (5, 19, 33, 8)]
    # a first run without limits tells which tokens come; some of them then serve as end tokens
    free = llm(dirs[name], name, dtype, num_pages=64)
    free.run_ahead = False
    base = free.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    sps = [SamplingParams(temperature=0.0, max_tokens=40, eos_token_ids=(base[0][13],)),
           SamplingParams(temperature=0.0, max_tokens=23),
           SamplingParams(temperature=0.7, top_p=0.9, max_tokens=40, seed=5, eos_token_ids=(base[2][30],)),
           SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)]

    def run(ahead):
        m = llm(dirs[name], name, dtype, num_pages=64)
        m.run_ahead = ahead
        rids = [m.add_request(p, sp) for p, sp in zip(prompts, sps)]
        log, steps = [], 0
        while m.has_work():
            outs = m.step()
            steps += 1
            log.append(sorted((o.request_id, o.token, o.finished, o.finish_reason) for o in outs))
            if steps == 30:
                assert m.abort(rids[3])
        m.engine.cache.check()
        assert m.engine.cache.free_pages() == [64]
        # the account of the steps: every token run and drawn is counted, the device's time lies inside
        # the time the steps took and is more than nothing
        torch.cuda.synchronize()
        m._settle_device_time()
        st = m.stats
        kept = sum(len(m.scheduler.requests[r].output) for r in rids)
        assert st.steps == steps and kept <= st.sampled <= kept + 2 * len(rids)     # a token drawn ahead for a request that had ended is dropped
        assert st.prefill_tokens == sum(len(p) for p in prompts) and st.tokens >= st.prefill_tokens + st.sampled - len(rids)
        assert 0.0 < st.device_s <= st.wall_s * 1.05 and not m._timed
        return log, [m.scheduler.requests[r].output for r in rids], m.steps_ahead

    log0, out0, ahead0 = run(False)
    log1, out1, ahead1 = run(True)
    assert ahead0 == 0 and ahead1 > 10
    assert out1 == out0 and log1 == log0
    assert len(out0[0]) <= 14 and out0[0][-1] == base[0][13] and len(out0[1]) == 23


@pytest.mark.parametrize("seed", [0, 1])
def test_random_traffic_is_the_same_with_and_without_steps_ahead(dirs, seed):
    """Forty requests of random lengths and limits arrive over time at a pool too small for them
    (so requests wait, are preempted and recomputed), some with end tokens, some drawn with a
    temperature, a few aborted: token for token the same with steps launched ahead and without,
    and every page is back at the end."""
    import random
    from rllm_b200.sampling import SamplingParams
    name = "D"
    cfg, _ = P.read_model_dir(dirs[name])
    V = cfg["vocab_size"]

    def run(ahead):
        r = random.Random(seed)
        m = llm(dirs[name], name, "float32", num_pages=18, max_active=6, max_tokens_per_step=48, max_chunk=32)
        m.run_ahead = ahead
        todo = []
        for i in range(40):
            sp = SamplingParams(temperature=r.choice([0.0, 0.0, 0.9]), top_p=r.choice([1.0, 0.8]),
                                max_tokens=r.randint(1, 40), seed=1000 + i,
                                eos_token_ids=tuple(r.sample(range(V), r.choice([0, 0, 40]))))
            todo.append((r.randint(0, 60), tiny.random_prompt(r.randint(1, 70), V, 300 + i), sp))
        abort_at = {r.randint(5, 80): r.randint(0, 39) for _ in range(4)}
        rids, step = {}, 0
        while todo or m.has_work():
            for item in [t for t in todo if t[0] <= step]:
                todo.remove(item)
                rids[len(rids)] = m.add_request(item[1], item[2])
            if step in abort_at and abort_at[step] in rids:
                m.abort(rids[abort_at[step]])
            if m.has_work():
                m.step()
            step += 1
            assert step < 5000
        m.engine.cache.check()
        assert m.engine.cache.free_pages() == [18]
        reqs = m.scheduler.requests
        return [(reqs[rids[i]].output, reqs[rids[i]].finish_reason) for i in sorted(rids)], \
            m.scheduler.preempted_total, m.steps_ahead

    a, pre_a, ahead_a = run(False)
    b, pre_b, ahead_b = run(True)
    assert ahead_a == 0 and ahead_b > 0 and pre_a > 0
    assert a == b


@pytest.mark.parametrize("name,dtype", [("D", "float32"), ("D", "bfloat16"), ("C", "float32")])
def test_a_shrinking_batch_reuses_padded_graphs(dirs, name, dtype):
    """Thirteen requests decode together and end one after the other. Decode graphs come in a
    short list of sizes (13 requests run in the graph for 16, the rows beyond them are stand-ins),
    so the batch meets a handful of captures on its way down, not one per size; and every
    request's tokens are what it gets alone."""
    from rllm_b200.engine.graphs import padded_rows
    from rllm_b200.sampling import SamplingParams
    assert [padded_rows(n) for n in (1, 8, 9, 12, 13, 33, 64, 65, 200)] == [1, 8, 12, 12, 16, 40, 64, 80, 208]
    cfg, w = P.read_model_dir(dirs[name])      # C: two groups of layers (all keys, a window of 24), pages of 4
    prompts = [tiny.random_prompt(3 + 2 * i, cfg["vocab_size"], 500 + i) for i in range(13)]
    sps = [SamplingParams(temperature=0.0, max_tokens=4 + 3 * i) for i in range(13)]
    pages = 64 if name == "D" else 400
    m = llm(dirs[name], name, dtype, num_pages=pages, max_active=16)
    outs = m.generate(prompts, sps)
    sizes = sorted({k[0] for k in m.engine.graphs.slots})
    assert set(sizes) <= {1, 2, 3, 4, 5, 6, 7, 8, 12, 16} and 16 in sizes and 12 in sizes
    for p_, sp, o in zip(prompts, sps, outs):
        assert len(o) == sp.max_tokens
        if dtype == "float32":
            assert o == P.greedy(cfg, w, p_, sp.max_tokens)
        else:       # a near tie may go either way in bfloat16: each token against the plain logits of its own history
            lg = P.forward(cfg, w, p_ + o[:-1])[len(p_) - 1:]
            for i, tok in enumerate(o):
                assert float(lg[i].max() - lg[i, tok]) <= 3e-2 * float(lg.abs().max()), (i, tok)
    m.engine.cache.check()
    assert set(m.engine.cache.free_pages()) == {pages}


def test_the_step_loop_reports_a_kernel_that_gave_up(dirs):
    """A kernel whose bounded wait ran out sets a device word and returns; the words travel to the
    host with every step's tokens, and `LLM.step` raises. (The word is set by hand here.)"""
    from rllm_b200.kernels.ops import KernelError
    from rllm_b200.sampling import SamplingParams
    m = llm(dirs["D"], "D", "bfloat16", num_pages=32)
    m.add_request([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=20))
    m.step(); m.step()
    m.engine.error_words[0] = 3 | (5 << 8)
    with pytest.raises(KernelError, match="role 3, detail 5"):
        for _ in range(3):
            m.step()
    m.engine.check()                                         # read and cleared


def test_a_bounded_wait_that_runs_out_is_reported_and_the_gpu_goes_on(dirs):
    """The kernels' own way out of a wait that never ends, for real: a one-warp kernel waits on an
    mbarrier nobody arrives at, with a limit of 200,000 cycles (a tenth of a millisecond), gives up,
    and records the failure in the device error word. The step loop raises at its next step, and
    after the word is read the GPU works as before. (With an arrival first, the same kernel records
    nothing.)"""
    import time
    from rllm_b200.kernels import ops, sm100
    from rllm_b200.kernels.ops import KernelError
    from rllm_b200.sampling import SamplingParams
    m = llm(dirs["D"], "D", "bfloat16", num_pages=32)
    m.add_request([1, 2, 3], SamplingParams(temperature=0.0, max_tokens=30))
    m.step(); m.step()
    sm100.wait_probe(m.engine.device, arrive_first=True)
    torch.cuda.synchronize()
    m.engine.check()                                         # the wait was met: nothing recorded
    t0 = time.time()
    sm100.wait_probe(m.engine.device, limit_cycles=200000)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0                            # it gave up after its limit, not later
    with pytest.raises(KernelError, match="role 9, detail 1"):
        for _ in range(3):
            m.step()
    m.engine.check()                                         # read and cleared
    x = torch.randn(8, 256, device="cuda:0").to(torch.bfloat16)
    w = torch.randn(128, 256, device="cuda:0").to(torch.bfloat16)
    got = sm100.gemm(x, w, ops.EPI_STORE_F32, split=False)   # a tcgen05 product afterwards
    assert float((got - x.float() @ w.float().t()).abs().max()) <= 1e-3 * float(got.abs().max())
    sm100.check_error("cuda:0")


def test_sampling_params_defaults_follow_the_reference():
    from rllm_b200.sampling import SamplingParams
    sp = SamplingParams()
    assert (sp.temperature, sp.top_p, sp.top_k, sp.min_p, sp.max_tokens) == (1.0, 1.0, 0, 0.0, 128)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)


def test_penalties_change_the_choice(dirs):
    from rllm_b200.sampling import SamplingParams
    name = "A"
    cfg, _ = P.read_model_dir(dirs[name])
    prompt = tiny.random_prompt(8, cfg["vocab_size"], 3)
    m = llm(dirs[name], name, "float32", num_pages=32)
    plain = m.generate([prompt], SamplingParams(temperature=0.0, max_tokens=24))[0]
    pen = m.generate([prompt], SamplingParams(temperature=0.0, max_tokens=24, presence_penalty=50.0))[0]
    assert len(set(pen)) == len(pen)                        # a used token is never chosen again
    assert plain[0] == pen[0]


def test_logit_bias_bans_and_forces_tokens(dirs):
    """A bias of -100 on the tokens greedy decoding would choose removes them from the output; a
    large bias on one token makes it the answer everywhere; ids beyond the vocabulary are passed
    over; the first token without bias is the plain one."""
    from rllm_b200.sampling import SamplingParams
    name = "B"
    cfg, w = P.read_model_dir(dirs[name])
    V = cfg["vocab_size"]
    prompt = tiny.random_prompt(11, V, 5)
    m = llm(dirs[name], name, "float32", num_pages=32)
    plain = m.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8))[0]
    assert plain == P.greedy(cfg, w, prompt, 8)
    banned = {t: -100.0 for t in set(plain)}
    banned[V + 5] = 3.0
    got = m.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, logit_bias=banned))[0]
    assert not set(got) & set(plain)
    # the plain rule, step by step, on the plain model's logits
    seq, want = list(prompt), []
    for _ in range(8):
        x = P.adjust_logits(P.forward(cfg, w, seq)[-1], [], logit_bias=banned)
        want.append(int(torch.argmax(x)))
        seq.append(want[-1])
    assert got == want
    forced = m.generate([prompt, prompt[:3]], SamplingParams(temperature=0.9, top_p=0.95, max_tokens=6, seed=3,
                                                           logit_bias={17: 200.0}))
    assert forced == [[17] * 6, [17] * 6]


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_logprobs_come_back_with_the_tokens(dirs, name, dtype):
    """Greedy and drawn requests side by side, some with log-probabilities and some without, with
    and without steps launched ahead: the tokens are what they are without log-probabilities, and
    every token's ln p and the listed alternatives are those of the plain rule on the plain
    model's logits."""
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    V = cfg["vocab_size"]
    prompts = [tiny.random_prompt(n, V, 20 + n) for n in (9, 5, 14)]
    sps = [SamplingParams(temperature=0.0, max_tokens=7, logprobs=True, top_logprobs=4),
           SamplingParams(temperature=0.8, top_k=12, top_p=0.9, max_tokens=9, seed=5, logprobs=True, top_logprobs=2),
           SamplingParams(temperature=0.7, max_tokens=8, seed=6)]
    tol = 1e-3 if dtype == "float32" else 0.15
    for ahead in (True, False):
        m = llm(dirs[name], name, dtype, num_pages=32)
        m.run_ahead = ahead
        reqs = m.generate(prompts, sps, details=True)
        bare = m.generate(prompts, [SamplingParams(**{**sp.__dict__, "logprobs": False, "top_logprobs": 0}) for sp in sps])
        assert [r.output for r in reqs] == bare
        assert reqs[2].logprobs == [] and [len(r.logprobs) for r in reqs[:2]] == [7, 9]
        for r, prompt, sp in zip(reqs[:2], prompts, sps):
            rows = P.forward(cfg, w, prompt + r.output[:-1])[len(prompt) - 1:]
            for tok, (lp, top), x in zip(r.output, r.logprobs, rows):
                want_lp, want_top = P.logprobs(x, sp.temperature, sp.top_k, tok, sp.top_logprobs)
                assert abs(lp - want_lp) <= tol
                assert len(top) == sp.top_logprobs and all(b <= a + 1e-6 for (_, a), (_, b) in zip(top, top[1:]))
                if dtype == "float32":
                    assert [t for t, _ in top] == [t for t, _ in want_top]
                    assert all(abs(a[1] - b[1]) <= tol for a, b in zip(top, want_top))
            if sp.greedy:
                assert all(top[0][0] == tok for tok, (_, top) in zip(r.output, r.logprobs))


def test_cli_run_and_batch(dirs, tmp_path):
    import os, subprocess, sys
    rllm = os.path.join(replay.ROOT, "bin", "rllm")
    cfg, w = P.read_model_dir(dirs["A"])
    prompt = tiny.random_prompt(9, cfg["vocab_size"], 12)
    want = P.greedy(cfg, w, prompt, 6)
    r = subprocess.run([sys.executable, rllm, "run", "--model", dirs["A"], "--prompt-ids",
                        " ".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0",
                        "--dtype", "float32", "--kv-pages", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.split()] == want and "tok/s" in r.stderr
    f = tmp_path / "prompts.txt"
    f.write_text(" ".join(map(str, prompt)) + "\n" + " ".join(map(str, prompt[:4])) + "\n")
    r = subprocess.run([sys.executable, rllm, "batch", "--model", dirs["A"], "--batch-file", str(f), "--ids",
                        "--max-tokens", "6", "--temperature", "0", "--dtype", "float32", "--kv-pages", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert [int(x) for x in lines[0].split("]")[1].split()] == want
    r = subprocess.run([sys.executable, rllm, "run", "--model", dirs["A"], "--prompt-ids", "1 2",
                        "--kv-quant", "turbo4"], capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "not built" in r.stderr


def test_cli_text_prompt_gets_bos_and_stops_at_eos(dirs, tmp_path):
    """`rllm run --prompt TEXT` with a tokenizer.json in the folder: the model's BOS goes in front
    of the text's tokens once, the output ends with the model's end-of-sequence token (both from
    config.json), and the text is streamed as it is decoded."""
    import json, os, shutil, subprocess, sys
    tk = pytest.importorskip("tokenizers")
    cfg, w = P.read_model_dir(dirs["A"])
    V = cfg["vocab_size"]
    prompt = [1, 5, 17, 3]                                   # BOS = 1, then "w5 w17 w3"
    want = P.greedy(cfg, w, prompt, 6)
    stop = want.index(want[2])                               # the output ends where the third token first appears
    d = str(tmp_path / "with_tokenizer")
    shutil.copytree(dirs["A"], d)
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    raw.update(bos_token_id=1, eos_token_id=want[stop])
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    tok = tk.Tokenizer(tk.models.WordLevel({f"w{i}": i for i in range(V)}, unk_token="w0"))
    tok.pre_tokenizer = tk.pre_tokenizers.Whitespace()
    tok.save(os.path.join(d, "tokenizer.json"))
    rllm = os.path.join(replay.ROOT, "bin", "rllm")
    r = subprocess.run([sys.executable, rllm, "run", "--model", d, "--prompt", "w5 w17 w3", "--max-tokens", "6",
                        "--temperature", "0", "--dtype", "float32", "--kv-pages", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == [f"w{t}" for t in want[: stop + 1]]
    assert f"prefill: {len(prompt)} tokens" in r.stderr
