"""The engine against the plain implementation, in 32-bit and in bfloat16, for every way of
cutting the same requests into steps. A difference that shows in one family only is a fault
of the cache or the batch; the failure names the first wrong (request, position)."""
import os

import numpy as np
import pytest
import torch

import replay
import tiny

pytestmark = pytest.mark.gpu

# Largest error at a position relative to that position's own largest logit. 32-bit: only
# summation order differs (measured 1.3e-6 or less on these models). bfloat16: weights are the
# same bfloat16 values in both, activations and cache are rounded to 8 bits of mantissa at
# every layer boundary (measured up to 1.0e-2 on these models).
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}

# D and E have the head sizes of the tensor-core attention kernels; their long requests span
# several key tiles, key ranges and pages, and a window's edge.
LENGTHS = {"A": [5, 11, 17, 40, 70], "B": [3, 9, 24, 40, 97], "C": [6, 33, 58, 90, 121],
           "D": [4, 70, 131, 300, 65], "E": [9, 150, 64, 257, 33], "F": [7, 90, 35, 140, 2]}


def requests_for(name):
    vocab = tiny.TINY[name][0]["vocab_size"]
    return {f"r{i}": tiny.random_prompt(n, vocab, 100 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: tiny.make_model_dir(root, n) for n in tiny.TINY}


@pytest.fixture(scope="module")
def plain(model_dirs):
    return {n: replay.plain_logits(model_dirs[n], requests_for(n)) for n in tiny.TINY}


def engine_for(model_dir, name, dtype, max_tokens):
    from rllm_b200.engine import load_engine
    return load_engine(model_dir, dtype=dtype, page_size=tiny.TINY[name][4], max_tokens=max_tokens,
                       max_requests=8)


FAMILIES = {
    "whole": replay.whole,
    "prefill_then_decode": replay.prefill_then_decode,
    "portions": replay.portions,
    "mixed": replay.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.TINY))
@pytest.mark.parametrize("family", list(FAMILIES))
def test_family_matches_plain(model_dirs, plain, name, dtype, family):
    reqs = requests_for(name)
    steps = FAMILIES[family](reqs)
    # a pool just large enough, so pages of finished requests are used again
    eng = engine_for(model_dirs[name], name, dtype, replay.max_live_tokens(steps, reqs))
    got = replay.run_in_process(eng, steps)
    worst = replay.compare(got, plain[name], TOL[dtype], f"tiny-{name} {dtype} {family}", per_position=True)
    assert all(n == eng.cache.groups[0].pool.num_pages for n in eng.cache.free_pages())
    print(f"tiny-{name} {dtype} {family}: worst relative error {worst:.2e}")


@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("family", list(FAMILIES))
def test_family_with_the_tcgen05_prefill_attention(model_dirs, plain, name, family, monkeypatch):
    """The engine takes the tcgen05 prefill attention from 512 keys; here from 16, so that the
    short requests of the tiny models (head sizes 64 and 128, a window on one layer of E) go
    through it in every family, beside decode tokens and with pages used again."""
    from rllm_b200.kernels import sm100
    monkeypatch.setattr(sm100, "TC_ATTENTION_MIN_KEYS", 16)
    calls = []
    real = sm100.attention_prefill_tc
    monkeypatch.setattr(sm100, "attention_prefill_tc", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    reqs = requests_for(name)
    steps = FAMILIES[family](reqs)
    eng = engine_for(model_dirs[name], name, "bfloat16", replay.max_live_tokens(steps, reqs))
    got = replay.run_in_process(eng, steps)
    replay.compare(got, plain[name], TOL["bfloat16"], f"tiny-{name} bfloat16 {family} (tcgen05 attention)",
                   per_position=True)
    if family in ("whole", "prefill_then_decode"):      # the other families' portions may all be under 128 rows
        assert calls, "the tcgen05 prefill kernel was not used"


@pytest.mark.parametrize("name", ["D", "E"])
def test_long_portions_beside_decode_tokens(model_dirs, plain, name, monkeypatch):
    """A step as the scheduler builds it under load: requests that decode in front, then a prompt
    portion long enough for the tcgen05 prefill attention. The single tokens then go to the decode
    kernel and the portion to the tcgen05 kernel, in one step, into one output."""
    from rllm_b200.kernels import sm100
    monkeypatch.setattr(sm100, "TC_ATTENTION_MIN_KEYS", 16)
    used = {"decode": 0, "tc": 0}
    real_d, real_t = sm100.attention_decode, sm100.attention_prefill_tc
    monkeypatch.setattr(sm100, "attention_decode", lambda *a, **k: (used.__setitem__("decode", used["decode"] + 1), real_d(*a, **k))[1])
    monkeypatch.setattr(sm100, "attention_prefill_tc", lambda *a, **k: (used.__setitem__("tc", used["tc"] + 1), real_t(*a, **k))[1])
    reqs = requests_for(name)
    a, b, c, d = "r1", "r2", "r3", "r4"          # D: 70, 131, 300, 65 tokens; E: 150, 64, 257, 33
    ent = lambda r, lo, hi: {"id": r, "tokens": reqs[r][lo:hi], "want": list(range(hi - lo))}
    na, nb, nc, nd = (len(reqs[r]) for r in (a, b, c, d))
    steps = [{"entries": [ent(a, 0, na - 3)], "end": []},
             {"entries": [ent(b, 0, nb - 3)], "end": []},
             {"entries": [ent(a, na - 3, na - 2), ent(b, nb - 3, nb - 2), ent(c, 0, 120)], "end": []},
             {"entries": [ent(a, na - 2, na - 1), ent(b, nb - 2, nb - 1), ent(c, 120, nc - 1), ent(d, 0, nd)], "end": [d]},
             {"entries": [ent(a, na - 1, na), ent(b, nb - 1, nb), ent(c, nc - 1, nc)], "end": [a, b, c]}]
    for i, s in enumerate(steps):
        s["step"] = i
    eng = engine_for(model_dirs[name], name, "bfloat16", replay.max_live_tokens(steps, reqs))
    before = dict(used)
    got = replay.run_in_process(eng, steps)
    want = {k: v for k, v in plain[name].items() if k[0] in (a, b, c, d)}
    replay.compare(got, want, TOL["bfloat16"], f"tiny-{name} bfloat16 portions beside decode tokens",
                   per_position=True)
    # steps 2 and 3 each went to both kernels, in every layer
    layers = tiny.TINY[name][0]["num_hidden_layers"]
    assert used["tc"] - before["tc"] >= 4 * layers and used["decode"] - before["decode"] >= 3 * layers


@pytest.mark.parametrize("name", list(tiny.TINY))
def test_float32_is_the_same_however_it_is_cut(model_dirs, name):
    """In 32-bit every family gives bit-identical logits: each output element is summed in
    an order that depends on its position only."""
    reqs = requests_for(name)
    base = None
    for family, make in FAMILIES.items():
        steps = make(reqs)
        eng = engine_for(model_dirs[name], name, "float32", replay.max_live_tokens(steps, reqs))
        got = replay.run_in_process(eng, steps)
        if base is None:
            base = got
        else:
            for key in base:
                assert np.array_equal(base[key], got[key]), f"{family}: {key} differs from whole"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_dirs, plain, tmp_path, dtype):
    """The same through bin/trace_run (a process of its own, JSON in, .f32 files out)."""
    name = "B"
    reqs = requests_for(name)
    steps = replay.mixed(reqs)
    vocab = tiny.TINY[name][0]["vocab_size"]
    got = replay.run_program(model_dirs[name], dtype, steps, str(tmp_path / "out"),
                             replay.max_live_tokens(steps, reqs), vocab,
                             extra_args=["--page-size", str(tiny.TINY[name][4])])
    replay.compare(got, plain[name], TOL[dtype], f"trace_run {dtype}", per_position=True)


@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_checked_run(model_dirs, plain, name, dtype, monkeypatch):
    """RLLM_B200_CHECKED=1: every step's block tables and cache slots are tested on the device before
    a kernel reads them. The families run as always and nothing is reported; then a table entry that
    names a page outside the pool is slipped in: the step runs to its end (the access is skipped, not
    made), and the next check names the entry."""
    from rllm_b200.engine import Entry
    from rllm_b200.engine.step import Engine, StepError
    monkeypatch.setenv("RLLM_B200_CHECKED", "1")
    reqs = requests_for(name)
    for family in ("prefill_then_decode", "mixed"):
        steps = FAMILIES[family](reqs)
        eng = engine_for(model_dirs[name], name, dtype, replay.max_live_tokens(steps, reqs))
        assert eng.checked
        got = replay.run_in_process(eng, steps)
        replay.compare(got, plain[name], TOL[dtype], f"tiny-{name} {dtype} {family} (checked)", per_position=True)
        eng.check()
    real = Engine.fill_meta

    def corrupt(self, host, lay, entries, rcs):
        real(self, host, lay, entries, rcs)
        host[int(lay.offs[8])] = self.cache.groups[0].pool.num_pages + 5       # first page of the first sequence
    monkeypatch.setattr(Engine, "fill_meta", corrupt)
    eng = engine_for(model_dirs[name], name, dtype, 256)
    logits = eng.step([Entry("x", reqs["r3"][:20], [19])])
    torch.cuda.synchronize()
    assert logits.shape[0] == 1
    with pytest.raises(StepError, match="block-table entry 0"):
        eng.check()
    eng.check()                                                              # read and cleared
