"""Builds replay traces (the JSON steps `bin/trace_run` reads) in the four families the
tests compare, and runs them either in-process through `Engine.step` or through the
`bin/trace_run` program. Every family asks for the logits at every position, so each can
be compared with the plain implementation's whole-sequence logits."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests):
    """Each request alone and whole: one step per request."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks,
                      "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def prefill_then_decode(requests, tail=32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        n0 = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:n0],
                      "want": list(range(n0))}], "end": []})
        for i in range(n0, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if n0 == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 2, 5, 3, 2, 11, 2, 4)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            if len(toks) - i - n == 1:      # never leave a 1-token rest: portions are >= 2
                n += 1
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[i:i + n],
                          "want": list(range(n))}], "end": [rid] if i + n == len(toks) else []})
            i += n
    return steps


def mixed(requests, max_live=4, chunk_sizes=(7, 3, 9, 2, 5), decode_tail=6, seed=0):
    """Up to `max_live` requests at a time: portions of some beside single tokens of others.
    A request's last `decode_tail` tokens go one per step (as decoding does); requests wait
    in line and start when a place is free, so pages of finished ones are used again. Every
    few steps one live request sits a step out."""
    rng = np.random.RandomState(seed)
    waiting = list(requests.items())
    live = {}   # rid -> next index
    steps = []
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        skip = None
        if len(live) > 1 and len(steps) % 3 == 2:
            skip = list(live)[rng.randint(len(live))]
        for rid in list(live):
            if rid == skip:
                continue
            toks = requests[rid]
            i = live[rid]
            rest = len(toks) - i
            if rest <= decode_tail:
                n = 1
            else:
                n = min(chunk_sizes[k % len(chunk_sizes)], rest - decode_tail)
                k += 1
                if n < 2 <= rest - decode_tail:
                    n = 2
            entries.append({"id": rid, "tokens": toks[i:i + n], "want": list(range(n))})
            live[rid] = i + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def max_live_tokens(steps, requests, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of `round_to`."""
    held, worst = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst


def collect(steps, outputs):
    """steps + per-step logits arrays -> {(request id, position): logits row}."""
    res, seen = {}, {}
    for st, arr in zip(steps, outputs):
        r = 0
        for e in st["entries"]:
            base = seen.get(e["id"], 0)
            for w in e["want"]:
                res[(e["id"], base + w)] = arr[r]
                r += 1
            seen[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            seen.pop(rid, None)
    return res


def run_in_process(engine, steps):
    from rllm_b200.engine import Entry
    outs = []
    for st in steps:
        logits = None
        if st["entries"]:
            logits = engine.step([Entry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
        outs.append(None if logits is None else logits.float().cpu().numpy())
        engine.end(st["end"])
        engine.cache.check()
    return collect(steps, outs)


def run_program(model_dir, dtype, steps, out_dir, max_tokens, vocab, extra_args=(), env=None):
    """Through bin/trace_run, as a user would."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens), *extra_args]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env, timeout=1200)
    if p.returncode != 0:
        raise RuntimeError(f"trace_run exited {p.returncode}\nstdout:\n{p.stdout}\nstderr:\n{p.stderr}")
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], p.stdout
    outs = []
    for st in steps:
        n = sum(len(e["want"]) for e in st["entries"])
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if n == 0:
            assert not os.path.exists(path)
            outs.append(None)
        else:
            outs.append(np.fromfile(path, dtype="<f4").reshape(n, vocab))
    return collect(steps, outs)


def plain_logits(model_dir, requests):
    import plain_llama
    cfg, w = plain_llama.read_model_dir(model_dir)
    res = {}
    for rid, toks in requests.items():
        lg = plain_llama.forward(cfg, w, toks).numpy()
        for i in range(len(toks)):
            res[(rid, i)] = lg[i]
    return res


def compare(got, want, tol, what="", per_position=False):
    """Largest |difference| over all (request, position), relative to the largest |logit| of
    the plain implementation (of the whole set, or with `per_position` of that position alone, so
    that a position with small logits has to be as right as one with large ones); names the first
    place beyond `tol`."""
    assert set(got) == set(want), f"{what}: positions differ: {sorted(set(want) ^ set(got))[:5]}"
    scale = max(float(np.abs(v).max()) for v in want.values())
    worst, first_bad = 0.0, None
    for key in sorted(want, key=lambda k: (str(k[0]), k[1])):
        a, b = got[key], want[key]
        assert np.isfinite(a).all(), f"{what}: non-finite logits at {key}"
        err = float(np.abs(a - b).max()) / (float(np.abs(b).max()) if per_position else scale)
        if err > tol and first_bad is None:
            first_bad = (key, err)
        worst = max(worst, err)
    assert first_bad is None, (f"{what}: first wrong place {first_bad[0]} (request, position) "
                               f"error {first_bad[1]:.3e} > {tol:.1e}; worst {worst:.3e}")
    return worst
