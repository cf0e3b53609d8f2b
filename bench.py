#!/usr/bin/env python3
"""Decode and prefill throughput of Llama 3.2 1B (random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line. `value`: decoded tokens per second at batch 8 with the context at
4,096 tokens when the timed steps end, timed on the device with CUDA events around K decode
steps (a "step" is one decode step of the whole batch). `e2e`: the same through the Python
entry point (`LLM.add_request` / `LLM.step`), host token ids in, host token ids out, every
step copying its inputs from pinned host memory and reading its tokens back. `prefill`: one
2,048-token prompt in one step. `roofline`: bytes the decode step has to read (every weight
once, and the cache of the live requests) over its time, against the measured copy
bandwidth. `points`: decode at batch 1 and 64 (`points_frac`: their roofline fractions);
`e2e_points`: the same two through the entry point, with the share of the time the host was
busy. Between timed steps nothing is flushed: one step reads 2.47 GB of weights, twenty times
the 126 MB L2. Each decode loop idles for `settle_s` between its prompts' prefill and its warm-up
steps (see `settle()`).

`--workloads mixed_3b,continuous_8b` (or `all`) adds, under `workloads`, the two serving runs the
larger model shapes are quoted for: 32 requests with prompts of 128 to 4,096 tokens and 256 decoded
tokens each at the 3B shape; 64 requests that reach 8,192 tokens of context, prompts cut into
portions of 512, at the 8B shape. Each goes through `LLM.add_request` / `LLM.step` (scheduler, mixed
steps, graphs where a step is all decoding) and reports tokens a second, steps, mean step time,
preemptions, the host's share, and the bytes and FLOPs the steps had to move and do against the
measured peaks. They take some twenty seconds each and are off in the default run.
This engine runs on one GPU: for --gpus N > 1 it says so and exits with 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {   # BASELINE.json configs[2]
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 8192, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
}
# The other two sizes the reference's benchmarks name, for `--model 3b|8b` (not the default run)
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8,
                head_dim=128, intermediate_size=8192)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
MODELS = {"1b": ("llama-3.2-1b-shape", "Llama 3.2 1B", LLAMA_1B), "3b": ("llama-3.2-3b-shape", "Llama 3.2 3B", LLAMA_3B),
          "8b": ("llama-3.1-8b-shape", "Llama 3.1 8B", LLAMA_8B)}
CONTEXT = 4096
PROMPT = 2048
PAGE = 16
SETTLE_S = 0.25     # idle time between a loop's prompts and its decode steps
# name -> (model, requests, shortest and longest prompt, decoded tokens each, portion, token budget a step)
WORKLOADS = {"mixed_3b": ("3b", 32, 128, 4096, 256, None, 4096),
             "continuous_8b": ("8b", 64, 8192 - 256, 8192 - 256, 256, 512, 2048)}


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            m = json.load(f)
        p.update({k: m[k] for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in m})
        p["source"] = "measured"
    return p


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, windows):
        if self.proc is not None:
            self.proc.terminate()
        rows = [r for t, r in self.rows if any(a <= t <= b for a, b in windows)] or [r for _, r in self.rows]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(rows)}


def weight_bytes(model):
    seen, total = set(), 0
    for part in model.parts():
        for p in part.params():
            t = getattr(part, p.attr)
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def prefill_flops(cfg, T):
    H, L, Q = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"] * cfg["head_dim"]
    KV, I, V = cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    linear = 2 * T * L * (H * (Q + 2 * KV) + Q * H + 3 * H * I)
    attn = L * 4 * Q * T * (T + 1) // 2          # QK^T and PV over the causal half
    return linear + attn + 2 * H * V             # logits for the last row only


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="1b", choices=sorted(MODELS), help="layer sizes (default: the 1B shape)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers where memory or time needs it")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--workloads", default="", help="comma-separated: mixed_3b, continuous_8b, or all")
    ap.add_argument("--phase", default="all", choices=["all", "prefill", "decode"],
                    help="run one part only (for profiling; the JSON line then lacks the other parts)")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket one timed step with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (Cargo.toml); no cargo/rustc in this image and no "
                          "network, so pip cannot build or install it"}))
        return 0
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    W, K = max(a.warmup, 3), a.steps

    import torch
    from rllm_b200.api import LLM
    from rllm_b200.engine import Entry
    from rllm_b200.kernels import ops
    from rllm_b200.sampling import SamplingParams

    pk = peaks()
    model_name, model_title, full_cfg = MODELS[a.model]
    full_layers = full_cfg["num_hidden_layers"]
    a.layers = a.layers or full_layers
    cfg = dict(full_cfg, num_hidden_layers=a.layers)
    # the headline batch is measured first, right after the prefill, the other two points after it
    batches = [a.batch] if a.no_points else [a.batch] + [b for b in (1, 64) if b != a.batch]
    pages = max(batches) * (CONTEXT // PAGE + 1) + 64
    llm = LLM(cfg, dtype="bfloat16", seed=0, page_size=PAGE, num_pages=pages, max_active=max(batches),
              max_tokens_per_step=8192)
    eng = llm.engine
    wbytes = weight_bytes(eng.model)
    kv_bytes_per_token = sum(2 * s.kv_heads * s.head_dim * 2 for s in eng.model.cache_specs())
    g = torch.Generator().manual_seed(0)
    rand_ids = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler()
    sampler.start()
    windows = []

    # ---------------------------------------------------------------- prefill, 2,048 tokens
    prompt = rand_ids(PROMPT)
    times = []
    for i in range(W + 5 if a.phase != "decode" else 0):
        torch.cuda.synchronize()
        t0, t1 = ev(), ev()
        w0 = time.time()
        t0.record()
        prof = a.profile_range and i == W
        if prof:
            torch.cuda.profiler.start()
        eng.step([Entry(f"p{i}", prompt, [PROMPT - 1])])
        if prof:
            torch.cuda.profiler.stop()
        t1.record()
        torch.cuda.synchronize()
        if i >= W:
            times.append(t0.elapsed_time(t1))
            windows.append((w0, time.time()))
        eng.end([f"p{i}"])
    pre_ms = statistics.median(times) if times else float("nan")
    pre_flops = prefill_flops(cfg, PROMPT)
    prefill = {"value": round(PROMPT / pre_ms * 1e3, 1), "tokens": PROMPT, "ms": round(pre_ms, 4),
               "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(pre_flops / (pre_ms * 1e-3) / 1e12, 1)}

    # ---------------------------------------------------------------- decode on the device
    def fill(B, start_ctx):
        ids = [f"d{B}_{i}" for i in range(B)]
        for rid in ids:
            left = start_ctx
            while left:
                n = min(left, 2048)
                eng.step([Entry(rid, rand_ids(n), [])])
                left -= n
        return ids

    def settle():
        # The prompts' prefill is a burst at the power cap, and decode steps that follow it without a gap run
        # 3 to 5 % slower for as long as the GPU stays busy (lower clocks; measured: 0.78 ms a step right behind
        # the prefill, 0.75 ms after 50 ms of idling or more). Which of the two a loop got used to depend on
        # whether a graph capture happened to lie between its prefill and its steps, so both loops idle here.
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)

    def decode_device(B):
        start_ctx = CONTEXT - (W + K)
        ids = fill(B, start_ctx)
        settle()
        toks = rand_ids(B)
        launches0 = None

        # Each step's token ids are the ones the step before drew, handed over on the device (the
        # way `LLM.step` launches a step ahead): the timed steps run back to back, no host in between.
        placeholders = [Entry(r, [0], [0]) for r in ids]

        def one(toks):
            logits = eng.step(placeholders, keep=False, feed=toks)
            return eng.backend.argmax(logits)
        toks = one(torch.tensor(toks, dtype=torch.int32, device=eng.device))
        for _ in range(W - 1):
            toks = one(toks)
        torch.cuda.synchronize()
        launches0 = ops.LAUNCHES
        t0, t1 = ev(), ev()
        w0 = time.time()
        t0.record()
        for k in range(K):
            prof = a.profile_range and k == 0 and B == a.batch
            if prof:
                torch.cuda.profiler.start()
            toks = one(toks)
            if prof:
                torch.cuda.profiler.stop()
        t1.record()
        torch.cuda.synchronize()
        windows.append((w0, time.time()))
        ms = t0.elapsed_time(t1) / K
        launches = ops.LAUNCHES - launches0
        ctx_mean = start_ctx + W + (K + 1) / 2
        eng.end(ids)
        return ms, launches, ctx_mean

    if a.phase == "prefill":
        print(json.dumps({"impl": "ours", "phase": "prefill", "prefill": prefill}))
        sampler.stop(windows)
        return 0

    # ---------------------------------------------------------------- end to end, host in/out
    def decode_e2e(B):
        # Prompts are admitted over a few steps (the token budget holds two of them), so the
        # requests get a few tokens of slack: nobody finishes, and the batch keeps its size,
        # until the timed steps are over. What is left is aborted.
        slack = B + 9
        start_ctx = CONTEXT - (W + K) - slack
        sp = SamplingParams(temperature=0.0, max_tokens=W + K + 2 * slack, ignore_eos=True)
        rids = [llm.add_request(rand_ids(start_ctx), sp) for _ in range(B)]
        made = {r: 0 for r in rids}

        def steps_until(n):
            while min(made.values()) < n:
                for o in llm.step():
                    if o.token is not None:
                        made[o.request_id] += 1
        steps_until(1)                            # the prompts
        settle()
        steps_until(1 + W)                        # warm-up decode steps of the whole batch
        torch.cuda.synchronize()
        h2d0 = eng.h2d_bytes
        llm.stats.reset()
        w0 = time.time()
        n = 0
        for _ in range(K):
            n += sum(o.token is not None for o in llm.step())
        torch.cuda.synchronize()
        dt = time.time() - w0
        e2e_h2d[B] = (eng.h2d_bytes - h2d0) / K
        e2e_host[B] = llm.stats.host_share
        e2e_plan[B] = (llm.stats.host_plan_s + llm.stats.host_record_s) / llm.stats.wall_s
        windows.append((w0, time.time()))
        assert n == B * K, "the batch changed size inside the timed steps"
        for r in rids:
            llm.abort(r)
        while llm.has_work():
            llm.step()
        return n / dt
    # A batch size's two measurements stand side by side, the headline batch first, and of the two the entry
    # point (the end-to-end figure is the one a user gets) before the device loop.
    e2e_h2d, e2e_host, e2e_plan = {}, {}, {}
    results, e2e_all, graph_replays = {}, {}, 0
    for B in batches:
        if a.phase == "all":
            e2e_all[B] = decode_e2e(B)
        replays0 = eng.graph_steps
        results[B] = decode_device(B)
        graph_replays += eng.graph_steps - replays0          # of the device loops, warm-up included
    ms, launches, ctx_mean = results[a.batch]
    step_bytes = wbytes + a.batch * ctx_mean * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9
    e2e_value = e2e_all.get(a.batch, float("nan"))
    e2e_points = {B: v for B, v in e2e_all.items() if B != a.batch}

    # ---------------------------------------------------------------- serving workloads (opt-in)
    def linear_flops_per_token(c):
        H, L, Q = c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"] * c["head_dim"]
        KV, I = c["num_key_value_heads"] * c["head_dim"], c["intermediate_size"]
        return 2 * L * (H * (Q + 2 * KV) + Q * H + 3 * H * I)

    def run_workload(name):
        mkey, n_req, lo, hi, n_new, chunk, budget = WORKLOADS[name]
        wname, _, wcfg = MODELS[mkey]
        rng = torch.Generator().manual_seed(1234)
        lens = torch.randint(lo, hi + 1, (n_req,), generator=rng).tolist()
        pages_w = sum((n + n_new) // PAGE + 2 for n in lens) + 64
        wl = LLM(wcfg, dtype="bfloat16", seed=0, page_size=PAGE, num_pages=pages_w, max_active=n_req,
                 max_tokens_per_step=budget, max_chunk=chunk)
        wl.warm_up(min(2048, budget))
        wb = weight_bytes(wl.engine.model)
        kvb = sum(2 * sp.kv_heads * sp.head_dim * 2 for sp in wl.engine.model.cache_specs())
        sp = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True)
        prompts = [torch.randint(0, wcfg["vocab_size"], (n,), generator=rng).tolist() for n in lens]
        torch.cuda.synchronize()
        wl.stats.reset()
        graphs0 = wl.engine.graph_steps
        w0 = time.time()
        for pr in prompts:
            wl.add_request(pr, sp)
        done = 0
        while wl.has_work():
            done += sum(o.token is not None for o in wl.step())
        torch.cuda.synchronize()
        dt = time.time() - w0
        windows.append((w0, time.time()))
        st = wl.stats
        assert done == n_req * n_new, f"{name}: {done} tokens drawn, {n_req * n_new} expected"
        nbytes = st.steps * wb + st.kv_positions * kvb
        flops = st.tokens * linear_flops_per_token(wcfg) + 4 * wcfg["num_hidden_layers"] * wcfg["num_attention_heads"] \
            * wcfg["head_dim"] * st.attn_pairs + 2 * wcfg["hidden_size"] * wcfg["vocab_size"] * st.sampled
        res = {"model": wname, "requests": n_req, "prompt_tokens": sum(lens), "decode_tokens": done,
               "portion": chunk, "token_budget": budget,
               "decode_tok_s": round(done / dt, 1), "all_tok_s": round(st.tokens / dt, 1), "seconds": round(dt, 3),
               "steps": st.steps, "graph_steps": wl.engine.graph_steps - graphs0, "mean_step_ms": round(dt / st.steps * 1e3, 3),
               "preemptions": st.preemptions, "host_share": round(st.host_share, 4),
               "host_plan_share": round(st.host_plan_s / st.wall_s, 4), "host_launch_share": round(st.host_launch_s / st.wall_s, 4),
               "host_record_share": round(st.host_record_s / st.wall_s, 4), "host_wait_share": round(st.wait_s / st.wall_s, 4),
               "device_busy": round(st.device_s / st.wall_s, 4),
               "hbm_frac": round(nbytes / dt / 1e9 / pk["hbm_gbs"], 4),
               "flop_frac": round(flops / dt / 1e12 / pk["bf16_tflops_sustained"], 4)}
        res["bound"] = "hbm" if res["hbm_frac"] >= res["flop_frac"] else "tensor"
        del wl
        torch.cuda.empty_cache()
        return res

    wanted = [w for w in (sorted(WORKLOADS) if a.workloads == "all" else a.workloads.split(",")) if w]
    for w in wanted:
        if w not in WORKLOADS:
            print(f"bench.py: unknown workload {w!r} (known: {sorted(WORKLOADS)})", file=sys.stderr)
            return 2
    workloads = {}
    if wanted:
        del llm, eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for w in wanted:
            workloads[w] = run_workload(w)
    clocks = sampler.stop(windows)

    out = {
        "metric": f"decode tok/s at batch {a.batch} ({model_title}, bf16, context {CONTEXT})",
        "value": round(a.batch / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random token ids, random weights N(0,0.02))",
        "impl": "ours",
        "config": {"model": model_name, "layers": a.layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": a.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "kv_page": PAGE, "settle_s": SETTLE_S, "parallelism": "single-gpu",
                   "l2": f"step reads {wbytes / 1e9:.1f} GB > 126 MB L2, no flush",
                   "peaks": pk["source"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s",
                "h2d_bytes_per_step": round(e2e_h2d[a.batch]) if a.batch in e2e_h2d else None,
                "d2h_bytes_per_step": 4 * a.batch, "steps": K, "host_share": round(e2e_host.get(a.batch, float("nan")), 4),
                "host_plan_record_share": round(e2e_plan.get(a.batch, float("nan")), 4)},
        "e2e_points": {f"decode_b{B}": {"value": round(v, 1), "h2d_bytes_per_step": round(e2e_h2d[B]),
                                        "d2h_bytes_per_step": 4 * B, "host_share": round(e2e_host[B], 4),
                                        "host_plan_record_share": round(e2e_plan[B], 4)}
                       for B, v in e2e_points.items()},
        "gpu_launches": launches, "graph_replays": graph_replays,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": {f"decode_b{B}": round(B / results[B][0] * 1e3, 1) for B in batches if B != a.batch},
        # the same roofline fraction (bytes the step has to read / its time / the copy bandwidth) per point
        "points_frac": {f"decode_b{B}": round((wbytes + B * results[B][2] * kv_bytes_per_token)
                                              / (results[B][0] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                        for B in batches if B != a.batch},
        "published": {"h100_nvl_b1_tok_s": 326, "note": "reference README, other hardware, batch 1"} if a.model == "1b" else None,
        "clocks": clocks,
    }
    if workloads:
        out["workloads"] = workloads
    if 1 in results:
        out["points"]["decode_b1"] = round(1 / results[1][0] * 1e3, 1)
        out["points_frac"]["decode_b1"] = round((wbytes + results[1][2] * kv_bytes_per_token)
                                                / (results[1][0] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
