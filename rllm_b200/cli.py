"""Command line in the reference's manner: `rllm run`, `rllm batch`, `rllm bench`, with the
reference's option names, meanings and defaults (src/commands/mod.rs:75-131, run.rs:20-22,
batch.rs:21-23, bench.rs:37-39). Options of parts that are not built (--chat, --system, --tp,
--stream-experts, --image, --kv-quant other than none) are accepted and refused with a
clear message. Added here: --prompt-ids (token ids instead of text), --dtype, --seed,
--page-size, --kv-pages, --random-weights (a configuration folder without weights).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _model_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True,
                   help="Path to model directory (contains config.json, tokenizer.json, *.safetensors).")
    p.add_argument("--max-tokens", type=int, default=128, help="Maximum number of tokens to generate.")
    p.add_argument("--temperature", type=float, default=1.0,
                   help="Sampling temperature. T=0 -> greedy (deterministic). Default 1.0.")
    p.add_argument("--top-p", type=float, default=0.9, help="Top-p (nucleus) sampling threshold. Default 0.9.")
    p.add_argument("--top-k", type=int, default=0, help="Keep only the k highest-scoring tokens; 0 = off.")
    p.add_argument("--min-p", type=float, default=0.0, help="Discard tokens with prob < min_p * max prob.")
    p.add_argument("--chat", action="store_true", help="(not built) chat template mode")
    p.add_argument("--system", default=None, help="(not built) system prompt for chat mode")
    p.add_argument("--tp", type=int, default=0, help="Tensor parallelism; this engine runs on one GPU (0 or 1).")
    p.add_argument("--stream-experts", action="store_true", help="(not built) MoE expert streaming")
    p.add_argument("--image", default=None, help="(not built) image input")
    p.add_argument("--kv-quant", default="none", help='KV cache quantization; only "none" is built.')
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--seed", type=int, default=None, help="Seed of the sampling random numbers.")
    p.add_argument("--page-size", type=int, default=16, help="Positions per cache page (reference: 16).")
    p.add_argument("--kv-pages", type=int, default=None, help="Pages in the cache pool (default: from free memory).")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="Ignore *.safetensors; draw random weights from SEED for the folder's config.json.")


def _refuse_unbuilt(a) -> None:
    bad = []
    if a.chat or a.system is not None:
        bad.append("--chat/--system (chat templates)")
    if a.tp not in (0, 1):
        bad.append("--tp > 1 (several GPUs)")
    if a.stream_experts:
        bad.append("--stream-experts")
    if a.image:
        bad.append("--image")
    if a.kv_quant != "none":
        bad.append(f"--kv-quant {a.kv_quant} (only 'none')")
    if bad:
        sys.exit("rllm: not built in this engine: " + "; ".join(bad))


def _load(a, max_active: int):
    from .api import LLM
    model = a.model
    if a.random_weights is not None:
        with open(os.path.join(a.model, "config.json")) as f:
            model = json.load(f)
    t0 = time.time()
    llm = LLM(model, dtype=a.dtype, seed=a.random_weights or 0, page_size=a.page_size,
              num_pages=a.kv_pages, max_active=max_active)
    if a.random_weights is None:
        llm.model_dir = a.model
    llm.warm_up()          # modules loaded, a first graph captured: the first request is not the slow one
    print(f"[rllm] model loaded in {time.time() - t0:.1f}s", file=sys.stderr)
    if not getattr(llm.engine.model.config, "eos_token_ids", ()):
        print("[rllm] the model folder names no end-of-sequence id (config.json / generation_config.json): "
              "generations run to --max-tokens", file=sys.stderr)
    return llm


def _params(a):
    from .sampling import SamplingParams
    return SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p,
                          max_tokens=a.max_tokens, seed=a.seed)


def _encode(llm, text: str | None, ids: str | None) -> list[int]:
    if ids is not None:
        return [int(x) for x in ids.replace(",", " ").split()]
    # the text's tokens without the tokenizer's own special tokens, the model's BOS in front exactly
    # once where it has one (src/model/tokenizer.rs:123-140)
    toks = llm.tokenizer().encode(text, add_special_tokens=False).ids
    bos = getattr(llm.engine.model.config, "bos_token_id", None)
    return ([bos] if bos is not None else []) + toks


def _show(llm, tokens: list[int], as_ids: bool) -> str:
    return " ".join(map(str, tokens)) if as_ids else llm.tokenizer().decode(tokens)


def cmd_run(a) -> int:
    """One prompt, streamed; logs prefill and generation tok/s as the reference does
    (src/commands/run.rs:82-119: prefill = prompt length / time to first token)."""
    _refuse_unbuilt(a)
    if (a.prompt is None) == (a.prompt_ids is None):
        sys.exit("rllm run: give exactly one of --prompt and --prompt-ids")
    llm = _load(a, 1)
    prompt = _encode(llm, a.prompt, a.prompt_ids)
    as_ids = a.prompt_ids is not None
    import torch
    llm.stats.reset()
    rid = llm.add_request(prompt, _params(a))
    t0 = time.time(); first = None; n = 0
    produced, shown = [], ""
    while llm.has_work():
        for out in llm.step():
            if out.token is None:
                print(f"\n[rllm] request ended: {out.finish_reason}", file=sys.stderr)
                continue
            if first is None:
                torch.cuda.synchronize(); first = time.time()
            n += 1
            if as_ids:
                sys.stdout.write(str(out.token) + " ")
            else:
                # the whole output decoded again, its new end printed: a character whose bytes are
                # spread over several tokens appears when its last token has come
                produced.append(out.token)
                text = llm.tokenizer().decode(produced)
                if not text.endswith("\ufffd") or out.finished:
                    sys.stdout.write(text[len(shown):])
                    shown = text
            sys.stdout.flush()
    torch.cuda.synchronize(); t1 = time.time()
    print()
    if first is not None:
        print(f"[rllm] prefill: {len(prompt)} tokens in {(first - t0) * 1e3:.1f} ms "
              f"({len(prompt) / max(first - t0, 1e-9):.1f} tok/s); generation: {n} tokens in "
              f"{(t1 - t0) * 1e3:.1f} ms ({n / max(t1 - t0, 1e-9):.1f} tok/s)", file=sys.stderr)
    print(f"[rllm] {llm.stats.line()}", file=sys.stderr)
    if hasattr(llm.engine.backend, "report"):
        llm.engine.backend.report()              # RLLM_B200_PROFILE=1: what is left since the last table
    return 0


def cmd_batch(a) -> int:
    """A file of prompts, one per line, all concurrent (src/commands/batch.rs:26-90)."""
    _refuse_unbuilt(a)
    with open(a.batch_file) as f:
        lines = [l.strip() for l in f if l.strip()]
    if not lines:
        sys.exit("rllm batch: the batch file is empty")
    llm = _load(a, len(lines))
    prompts = [_encode(llm, None if a.ids else l, l if a.ids else None) for l in lines]
    import torch
    t0 = time.time()
    outs = llm.generate(prompts, _params(a))
    torch.cuda.synchronize(); dt = time.time() - t0
    for i, o in enumerate(outs):
        print(f"[{i}] {_show(llm, o, a.ids)}")
    total = sum(len(o) for o in outs)
    print(f"[rllm] {len(outs)} prompts, {total} tokens in {dt:.2f}s ({total / dt:.1f} tok/s)", file=sys.stderr)
    return 0


def cmd_bench(a) -> int:
    """Throughput on synthetic prompts of random token ids (the reference's `bench` measures
    time to first token with and without its prefix cache, src/commands/bench.rs:52-195; this
    engine has no prefix cache, so it reports time to first token and tok/s per request)."""
    _refuse_unbuilt(a)
    n = max(1, min(a.prompts, 64))
    llm = _load(a, n)
    import torch
    vocab = llm.engine.vocab
    g = torch.Generator().manual_seed(a.seed or 0)
    prompts = [torch.randint(0, vocab, (a.prompt_len,), generator=g).tolist() for _ in range(n)]
    from dataclasses import replace
    sp = replace(_params(a), ignore_eos=True)
    ids = [llm.add_request(p, sp) for p in prompts]
    t0 = time.time(); ttft = {}; count = 0
    while llm.has_work():
        outs = llm.step()
        torch.cuda.synchronize()
        for o in outs:
            if o.token is not None:
                count += 1
                ttft.setdefault(o.request_id, time.time() - t0)
    dt = time.time() - t0
    print(json.dumps({"prompts": n, "prompt_len": a.prompt_len, "generated": count,
                      "seconds": round(dt, 4), "tok_per_s": round(count / dt, 1),
                      "ttft_ms_mean": round(1e3 * sum(ttft.values()) / max(len(ttft), 1), 2)}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rllm", description="rllm_b200: inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    r = sub.add_parser("run", help="stream one completion")
    _model_args(r)
    r.add_argument("--prompt", default=None, help="Prompt text to complete.")
    r.add_argument("--prompt-ids", default=None, help="Prompt as token ids (space or comma separated).")
    r.set_defaults(fn=cmd_run)
    b = sub.add_parser("batch", help="a file of prompts, all concurrent")
    _model_args(b)
    b.add_argument("--batch-file", required=True, help="File with one prompt per line.")
    b.add_argument("--ids", action="store_true", help="Lines are token ids, output is token ids.")
    b.set_defaults(fn=cmd_batch)
    c = sub.add_parser("bench", help="throughput on synthetic prompts")
    _model_args(c)
    c.add_argument("--prompts", type=int, default=3, help="Number of prompts to run. Default 3.")
    c.add_argument("--prompt-len", type=int, default=128, help="Tokens per synthetic prompt.")
    c.set_defaults(fn=cmd_bench)
    for name in ("serve", "quantize"):
        x = sub.add_parser(name, help="(not built in this engine)")
        x.set_defaults(fn=lambda a, name=name: sys.exit(f"rllm {name}: not built in this engine"))
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
