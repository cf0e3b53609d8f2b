"""Times one kernel at a time at given sizes: the tool the launch choices (token tile, ranges of K,
ranges of keys) were tuned with, and the small case a profiler is pointed at.

    python -m rllm_b200.kernels.microbench gemm --shape gateup --tokens 1,8,64
    python -m rllm_b200.kernels.microbench gemm --n 3072 --k 2048 --epilogue store --tokens 2048
    python -m rllm_b200.kernels.microbench attn-decode --batch 64 --context 3000 --splits 1,2,3
    python -m rllm_b200.kernels.microbench attn-prefill --tokens 2048 --kernel tc
    python -m rllm_b200.kernels.microbench sample --rows 8 --top-p 0.9
    ... --plain 3      # no timing: three plain launches and a synchronize (for ncu -k ... -c ...)

Timing: the kernel runs back to back over `--copies` distinct weight (or cache) tensors, larger
together than the 126 MB L2, captured in a CUDA graph and replayed; CUDA events bracket five
replays. Back-to-back launches of one kernel overlap through programmatic dependent launch as
they do inside a decode step. Sizes default to the Llama 3.2 1B shapes.
"""
from __future__ import annotations

import argparse
import sys

import torch

from . import ops, sm100

DEV = "cuda:0"
SHAPES = {   # name -> (output features, inner size, epilogue)
    "qkv": (3072, 2048, "store"), "o": (2048, 2048, "accum"), "gateup": (8192, 2048, "swiglu"),
    "down": (2048, 8192, "accum"), "head": (128256, 2048, "store_f32"),
    "qkv-rope": (3072, 2048, "rope"),     # 32 + 2 x 8 heads of 64, rotated and written to a paged cache in the epilogue
}
EPI = {"store": ops.EPI_STORE, "store_f32": ops.EPI_STORE_F32, "accum": ops.EPI_ACCUM_F32,
       "swiglu": ops.EPI_SWIGLU}


def timed(fns, reps: int = 5) -> float:
    """Microseconds per call of the callables in `fns`, replayed as one CUDA graph."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def run(fns, plain: int, label: str, nbytes: float = 0.0, flops: float = 0.0) -> None:
    if plain:
        for _ in range(plain):
            fns[0]()
        torch.cuda.synchronize()
        print(f"{label}: {plain} plain launches done")
        return
    us = timed(fns)
    extra = ""
    if nbytes:
        extra += f"  {nbytes / us / 1e3:7.0f} GB/s"
    if flops:
        extra += f"  {flops / us / 1e6:7.1f} TFLOP/s"
    print(f"{label}: {us:8.2f} us{extra}", flush=True)


def cmd_gemm(a) -> None:
    if a.shape:
        N, K, epi_name = SHAPES[a.shape]
    else:
        N, K, epi_name = a.n, a.k, a.epilogue
    sm100.set_pairs(a.pairs)
    sm100.set_token_rows(not a.weight_rows)
    if epi_name == "rope":
        return cmd_gemm_rope(a, N, K)
    epi = EPI[epi_name]
    rows = 2 * N if epi == ops.EPI_SWIGLU else N
    copies = max(1, min(a.copies, int(2e9 // (rows * K * 2)) or 1))
    ws = [torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    split = a.ranges if a.ranges > 1 else not a.no_split      # a number: that many ranges of K (tcgen05 small tiles)
    for T in a.tokens:
        out = torch.zeros(T, N, device=DEV, dtype=torch.float32) if epi == ops.EPI_ACCUM_F32 else None
        if a.norm:
            h = torch.randn(T, K, device=DEV)
            g = torch.ones(K, device=DEV)
            fns = [(lambda w=w: sm100.gemm_norm(h, g, 1e-5, w, epi, split=split)) for w in ws]
        else:
            x = torch.randn(T, K, device=DEV, dtype=torch.bfloat16)
            fns = [(lambda w=w: sm100.gemm(x, w, epi, out=out, split=split)) for w in ws]
        bn, sp = sm100.plan(epi, T, N, K, split=split)
        run(fns, a.plain, f"gemm {epi_name} T={T} N={N} K={K} tile={bn} ranges={sp}" + (" norm" if a.norm else ""),
            nbytes=rows * K * 2, flops=2.0 * T * rows * K)
    sm100.check_error(DEV)


def cmd_gemm_rope(a, N: int, K: int) -> None:
    """The q/k/v product with rotation and cache write in its epilogue (heads of 64, a quarter of them k and v each)."""
    hd, page = 64, 16
    nkv = N // hd // 6
    nh = N // hd - 2 * nkv
    copies = max(1, min(a.copies, int(2e9 // (N * K * 2)) or 1))
    ws = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=DEV, dtype=torch.float32) / hd))).contiguous()
    for T in a.tokens:
        pages = (T + page - 1) // page
        kc = torch.zeros(pages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        pos = torch.arange(T, device=DEV, dtype=torch.int32)
        slots = torch.arange(T, device=DEV, dtype=torch.int32)
        table = ops.rope_table(pos, inv_freq, T)
        split = a.ranges if a.ranges > 1 else not a.no_split
        if a.norm:
            h = torch.randn(T, K, device=DEV)
            g = torch.ones(K, device=DEV)
            x, norm = None, (h, g, 1e-5)
        else:
            x, norm = torch.randn(T, K, device=DEV, dtype=torch.bfloat16), None
        fns = [(lambda w=w: sm100.gemm_qkv_rope(x, w, pos, inv_freq, slots, kc, vc, nh, nkv, hd, page, hd,
                                                split=split, table=table, norm=norm)) for w in ws]
        run(fns, a.plain, f"gemm qkv+rope T={T} N={N} K={K} heads {nh}/{nkv} of {hd}" + (" norm" if a.norm else "")
            + (f" ranges asked {a.ranges}" if a.ranges > 1 else ""), nbytes=N * K * 2, flops=2.0 * T * N * K)
    sm100.check_error(DEV)


def cmd_attn_decode(a) -> None:
    nh, nkv, hd, page = a.heads, a.kv_heads, a.head_dim, a.page
    pages_per = (a.context + page - 1) // page
    used = a.batch * pages_per
    npages = max(used, a.pool_pages)          # a pool larger than what the sequences hold spreads their pages
    per_copy = npages * nkv * page * hd * 2 * 2
    copies = max(1, min(a.copies, int(4e9 // per_copy) or 1))
    caches = [(torch.randn(npages, nkv, page, hd, device=DEV, dtype=torch.bfloat16),
               torch.randn(npages, nkv, page, hd, device=DEV, dtype=torch.bfloat16)) for _ in range(copies)]
    if a.page_order == "random":              # a sequence's pages anywhere in the pool
        order = torch.randperm(npages, device=DEV)[:used]
    elif a.page_order == "reversed":          # each sequence a run of neighbouring pages, falling
        order = torch.arange(used - 1, -1, -1, device=DEV)
    else:                                     # each sequence a run of neighbouring pages, rising
        order = torch.arange(used, device=DEV)
    bt = order.to(torch.int32).view(a.batch, pages_per).contiguous()
    lens = torch.full((a.batch,), a.context, dtype=torch.int32, device=DEV)
    q = torch.randn(a.batch, nh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    nbytes = a.batch * a.context * nkv * hd * 2 * 2
    auto = sm100.decode_splits(a.batch, nkv, a.context, sm100.init(DEV).sm_count)
    for sp in (a.splits or [auto]):
        fns = [(lambda kc=kc, vc=vc: sm100.attention_decode(q, kc, vc, lens, bt, nh, hd ** -0.5, None, a.context,
                                                            splits=sp, out=out)) for kc, vc in caches]
        run(fns, a.plain, f"attn-decode B={a.batch} ctx={a.context} hd={hd} page={page} pages {a.page_order} of {npages} "
            f"ranges={sp} (auto {auto})",
            nbytes=nbytes)


def cmd_attn_prefill(a) -> None:
    nh, nkv, hd, page = a.heads, a.kv_heads, a.head_dim, a.page
    T = a.tokens[0]
    pages_per = (T + page - 1) // page
    kc = torch.randn(pages_per, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn(pages_per, nkv, page, hd, device=DEV, dtype=torch.bfloat16)
    bt = torch.arange(pages_per, device=DEV, dtype=torch.int32).view(1, pages_per)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cu, lens = i32([0, T]), i32([T])
    q = torch.randn(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    if a.kernel == "tc":
        f = lambda: sm100.attention_prefill_tc(q, kc, vc, cu, lens, bt, T, nh, hd ** -0.5, None, out=out)
    else:
        f = lambda: sm100.attention_fa(q, kc, vc, cu, lens, bt, T, T, T, nh, hd ** -0.5, None, splits=1, out=out)
    run([f] * 4, a.plain, f"attn-prefill ({a.kernel}) T={T} heads={nh}/{nkv} hd={hd}",
        flops=4.0 * nh * hd * T * (T + 1) / 2)
    sm100.check_error(DEV)


def cmd_sample(a) -> None:
    R, V = a.rows, a.vocab
    logits = torch.randn(R, V, device=DEV) * 3
    vec = lambda v, dt=torch.float32: torch.full((R,), v, dtype=dt, device=DEV)
    u = torch.rand(R, device=DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    if a.temperature <= 0:
        f = lambda: ops.argmax(logits, out=out)
        what = "argmax"
    else:
        kw = dict(top_k=vec(a.top_k, torch.int32) if a.top_k > 0 else None, top_p=vec(a.top_p) if a.top_p < 1 else None,
                  min_p=vec(a.min_p) if a.min_p > 0 else None)
        temp = vec(a.temperature)
        f = lambda: ops.sample(logits, temp, u, out=out, **kw)
        what = f"temperature {a.temperature} top-k {a.top_k} top-p {a.top_p} min-p {a.min_p}"
    run([f] * 4, a.plain, f"sample rows={R} vocab={V} {what}", nbytes=R * V * 4)


def main(argv=None) -> int:
    ints = lambda s: [int(x) for x in s.split(",")]
    ap = argparse.ArgumentParser(prog="python -m rllm_b200.kernels.microbench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("sample")
    p.add_argument("--plain", type=int, default=0, help="N plain launches instead of timing")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--temperature", type=float, default=0.8, help="0: the argmax kernel")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0)
    for name in ("gemm", "attn-decode", "attn-prefill"):
        p = sub.add_parser(name)
        p.add_argument("--plain", type=int, default=0, help="N plain launches instead of timing")
        p.add_argument("--copies", type=int, default=8, help="distinct weight / cache tensors to cycle through")
        if name == "gemm":
            p.add_argument("--shape", choices=sorted(SHAPES))
            p.add_argument("--n", type=int, default=2048)
            p.add_argument("--k", type=int, default=2048)
            p.add_argument("--epilogue", choices=sorted(EPI), default="store")
            p.add_argument("--tokens", type=ints, default=[1, 8, 64, 2048])
            p.add_argument("--norm", action="store_true", help="RMSNorm in front, in the same kernel")
            p.add_argument("--no-split", action="store_true")
            p.add_argument("--weight-rows", action="store_true",
                           help="gate/up of long portions with the weight rows on the accumulator's rows (default: the tokens)")
            p.add_argument("--pairs", action="store_true", help="long portions on pairs of CTAs (tcgen05.mma.cta_group::2)")
            p.add_argument("--ranges", type=int, default=0, help="ranges of K to force on the tcgen05 small-tile kernel")
        else:
            p.add_argument("--heads", type=int, default=32)
            p.add_argument("--kv-heads", type=int, default=8)
            p.add_argument("--head-dim", type=int, default=64)
            p.add_argument("--page", type=int, default=16)
            if name == "attn-decode":
                p.add_argument("--batch", type=int, default=8)
                p.add_argument("--context", type=int, default=3000)
                p.add_argument("--splits", type=ints, default=None)
                p.add_argument("--page-order", choices=["random", "rising", "reversed"], default="random")
                p.add_argument("--pool-pages", type=int, default=0, help="pages of the pool (at least what the sequences hold)")
            else:
                p.add_argument("--tokens", type=ints, default=[2048])
                p.add_argument("--kernel", choices=["tc", "fa"], default="tc",
                               help="tc: tcgen05 kernel (head sizes 64 and 128); fa: mma.sync kernel")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench: no CUDA device", file=sys.stderr)
        return 1
    {"gemm": cmd_gemm, "attn-decode": cmd_attn_decode, "attn-prefill": cmd_attn_prefill, "sample": cmd_sample}[a.cmd](a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
