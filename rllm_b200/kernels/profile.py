"""Per-operation timing of the launch-by-launch path, switched on with RLLM_B200_PROFILE=1.

Every backend operation (embedding, norm, the q/k/v product with rotation and cache write,
attention, the output, gate/up and down products, the head, sampling) is bracketed by a pair of
CUDA events on the launching stream; the pairs are read when a report is asked for, so that no
operation waits for a measurement. With the switch on, decode steps do not replay CUDA graphs
(events cannot sit inside a replayed graph), so the step times are those of the launch-by-launch
path: the shares say where a step's time goes, the absolute times are not the serving path's.
A report lists, per class, calls, mean microseconds, the bytes and FLOPs the operation has to move
and do (counted from its operands' shapes) and what fraction of the measured copy bandwidth or
tensor throughput that is.

The counterpart of the reference's RLLM_PROFILE timers (src/model/profile.rs:19-100, call sites
src/model/registry/llama.rs:159-258), which bracket the same classes with a device synchronize.
"""
from __future__ import annotations

import json
import os
import sys
from collections import OrderedDict

import torch


def enabled() -> bool:
    return os.environ.get("RLLM_B200_PROFILE") == "1"


def _peaks() -> tuple[float, float]:
    """(copy bandwidth in bytes/s, bf16 tensor throughput in FLOP/s): the measured ones if the file
    with them lies beside the package, else the nominal 7.7 TB/s and 2.25 PFLOP/s."""
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
        return m["hbm_gbs"] * 1e9, m["bf16_tflops"] * 1e12
    except (OSError, KeyError, ValueError):
        return 7.7e12, 2.25e15


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


class OpProfile:
    """Wraps a `Backend`: the same methods, each timed under a class name."""

    # backend method -> (class name, function of (args, kwargs, result) -> (bytes, flops))
    def __init__(self, backend):
        self._be = backend
        self.classes: OrderedDict[str, list] = OrderedDict()     # name -> [calls, bytes, flops, [event pairs]]
        self._free: list = []
        self.tokens = 0

    def __getattr__(self, name):
        return getattr(self._be, name)

    # ---- bookkeeping
    def _timed(self, cls: str, nbytes: int, flops: int, fn, *a, **k):
        if torch.cuda.is_current_stream_capturing():
            return fn(*a, **k)
        e0, e1 = self._free.pop() if self._free else (torch.cuda.Event(enable_timing=True),
                                                      torch.cuda.Event(enable_timing=True))
        e0.record()
        out = fn(*a, **k)
        e1.record()
        rec = self.classes.setdefault(cls, [0, 0, 0, [], 0.0])
        rec[0] += 1; rec[1] += nbytes; rec[2] += flops; rec[3].append((e0, e1))
        return out

    def _settle(self) -> None:
        torch.cuda.synchronize(self._be.device)
        for rec in self.classes.values():
            for e0, e1 in rec[3]:
                rec[4] += e0.elapsed_time(e1) * 1e3           # microseconds
                self._free.append((e0, e1))
            rec[3] = []

    def report(self, file=None, reset: bool = True) -> dict:
        """Print the table (to stderr by default) and return it as a dict."""
        self._settle()
        bw, tf = _peaks()
        total = sum(r[4] for r in self.classes.values()) or 1.0
        out = {}
        lines = [f"[rllm profile] {'class':<12}{'calls':>8}{'mean us':>10}{'share':>8}{'GB/s':>9}{'of copy':>9}"
                 f"{'TFLOP/s':>9}{'of peak':>9}"]
        for name, (calls, nbytes, flops, _, us) in self.classes.items():
            if not calls:
                continue
            sec = us * 1e-6
            gbs, tfl = nbytes / sec / 1e9 if sec else 0.0, flops / sec / 1e12 if sec else 0.0
            out[name] = {"calls": calls, "mean_us": us / calls, "share": us / total, "gbs": gbs, "hbm_frac": gbs * 1e9 / bw,
                         "tflops": tfl, "tensor_frac": tfl * 1e12 / tf}
            lines.append(f"[rllm profile] {name:<12}{calls:>8}{us / calls:>10.1f}{us / total:>8.1%}{gbs:>9.0f}"
                         f"{gbs * 1e9 / bw:>9.2f}{tfl:>9.1f}{tfl * 1e12 / tf:>9.3f}")
        print("\n".join(lines), file=file or sys.stderr, flush=True)
        if reset:
            self.classes.clear()
        return out

    # ---- the backend's operations
    def embed(self, ids, table, err=None):
        return self._timed("embed", ids.numel() * table.shape[1] * (table.element_size() + 4), 0,
                           self._be.embed, ids, table, err=err)

    def rmsnorm(self, x, w, eps, out_dtype=None, rows=None):
        T = x.shape[0] if rows is None else rows.numel()
        return self._timed("norm", T * x.shape[1] * 6, 0, self._be.rmsnorm, x, w, eps, out_dtype, rows)

    def _product(self, cls, x, w, fn, *a, **k):
        T = x.shape[0]
        return self._timed(cls, _nbytes(w) + T * (w.shape[0] + w.shape[1]) * 2, 2 * T * w.shape[0] * w.shape[1],
                           fn, *a, **k)

    def linear(self, x, w, bias=None):
        return self._product("linear", x, w, self._be.linear, x, w, bias=bias)

    def linear_f32(self, x, w):
        return self._product("head", x, w, self._be.linear_f32, x, w)

    def linear_residual(self, x, w, residual):
        cls = "o" if w.shape[0] >= w.shape[1] else "down"       # a square or widening product: the mixer's output
        return self._product(cls, x, w, self._be.linear_residual, x, w, residual)

    def linear_swiglu(self, x, w_gate_up):
        return self._product("gate_up", x, w_gate_up, self._be.linear_swiglu, x, w_gate_up)

    def qkv_rope_cache_write(self, x, w_qkv, *a, **k):
        return self._product("qkv+rope", x, w_qkv, self._be.qkv_rope_cache_write, x, w_qkv, *a, **k)

    def rope_cache_write(self, qkv, *a, **k):
        return self._timed("rope", 2 * _nbytes(qkv), 0, self._be.rope_cache_write, qkv, *a, **k)

    def attention(self, q, cache, ctx, nh, scale, window):
        hd = q.shape[1] // nh
        nkv = cache.k.shape[1] if cache.k is not None else nh
        lens, qs = ctx.kv_lens_host, ctx.q_lens_host
        if lens is None:
            lens, qs = [ctx.max_kv_len] * ctx.num_seqs, [1] * ctx.num_seqs
        seen = [min(L, window + q - 1) if window else L for L, q in zip(lens, qs)]
        pairs = sum(q * (s - q) + q * (q + 1) // 2 for s, q in zip(seen, qs))
        nbytes = sum(seen) * nkv * hd * 2 * cache.k.element_size() + 2 * _nbytes(q)
        return self._timed("attention", nbytes, 4 * nh * hd * pairs, self._be.attention, q, cache, ctx, nh, scale, window)

    def argmax(self, logits):
        return self._timed("sample", _nbytes(logits), 0, self._be.argmax, logits)

    def sample(self, logits, *a, **k):
        return self._timed("sample", _nbytes(logits), 0, self._be.sample, logits, *a, **k)

    def logprobs(self, logits, *a, **k):
        return self._timed("sample", _nbytes(logits), 0, self._be.logprobs, logits, *a, **k)
