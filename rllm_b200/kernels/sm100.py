"""Python face of the tcgen05 / TMA kernels (library "sm100"), which only the bfloat16 path
calls. Holds the device error word that a bounded wait sets when it runs out."""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p, POINTER, byref

import torch

from . import ops

_P = c_void_p
ops.register_signatures("sm100", {
    "rllm_tc_gemm": [c_int, _P, c_longlong, _P, _P, c_longlong, c_int, c_int, c_int, c_int, _P, c_int, _P],
    "rllm_tc_gemm_set_pairs": [c_int],
    "rllm_tc_gemm_set_token_rows": [c_int],
    "rllm_tc_gemm_plan": [c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int)],
    "rllm_tc_gemm_norm": [c_int, _P, c_longlong, _P, _P, c_int, c_float, _P, _P, c_longlong, c_int, c_int, c_int,
                          c_int, _P, c_int, _P],
    "rllm_tc_gemm_norm_max_tokens": [],
    "rllm_tc_gemm_qkv_rope": [_P, c_longlong, _P, c_longlong, _P, c_int, c_float, _P, _P, c_longlong, c_int, c_int,
                              _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int, _P],
    "rllm_stream_gemm_supported": [c_int, c_int, c_int, c_int, c_int, c_int],
    "rllm_stream_gemm": [c_int, _P, c_longlong, _P, c_longlong, _P, _P, c_int, c_float, _P, _P, c_longlong, c_int,
                         c_int, c_int, c_int, _P],
    "rllm_stream_gemm_qkv_rope": [_P, c_longlong, _P, c_longlong, _P, c_int, c_float, _P, _P, c_longlong, c_int, c_int,
                                  _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "rllm_wait_probe": [_P, c_longlong, c_int, _P],
    "rllm_attention_fa": [_P, c_int, _P, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_float, c_int, c_int, _P, _P, _P],
    "rllm_attention_prefill_tc": [_P, c_int, _P, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_float, c_int, _P, c_int, _P],
    "rllm_attention_decode": [_P, c_int, _P, _P, c_longlong, _P, c_int, _P, _P, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_float, c_int, c_int, _P, _P],
})


class _State:
    def __init__(self, device):
        self.device = device
        # word 0: set by a kernel whose bounded wait ran out; words 1 and 2: for the engine's own
        # flags (a token id outside the table; in checked runs a page or slot outside the pool), so
        # that one small copy brings them all to the host; word 3 spare
        self.err = torch.zeros(4, dtype=torch.int32, device=device)
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count


_states: dict[int, _State] = {}


def init(device) -> _State:
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        cap = torch.cuda.get_device_capability(idx)
        if cap[0] != 10:
            raise ops.KernelError(f"the tcgen05 kernels need an sm_100 device, this one is sm_{cap[0]}{cap[1]}")
        ops._fn("sm100", "rllm_tc_gemm")          # builds / loads the library, or raises
        st = _states[idx] = _State(torch.device("cuda", idx))
    return st


def check_error(device) -> None:
    """Raise if a kernel's bounded wait ran out since the last check (reads the device word)."""
    st = init(device)
    code = int(st.err[0].item())
    if code:
        st.err[0].zero_()
        raise ops.KernelError(f"a kernel's bounded wait ran out (role {code & 0xff}, detail {code >> 8}); "
                              f"its output is not valid")


def wait_probe(device, limit_cycles: int = 200000, arrive_first: bool = False) -> None:
    """Launch the one-warp kernel that waits on an mbarrier nobody arrives at (unless `arrive_first`)
    for at most `limit_cycles` cycles and records the time-out in the error word: the bounded wait
    of the tcgen05 kernels, exercised where nothing else is in flight."""
    st = init(device)
    ops._check(ops._fn("sm100", "rllm_wait_probe")(st.err.data_ptr(), int(limit_cycles), int(arrive_first),
                                                   ops._stream()), "wait_probe")


EPI_QKV_ROPE = 4
STREAM = os.environ.get("RLLM_B200_NO_STREAM_GEMM") != "1"
_stream_ok: dict[tuple, bool] = {}


def stream_supported(epilogue: int, norm: bool, T: int, N: int, K: int, hd: int = 0) -> bool:
    """Does the weight-streaming kernel for steps of at most 8 tokens take this product? (N: output
    features, of one half with the SwiGLU epilogue.)"""
    if not STREAM or T > 8:
        return False
    key = (epilogue, norm, T, N, K, hd)
    ok = _stream_ok.get(key)
    if ok is None:
        ok = _stream_ok[key] = bool(ops._fn("sm100", "rllm_stream_gemm_supported")(epilogue, int(norm), T, N, K, hd))
    return ok


def set_pairs(on: bool) -> None:
    """Products of long prompt portions on pairs of CTAs (`tcgen05.mma.cta_group::2`) or on single CTAs
    (the default: measured level or faster)."""
    ops._fn("sm100", "rllm_tc_gemm_set_pairs")(int(on))


def set_token_rows(on: bool) -> None:
    """Gate/up products of portions of more than 64 tokens with the tokens on the accumulator's rows."""
    ops._fn("sm100", "rllm_tc_gemm_set_token_rows")(int(on))


def gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1]
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.shape[0] > 0)


def plan(epilogue: int, T: int, N: int, K: int, device="cuda:0", split: bool | int = True) -> tuple[int, int]:
    """(token tile, ranges of K = CTAs per cluster) the tcgen05 launcher chooses for a problem.
    `split`: False one CTA per tile, True its own choice, a number > 1 that many ranges."""
    st = init(device)
    bn, sp = c_int(), c_int()
    ops._fn("sm100", "rllm_tc_gemm_plan")(epilogue, T, N, K, st.sm_count, int(split), byref(bn), byref(sp))
    return bn.value, sp.value


def gemm(x: torch.Tensor, w: torch.Tensor, epilogue: int, out: torch.Tensor | None = None,
         split: bool = True) -> torch.Tensor:
    """C = X W^T on the tensor cores. x [T, K] bf16 (unit inner stride); w [N, K] bf16 ([2N, K] with
    the SwiGLU epilogue). `out` is required for the accumulate epilogue (the float residual)."""
    if not gemm_supported(x, w):
        raise ops.KernelError("tc gemm: operands must be bfloat16, K a multiple of 8, 16-byte aligned")
    st = init(x.device)
    T, K = x.shape
    N = w.shape[0] // 2 if epilogue == ops.EPI_SWIGLU else w.shape[0]
    out_dtype = torch.float32 if epilogue in (ops.EPI_STORE_F32, ops.EPI_ACCUM_F32) else torch.bfloat16
    if out is None:
        if epilogue == ops.EPI_ACCUM_F32:
            raise ops.KernelError("accumulate epilogue needs the residual tensor as out")
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    if out.dtype != out_dtype or out.shape != (T, N) or out.stride(1) != 1:
        raise ops.KernelError(f"tc gemm out must be [{T}, {N}] of {out_dtype}")
    if split and stream_supported(epilogue, False, T, N, K):
        rc = ops._fn("sm100", "rllm_stream_gemm")(
            epilogue, x.data_ptr(), x.stride(0), None, 0, None, None, 0, 0.0, w.data_ptr(), out.data_ptr(),
            out.stride(0), T, N, K, st.sm_count, ops._stream())
        ops._check(rc, "stream_gemm")
        return out
    rc = ops._fn("sm100", "rllm_tc_gemm")(
        epilogue, x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), T, N, K,
        int(split), st.err.data_ptr(), st.sm_count, ops._stream())
    ops._check(rc, "tc_gemm")
    return out


_norm_max = None


def norm_max_tokens() -> int:
    """The most tokens a step may bring for the products with RMSNorm in front."""
    global _norm_max
    if _norm_max is None:
        _norm_max = int(ops._fn("sm100", "rllm_tc_gemm_norm_max_tokens")())
    return _norm_max


def norm_supported(h: torch.Tensor, g: torch.Tensor, w: torch.Tensor, rows: torch.Tensor | None = None) -> bool:
    """Can `rmsnorm(h[rows]) W^T` run as one kernel? h float32 [*, K] rows, g the norm weight."""
    T = h.shape[0] if rows is None else rows.numel()
    return (h.dtype == torch.float32 and h.dim() == 2 and h.stride(1) == 1 and h.stride(0) % 4 == 0
            and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous() and h.shape[1] == w.shape[1]
            and h.shape[1] % 8 == 0 and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous()
            and g.numel() == h.shape[1] and h.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and g.data_ptr() % 16 == 0 and 0 < T <= norm_max_tokens()
            and (rows is None or (rows.dtype == torch.int32 and rows.is_contiguous())))


def gemm_norm(h: torch.Tensor, g: torch.Tensor, eps: float, w: torch.Tensor, epilogue: int,
              rows: torch.Tensor | None = None, split: bool = True) -> torch.Tensor:
    """C = rmsnorm(h[rows]; g, eps) W^T in one kernel (store, store-float or SwiGLU epilogue)."""
    if not norm_supported(h, g, w, rows):
        raise ops.KernelError("tc gemm with norm: float32 rows of K % 8 == 0 values, at most "
                              f"{norm_max_tokens()} tokens, bfloat16 weights, 16-byte aligned")
    if epilogue not in (ops.EPI_STORE, ops.EPI_STORE_F32, ops.EPI_SWIGLU):
        raise ops.KernelError("tc gemm with norm: epilogue must be store, store-float or SwiGLU")
    st = init(h.device)
    T = h.shape[0] if rows is None else rows.numel()
    K = h.shape[1]
    N = w.shape[0] // 2 if epilogue == ops.EPI_SWIGLU else w.shape[0]
    out = torch.empty((T, N), dtype=torch.float32 if epilogue == ops.EPI_STORE_F32 else torch.bfloat16,
                      device=h.device)
    if split and stream_supported(epilogue, True, T, N, K):
        rc = ops._fn("sm100", "rllm_stream_gemm")(
            epilogue, None, 0, h.data_ptr(), h.stride(0), ops._ptr(rows), g.data_ptr(), ops._dt(g, "norm weight"),
            float(eps), w.data_ptr(), out.data_ptr(), out.stride(0), T, N, K, st.sm_count, ops._stream())
        ops._check(rc, "stream_gemm_norm")
        return out
    rc = ops._fn("sm100", "rllm_tc_gemm_norm")(
        epilogue, h.data_ptr(), h.stride(0), ops._ptr(rows), g.data_ptr(), ops._dt(g, "norm weight"), float(eps),
        w.data_ptr(), out.data_ptr(), out.stride(0), T, N, K, int(split), st.err.data_ptr(), st.sm_count,
        ops._stream())
    ops._check(rc, "tc_gemm_norm")
    return out


def qkv_rope_supported(x: torch.Tensor, w: torch.Tensor, kcache, hd: int, rot_dim: int | None = None) -> bool:
    """Rotation and cache write in the product's epilogue: heads that divide the 128 rows of a tile; from
    65 tokens on (the kernel of long portions, which moves 8 neighbouring features at a time) head size
    and rotated part in steps of 16."""
    rot_dim = hd if rot_dim is None else rot_dim
    long_ok = hd % 16 == 0 and rot_dim % 16 == 0
    return gemm_supported(x, w) and 128 % hd == 0 and (x.shape[0] <= 64 or long_ok) and \
        (kcache is None or kcache.dtype == torch.bfloat16)


def gemm_qkv_rope(x: torch.Tensor | None, w_qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                  slots: torch.Tensor | None, kcache: torch.Tensor | None, vcache: torch.Tensor | None,
                  nh: int, nkv: int, hd: int, page_size: int, rot_dim: int, split: bool = True,
                  norm: tuple | None = None, table: torch.Tensor | None = None) -> torch.Tensor:
    """qkv = x w_qkv^T with q and k rotated by position and k, v written to the paged cache at
    `slots` (None: no write), all in the product's epilogue. Returns qkv [T, (nh + 2 nkv) * hd].
    `norm` = (h, g, eps) instead of x: RMSNorm of the float rows h in front, in the same kernel.
    `table`: `ops.rope_table` of these positions ([T, rot_dim / 2, 2]); else the angles are computed here."""
    T, K = norm[0].shape if norm is not None else x.shape
    # steps of at most 8 tokens: the weight-streaming kernel (any head size that is a multiple of 32)
    streamed = split and rot_dim == hd and stream_supported(EPI_QKV_ROPE, norm is not None, T, (nh + 2 * nkv) * hd, K, hd)
    if norm is not None:
        h, g, eps = norm
        if not norm_supported(h, g, w_qkv) or (128 % hd and not streamed) or \
                (kcache is not None and kcache.dtype != torch.bfloat16):
            raise ops.KernelError("tc gemm with norm and rotary epilogue: sizes not supported")
        dev = h.device
    else:
        if not (gemm_supported(x, w_qkv) and (128 % hd == 0 or streamed)
                and (kcache is None or kcache.dtype == torch.bfloat16)):
            raise ops.KernelError("tc gemm with rotary epilogue: bfloat16 operands and a head size dividing 128")
        dev = x.device
    st = init(dev)
    N = (nh + 2 * nkv) * hd
    if w_qkv.shape[0] != N:
        raise ops.KernelError(f"w_qkv must have {N} rows, got {w_qkv.shape[0]}")
    if positions.dtype != torch.int32 or positions.numel() < T or inv_freq.dtype != torch.float32 \
            or inv_freq.numel() < rot_dim // 2:
        raise ops.KernelError("positions must be int32 [T] and inv_freq float32 [rot_dim/2]")
    if slots is not None:
        if slots.dtype != torch.int32 or slots.numel() < T:
            raise ops.KernelError("slots must be int32 [T]")
        for c in (kcache, vcache):
            if c is None or c.dtype != torch.bfloat16 or c.dim() != 4 or tuple(c.shape[1:]) != (nkv, page_size, hd) \
                    or not c.is_contiguous():
                raise ops.KernelError(f"caches must be contiguous bfloat16 [pages, {nkv}, {page_size}, {hd}]")
    if table is not None and (table.dtype != torch.float32 or tuple(table.shape) != (T, rot_dim // 2, 2)
                              or not table.is_contiguous()):
        raise ops.KernelError(f"rope table must be contiguous float32 [{T}, {rot_dim // 2}, 2]")
    out = torch.empty((T, N), dtype=torch.bfloat16, device=dev)
    if norm is not None:
        xa = (None, 0, h.data_ptr(), h.stride(0), g.data_ptr(), ops._dt(g, "norm weight"), float(eps))
    else:
        xa = (x.data_ptr(), x.stride(0), None, 0, None, 0, 0.0)
    if streamed:
        rc = ops._fn("sm100", "rllm_stream_gemm_qkv_rope")(
            *xa, w_qkv.data_ptr(), out.data_ptr(), out.stride(0), T, K, positions.data_ptr(),
            inv_freq.data_ptr(), ops._ptr(table), ops._ptr(slots), ops._ptr(kcache) if slots is not None else None,
            ops._ptr(vcache) if slots is not None else None, nh, nkv, hd, page_size, st.sm_count, ops._stream())
        ops._check(rc, "stream_gemm_qkv_rope")
        return out
    rc = ops._fn("sm100", "rllm_tc_gemm_qkv_rope")(
        *xa, w_qkv.data_ptr(), out.data_ptr(), out.stride(0), T, K, positions.data_ptr(),
        inv_freq.data_ptr(), ops._ptr(table), ops._ptr(slots), ops._ptr(kcache) if slots is not None else None,
        ops._ptr(vcache) if slots is not None else None, nh, nkv, hd, page_size, rot_dim, int(split),
        st.err.data_ptr(), st.sm_count, ops._stream())
    ops._check(rc, "tc_gemm_qkv_rope")
    return out


def attention_supported(q: torch.Tensor, kcache: torch.Tensor) -> bool:
    return q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and kcache.shape[3] in (64, 128)


def attention_splits(num_seqs: int, nkv: int, max_rows: int, max_kv_len: int, sm_count: int) -> int:
    """How many ranges the keys of a sequence are cut into. Prefill-sized tiles fill the GPU
    by themselves; decode-sized batches are cut until about four CTAs per SM exist, each with
    at least two 64-key tiles."""
    if max_rows > 16:
        return 1
    base = max(1, num_seqs * nkv)
    want = (4 * sm_count + base - 1) // base
    return max(1, min(want, max_kv_len // 128, 64))


def attention_fa(q, kcache, vcache, cu_q, kv_lens, block_table, num_tokens, max_q_len, max_kv_len, nh,
                 scale, window, splits=None, out=None):
    """Tiled tensor-core attention over the paged cache (bf16, head size 64 or 128)."""
    st = init(q.device)
    _, nkv, page_size, hd = kcache.shape
    S = kv_lens.numel()
    G = nh // nkv
    if splits is None:
        splits = attention_splits(S, nkv, max_q_len * G, max_kv_len, st.sm_count)
    if out is None:
        out = torch.empty((q.shape[0], nh * hd), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        need = num_tokens * nh * splits
        part_o = torch.empty(need * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(need * 2, dtype=torch.float32, device=q.device)
    rc = ops._fn("sm100", "rllm_attention_fa")(
        q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(), out.stride(0),
        cu_q.data_ptr(), kv_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0), S, num_tokens,
        max_q_len, nh, nkv, hd, page_size, float(scale), int(window or 0), splits,
        None if part_o is None else part_o.data_ptr(), None if part_ml is None else part_ml.data_ptr(),
        ops._stream())
    ops._check(rc, "attention_fa", 2 if splits > 1 else 1)
    return out


TC_ATTENTION_MIN_KEYS = int(os.environ.get("RLLM_B200_TC_ATTENTION_MIN_KEYS", "512"))


def prefill_tc_supported(q: torch.Tensor, kcache: torch.Tensor) -> bool:
    return (q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and kcache.shape[3] in (64, 128)
            and kcache.is_contiguous() and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and kcache.data_ptr() % 16 == 0)


def attention_prefill_tc(q, kcache, vcache, cu_q, kv_lens, block_table, max_q_len, nh, scale, window, out=None):
    """Prefill attention on the tcgen05 tensor cores (bf16, head size 64 or 128): tiles of 128 rows x
    128 (64) keys, both products with their accumulators in TMEM."""
    if not prefill_tc_supported(q, kcache):
        raise ops.KernelError("attention_prefill_tc: bfloat16, head size 64 or 128, rows 16-byte aligned")
    st = init(q.device)
    _, nkv, page_size, hd = kcache.shape
    if out is None:
        out = torch.empty((q.shape[0], nh * hd), dtype=torch.bfloat16, device=q.device)
    rc = ops._fn("sm100", "rllm_attention_prefill_tc")(
        q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(), out.stride(0),
        cu_q.data_ptr(), kv_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0), kv_lens.numel(),
        max_q_len, kcache.shape[0], nh, nkv, hd, page_size, float(scale), int(window or 0), st.err.data_ptr(),
        st.sm_count, ops._stream())
    ops._check(rc, "attention_prefill_tc")
    return out


def decode_supported(q: torch.Tensor, kcache: torch.Tensor, nh: int) -> bool:
    _, nkv, page_size, hd = kcache.shape
    return attention_supported(q, kcache) and nh // nkv <= 16 and kcache.data_ptr() % 16 == 0


def decode_splits(num_seqs: int, nkv: int, max_kv_len: int, sm_count: int) -> int:
    """Ranges the keys of a sequence are cut into (= CTAs per cluster). Measured on a B200: a CTA
    costs about as much as 1,150 keys before its first key and a range 30 more at the merge, two CTAs
    fit an SM, and CTAs beyond that wait for a free place; the number of ranges with the least
    (rounds of CTAs over the places) x (1,150 + keys per range) + 30 x ranges is taken. Up to 8
    ranges any number; 12 and 16 (clusters beyond the portable size, for one or two long sequences:
    16,384 keys of one sequence 13.3 us against 18.3 with 8) only from 16,384 keys on and while the CTAs
    leave a quarter of the places free: a large cluster needs its places inside one GPC (9 ranges of 4
    sequences, 288 CTAs on 296 places: 16.7 us against 10.8 with 8), and inside a decode step, behind a
    kernel whose CTAs fill whole SMs, it starts later than a small one (4,096 keys: 6.3 us against 6.9
    alone, but the step at batch 1 0.621 ms against 0.615, at batch 2 0.692 against 0.642)."""
    base = max(1, num_seqs * nkv)
    places = 2 * sm_count
    best, best_cost = 1, None
    for s in (1, 2, 3, 4, 5, 6, 7, 8, 12, 16):
        if s > 1 and max_kv_len // s < 64:
            break
        if s > 8 and (base * s * 4 > places * 3 or max_kv_len < 16384):
            break
        cost = -(-base * s // places) * (1150 + max_kv_len / s) + 30 * s
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


def attention_decode(q, kcache, vcache, kv_lens, block_table, nh, scale, window, max_kv_len, splits=None,
                     out=None):
    """Attention for a step in which every sequence brings one token: the ranges of a sequence's
    keys are merged inside a thread-block cluster (bf16, head size 64 or 128, any page size)."""
    st = init(q.device)
    num_pages, nkv, page_size, hd = kcache.shape
    S = kv_lens.numel()
    if not decode_supported(q, kcache, nh) or q.shape[0] != S:
        raise ops.KernelError("attention_decode: one bfloat16 query row per sequence, head size 64 or 128, "
                              "at most 16 heads per kv head")
    if vcache.shape != kcache.shape or vcache.dtype != kcache.dtype or not kcache.is_contiguous() \
            or not vcache.is_contiguous() or block_table.dtype != torch.int32 or kv_lens.dtype != torch.int32:
        raise ops.KernelError("attention_decode: caches must be contiguous and alike, tables int32")
    if splits is None:
        splits = decode_splits(S, nkv, max_kv_len, st.sm_count)
    if out is None:
        out = torch.empty((S, nh * hd), dtype=torch.bfloat16, device=q.device)
    rc = ops._fn("sm100", "rllm_attention_decode")(
        q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), num_pages, out.data_ptr(),
        out.stride(0), kv_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0), S, nh, nkv, hd,
        page_size, float(scale), int(window or 0), int(splits), st.err.data_ptr(), ops._stream())
    ops._check(rc, "attention_decode")
    return out


def attention(q, cache, ctx, nh, scale, window):
    """The backend's hook: None when this kernel does not take the sizes at hand."""
    if not attention_supported(q, cache.k):
        return None
    if ctx.max_q_len == 1 and decode_supported(q, cache.k, nh):
        return attention_decode(q, cache.k, cache.v, ctx.kv_lens, cache.block_table, nh, scale, window,
                                ctx.max_kv_len)
    nkv = cache.k.shape[1]
    G = nh // nkv
    if ctx.max_q_len * G >= 128 and ctx.max_kv_len >= TC_ATTENTION_MIN_KEYS \
            and prefill_tc_supported(q, cache.k) and os.environ.get("RLLM_B200_NO_TC_ATTENTION") != "1":
        # long portions over long contexts: tiles of 128 (token, head) rows x 128 keys on the tcgen05
        # tensor cores (measured against the mma.sync kernel, head size 64: level at 512 keys, 1.4 x at
        # 1,024, 2.3 x at 2,048; head size 128: 1.2 x at 512, 2 x at 1,024, 3.2 x at 2,048; behind at 256)
        lens = ctx.q_lens_host
        D = 0                    # sequences in front that bring one token each (the scheduler puts decoding first)
        if lens is not None and ctx.kv_lens_host is not None and decode_supported(q, cache.k, nh):
            while D < len(lens) and lens[D] == 1:
                D += 1
        if 0 < D < len(lens) and max(lens[D:]) * G >= 128:
            # a mixed step: the decode kernel for the single tokens (a row tile of the other kernel
            # would hold one token's heads and nothing else), the portions after them on tcgen05
            hd = cache.k.shape[3]
            out = torch.empty((q.shape[0], nh * hd), dtype=torch.bfloat16, device=q.device)
            attention_decode(q[:D], cache.k, cache.v, ctx.kv_lens[:D], cache.block_table[:D], nh, scale, window,
                             max(ctx.kv_lens_host[:D]), out=out[:D])
            attention_prefill_tc(q, cache.k, cache.v, ctx.cu_q[D:], ctx.kv_lens[D:], cache.block_table[D:],
                                 max(lens[D:]), nh, scale, window, out=out)
            return out
        return attention_prefill_tc(q, cache.k, cache.v, ctx.cu_q, ctx.kv_lens, cache.block_table, ctx.max_q_len,
                                    nh, scale, window)
    return attention_fa(q, cache.k, cache.v, ctx.cu_q, ctx.kv_lens, cache.block_table, ctx.num_tokens,
                        ctx.max_q_len, ctx.max_kv_len, nh, scale, window)
