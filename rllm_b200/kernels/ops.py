"""Python face of the CUDA kernels: checks shapes, dtypes and devices, then calls
the `extern "C"` launchers on torch's current stream.

There is no CPU or library path behind these functions. A tensor that is not on
a CUDA device, a size a kernel cannot take, or a failed launch raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

DT_F32, DT_BF16 = 0, 1
_DT = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}

EPI_STORE, EPI_STORE_F32, EPI_ACCUM_F32, EPI_SWIGLU = 0, 1, 2, 3

_ERR = {-1: "unsupported dtype", -2: "unsupported size", -3: "misaligned operand",
        -4: "problem too large for this kernel", -5: "kernel set-up failed"}


class KernelError(RuntimeError):
    pass


_P = c_void_p
_SIGS = {
    "simt": {
        "rllm_embed": [_P, _P, c_int, _P, c_int, c_int, c_int, _P, _P],
        "rllm_rmsnorm": [_P, _P, _P, c_int, _P, c_int, c_int, c_int, c_float, _P],
        "rllm_rope_table": [_P, _P, _P, c_int, c_int, _P],
        "rllm_rope_cache_write": [_P, c_int, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                                  c_int, _P],
        "rllm_gather_rows": [_P, _P, _P, c_int, c_int, _P],
        "rllm_step_meta": [_P, _P, c_int, _P, c_int, _P],
        "rllm_add_into": [_P, _P, c_int, c_longlong, _P],
        "rllm_add_bias": [_P, _P, c_int, c_int, c_int, c_longlong, _P],
        "rllm_check_meta": [_P, c_int, _P, c_int, c_int, c_int, _P, _P],
        "rllm_silu_gate": [_P, _P, c_int, c_int, c_int, _P],
        "rllm_gemm_simt": [c_int, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
        "rllm_paged_attention_simt": [c_int, _P, c_int, _P, _P, _P, c_int, _P, _P, _P, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_float, c_int, _P],
        "rllm_argmax": [_P, c_int, c_int, _P, _P],
        "rllm_sample": [_P, c_int, c_int, _P, _P, _P, _P, _P, _P, _P],
        "rllm_add_at": [_P, c_int, c_int, _P, _P, _P, c_int, _P],
        "rllm_logprobs": [_P, c_int, c_int, _P, _P, _P, _P, c_int, c_int, _P, _P, _P],
    },
}
_fn_cache: dict[str, object] = {}


def _fn(lib: str, name: str):
    f = _fn_cache.get(name)
    if f is None:
        cdll = build.load_library(lib)
        try:
            f = getattr(cdll, name)
        except AttributeError as e:
            raise KernelError(f"kernel library '{lib}' lacks symbol {name}") from e
        f.restype = c_int
        f.argtypes = _SIGS[lib][name]
        _fn_cache[name] = f
    return f


def register_signatures(lib: str, sigs: dict) -> None:
    _SIGS.setdefault(lib, {}).update(sigs)


LAUNCHES = 0          # kernel launches issued through this module (bench.py reports it)


def _check(rc: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += launches
        return
    if rc < 0:
        raise KernelError(f"{what}: {_ERR.get(rc, 'refused')} (code {rc})")
    raise KernelError(f"{what}: CUDA launch failed with error {rc}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (asked once per launch: the short way, where torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this engine has no CPU path)")


def _dt(t: torch.Tensor, name: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------------------------

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None,
          err: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32. ids int32 [T]; table [V, H] float32/bfloat16."""
    _cuda(ids, "ids"); _cuda(table, "table")
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("ids must be a contiguous int32 vector")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("table must be a contiguous [V, H] matrix")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(_fn("simt", "rllm_embed")(ids.data_ptr(), table.data_ptr(), _dt(table, "table"),
                                     out.data_ptr(), T, H, V, _ptr(err), _stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
            out: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w. x float32 [T, H]; w [H]. With `rows` (int32 [R]) only
    those rows of x are normalised: y [R, H]."""
    _cuda(x, "x"); _cuda(w, "w")
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("rmsnorm input must be a contiguous float32 [T, H]")
    T, H = x.shape
    if rows is not None:
        if rows.dtype != torch.int32 or rows.dim() != 1 or not rows.is_contiguous():
            raise KernelError("rmsnorm rows must be a contiguous int32 vector")
        T = rows.numel()
    if w.shape != (H,) or not w.is_contiguous():
        raise KernelError(f"rmsnorm weight must be [{H}], got {tuple(w.shape)}")
    if out is None:
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _check(_fn("simt", "rllm_rmsnorm")(x.data_ptr(), _ptr(rows), w.data_ptr(), _dt(w, "w"), out.data_ptr(),
                                       _dt(out, "out"), T, H, float(eps), _stream()), "rmsnorm")
    return out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, T: int) -> torch.Tensor:
    """(cos, sin)(positions[t] * inv_freq[i]) as float32 [T, len(inv_freq), 2]: a step's rotations,
    made once and read by every layer."""
    _cuda(positions, "positions"); _cuda(inv_freq, "inv_freq")
    if positions.dtype != torch.int32 or positions.numel() < T or inv_freq.dtype != torch.float32 \
            or not inv_freq.is_contiguous():
        raise KernelError("rope_table takes int32 positions [T] and float32 inverse frequencies")
    out = torch.empty((T, inv_freq.numel(), 2), dtype=torch.float32, device=positions.device)
    _check(_fn("simt", "rllm_rope_table")(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), T,
                                          inv_freq.numel(), _stream()), "rope_table")
    return out


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                     slots: torch.Tensor | None, kcache: torch.Tensor | None,
                     vcache: torch.Tensor | None, nh: int, nkv: int, hd: int, page_size: int,
                     rot_dim: int | None = None, table: torch.Tensor | None = None) -> None:
    """Rotate q and k of `qkv` [T, (nh+2nkv)*hd] (q in place) and write k, v to the cache.
    `table`: `rope_table(positions, inv_freq[:rot_dim // 2], T)`, else the angles are computed here."""
    _cuda(qkv, "qkv")
    T = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != (nh + 2 * nkv) * hd or not qkv.is_contiguous():
        raise KernelError(f"qkv must be contiguous [T, {(nh + 2 * nkv) * hd}], got {tuple(qkv.shape)}")
    rot_dim = hd if rot_dim is None else rot_dim
    if inv_freq.dtype != torch.float32 or inv_freq.numel() < rot_dim // 2:
        raise KernelError("inv_freq must hold rot_dim/2 float32 values")
    if positions.dtype != torch.int32 or positions.numel() < T:
        raise KernelError("positions must be int32 [T]")
    if slots is not None:
        if slots.dtype != torch.int32 or slots.numel() < T:
            raise KernelError("slots must be int32 [T]")
        for c, n in ((kcache, "kcache"), (vcache, "vcache")):
            if c is None or c.dtype != qkv.dtype or c.dim() != 4 or c.shape[1:] != (nkv, page_size, hd) \
                    or not c.is_contiguous():
                raise KernelError(f"{n} must be contiguous [pages, {nkv}, {page_size}, {hd}] of {qkv.dtype}")
    if table is not None and (table.dtype != torch.float32 or tuple(table.shape) != (T, rot_dim // 2, 2)
                              or not table.is_contiguous()):
        raise KernelError(f"rope table must be contiguous float32 [{T}, {rot_dim // 2}, 2]")
    _check(_fn("simt", "rllm_rope_cache_write")(
        qkv.data_ptr(), _dt(qkv, "qkv"), positions.data_ptr(), inv_freq.data_ptr(), _ptr(table), _ptr(slots),
        _ptr(kcache), _ptr(vcache), T, nh, nkv, hd, page_size, rot_dim, _stream()), "rope_cache_write")


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _cuda(x, "x")
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or rows.dtype != torch.int32:
        raise KernelError("gather_rows takes float32 [T, H] and int32 rows")
    out = torch.empty((rows.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    _check(_fn("simt", "rllm_gather_rows")(x.data_ptr(), rows.data_ptr(), out.data_ptr(),
                                           rows.numel(), x.shape[1], _stream()), "gather_rows")
    return out


def add_into(residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """residual (float32) += delta (float32 or bfloat16), element-wise, in place."""
    _cuda(residual, "residual")
    if residual.dtype != torch.float32 or residual.shape != delta.shape \
            or not residual.is_contiguous() or not delta.is_contiguous():
        raise KernelError("add_into takes a contiguous float32 residual and a delta of its shape")
    _check(_fn("simt", "rllm_add_into")(residual.data_ptr(), delta.data_ptr(), _dt(delta, "delta"),
                                        residual.numel(), _stream()), "add_into")
    return residual


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y [T, N] += bias [N], in place; both float32 or both bfloat16."""
    _cuda(y, "y"); _cuda(bias, "bias")
    if y.dim() != 2 or y.stride(1) != 1 or bias.dtype != y.dtype or bias.shape != (y.shape[1],) \
            or not bias.is_contiguous():
        raise KernelError("add_bias takes y [T, N] with unit inner stride and a bias [N] of the same dtype")
    _check(_fn("simt", "rllm_add_bias")(y.data_ptr(), bias.data_ptr(), _dt(y, "y"), y.shape[0], y.shape[1],
                                        y.stride(0), _stream()), "add_bias")
    return y


def check_meta(block_table: torch.Tensor, slots: torch.Tensor, num_pages: int, page_size: int,
               err: torch.Tensor) -> None:
    """Checked runs: entries of a step's block table [S, P] outside [-1, num_pages) and slots outside
    [-1, num_pages * page_size) are put to -1 (kernels then skip them) and `err` (one int32 on the
    device) records the first offender: 1 + index into the table, or 0x40000000 | index of the slot."""
    if block_table.dtype != torch.int32 or slots.dtype != torch.int32 or err.dtype != torch.int32 \
            or not block_table.is_contiguous() or not slots.is_contiguous():
        raise KernelError("check_meta takes contiguous int32 tensors")
    _check(_fn("simt", "rllm_check_meta")(block_table.data_ptr(), block_table.numel(), slots.data_ptr(), slots.numel(),
                                          int(num_pages), int(page_size), err.data_ptr(), _stream()), "check_meta")


def silu_gate(gu: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gu[t, i]) * gu[t, I + i] for gu [T, 2I]."""
    _cuda(gu, "gu")
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    _check(_fn("simt", "rllm_silu_gate")(gu.data_ptr(), out.data_ptr(), _dt(gu, "gu"), T, I2 // 2,
                                         _stream()), "silu_gate")
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, epilogue: int, out: torch.Tensor | None = None,
              bias: torch.Tensor | None = None) -> torch.Tensor:
    """C = A W^T on the CUDA cores (float accumulate). a [T, K]; w [N, K] ([2N, K] for SwiGLU)."""
    _cuda(a, "a"); _cuda(w, "w")
    if a.dim() != 2 or w.dim() != 2 or a.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("gemm takes a [T, K] (unit inner stride) and a contiguous w [N, K]")
    if a.dtype != w.dtype:
        raise KernelError(f"gemm operands differ in dtype: {a.dtype} vs {w.dtype}")
    T, K = a.shape
    N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm inner sizes differ: a {tuple(a.shape)}, w {tuple(w.shape)}")
    if epilogue == EPI_SWIGLU and w.shape[0] % 2:
        raise KernelError("SwiGLU epilogue needs an even number of weight rows")
    out_dtype = torch.float32 if epilogue in (EPI_STORE_F32, EPI_ACCUM_F32) else a.dtype
    if out is None:
        if epilogue == EPI_ACCUM_F32:
            raise KernelError("accumulate epilogue needs the residual tensor as out")
        out = torch.empty((T, N), dtype=out_dtype, device=a.device)
    if out.dtype != out_dtype or out.shape != (T, N) or out.stride(1) != 1:
        raise KernelError(f"gemm out must be [{T}, {N}] of {out_dtype}")
    if bias is not None and (bias.dtype != a.dtype or bias.numel() != N or epilogue == EPI_SWIGLU):
        raise KernelError("gemm bias must be [N] of the operand dtype (not with SwiGLU)")
    _check(_fn("simt", "rllm_gemm_simt")(_dt(a, "a"), epilogue, a.data_ptr(), w.data_ptr(),
                                         out.data_ptr(), _ptr(bias), T, N, K, a.stride(0),
                                         out.stride(0), _stream()), "gemm_simt")
    return out


def paged_attention_simt(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         token_seq: torch.Tensor, positions: torch.Tensor,
                         block_table: torch.Tensor, nh: int, scale: float, window: int | None,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """Attention over the paged cache for every query token. q: [T, >= nh*hd] view whose row
    stride may exceed nh*hd (the q part of a qkv buffer); caches [pages, nkv, page, hd]."""
    _cuda(q, "q")
    T = q.shape[0]
    _, nkv, page_size, hd = kcache.shape
    if q.stride(1) != 1 or q.shape[1] != nh * hd:
        raise KernelError(f"q must be [T, {nh * hd}] with unit inner stride")
    if kcache.dtype != q.dtype or vcache.dtype != q.dtype or vcache.shape != kcache.shape \
            or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("k and v caches must be contiguous, alike, and of q's dtype")
    for t, n in ((token_seq, "token_seq"), (positions, "positions"), (block_table, "block_table")):
        if t.dtype != torch.int32:
            raise KernelError(f"{n} must be int32")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block_table must be [sequences, pages] with unit inner stride")
    if out is None:
        out = torch.empty((T, nh * hd), dtype=q.dtype, device=q.device)
    _check(_fn("simt", "rllm_paged_attention_simt")(
        _dt(q, "q"), q.data_ptr(), q.stride(0), kcache.data_ptr(), vcache.data_ptr(), out.data_ptr(),
        out.stride(0), token_seq.data_ptr(), positions.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), T, nh, nkv, hd, page_size, float(scale), int(window or 0), _stream()),
        "paged_attention_simt")
    return out


def step_meta(host: torch.Tensor, dev: torch.Tensor, n: int, feed: torch.Tensor | None = None) -> None:
    """The first `n` int32 words of the pinned host buffer into the device buffer, by a kernel that
    reads the host memory directly; the leading `feed.numel()` words from the device vector `feed`
    instead, if given."""
    if host.dtype != torch.int32 or dev.dtype != torch.int32 or not host.is_pinned() or not dev.is_cuda \
            or not (0 < n <= min(host.numel(), dev.numel())):
        raise KernelError("step_meta takes a pinned int32 host buffer, an int32 device buffer and a count within both")
    if feed is not None and (feed.dtype != torch.int32 or not feed.is_cuda or not feed.is_contiguous()
                             or feed.numel() > n):
        raise KernelError("step_meta: feed must be a contiguous int32 device vector no longer than the count")
    _check(_fn("simt", "rllm_step_meta")(host.data_ptr(), dev.data_ptr(), n, _ptr(feed),
                                         0 if feed is None else feed.numel(), _stream()), "step_meta")


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _cuda(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise KernelError("argmax takes contiguous float32 logits [R, V]")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _check(_fn("simt", "rllm_argmax")(logits.data_ptr(), R, V, out.data_ptr(), _stream()), "argmax")
    return out


def add_at(logits: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor, vals: torch.Tensor) -> None:
    """logits[rows[i], cols[i]] += vals[i] in place; distinct (row, col) pairs, every one inside the
    matrix (the caller's duty: they are not checked on the device). The lists: int32, int32, float32
    on the device or in pinned host memory."""
    _cuda(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise KernelError("add_at takes contiguous float32 logits [R, V]")
    n = rows.numel()
    for t, d in ((rows, torch.int32), (cols, torch.int32), (vals, torch.float32)):
        if t.dtype != d or t.numel() != n or not (t.is_cuda or t.is_pinned()) or not t.is_contiguous():
            raise KernelError("add_at: rows and cols int32, vals float32, alike in length, on the device or pinned")
    R, V = logits.shape
    _check(_fn("simt", "rllm_add_at")(logits.data_ptr(), R, V, rows.data_ptr(), cols.data_ptr(), vals.data_ptr(), n,
                                      _stream()), "add_at")


TOP_LOGPROBS_MAX = 20


def logprobs(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None, chosen: torch.Tensor,
             rows: torch.Tensor, n_top: int) -> tuple[torch.Tensor, torch.Tensor]:
    """For each listed row of float32 logits [R, V]: ln p of the chosen token and the n_top most
    probable tokens under softmax(x / T over what top-k keeps), x itself where T is 0. Returns
    (float32 [n, 1 + n_top], int32 [n, n_top]) on the device; an entry that does not exist is
    (-inf, -1). temperature [R] float32, top_k [R] int32 or None and rows [n] int32 on the device
    or pinned; chosen [R] int32 on the device."""
    _cuda(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise KernelError("logprobs takes contiguous float32 logits [R, V]")
    R, V = logits.shape
    n = rows.numel()
    if not 0 <= n_top <= TOP_LOGPROBS_MAX:
        raise KernelError(f"top_logprobs must be 0..{TOP_LOGPROBS_MAX}, got {n_top}")
    for t, name, d, ln in ((temperature, "temperature", torch.float32, R), (top_k, "top_k", torch.int32, R),
                           (rows, "rows", torch.int32, n)):
        if t is not None and (t.dtype != d or t.numel() != ln or not (t.is_cuda or t.is_pinned()) or not t.is_contiguous()):
            raise KernelError(f"logprobs: {name} must be a {d} vector of length {ln} on the device or pinned")
    if chosen.dtype != torch.int32 or chosen.numel() != R or not chosen.is_cuda or not chosen.is_contiguous():
        raise KernelError(f"logprobs: chosen must be an int32 vector of length {R} on the device")
    lp = torch.empty((n, 1 + n_top), dtype=torch.float32, device=logits.device)
    ids = torch.empty((n, max(n_top, 1)), dtype=torch.int32, device=logits.device)
    _check(_fn("simt", "rllm_logprobs")(logits.data_ptr(), R, V, temperature.data_ptr(), _ptr(top_k), chosen.data_ptr(),
                                        rows.data_ptr(), n, n_top, lp.data_ptr(), ids.data_ptr(), _stream()), "logprobs")
    return lp, ids[:, :n_top]


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           top_k: torch.Tensor | None = None, top_p: torch.Tensor | None = None,
           min_p: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One draw per row with per-row parameters: vectors of length R on the device, or in pinned host
    memory, which the kernel then reads itself (a few words a row; no copy to wait for)."""
    _cuda(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise KernelError("sample takes contiguous float32 logits [R, V]")
    R, V = logits.shape
    for t, n, d in ((temperature, "temperature", torch.float32), (uniform, "uniform", torch.float32),
                    (top_k, "top_k", torch.int32), (top_p, "top_p", torch.float32),
                    (min_p, "min_p", torch.float32)):
        if t is not None and (t.dtype != d or t.numel() != R or not (t.is_cuda or t.is_pinned()) or not t.is_contiguous()):
            raise KernelError(f"{n} must be a {d} vector of length {R} on the device or in pinned host memory")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _check(_fn("simt", "rllm_sample")(logits.data_ptr(), R, V, temperature.data_ptr(), _ptr(top_k),
                                      _ptr(top_p), _ptr(min_p), uniform.data_ptr(), out.data_ptr(),
                                      _stream()), "sample")
    return out
