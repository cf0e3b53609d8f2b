"""Python face of the tcgen05 / TMA kernels (library "sm100"), which only the bfloat16 path
calls. Holds the scratch memory of the split-K product (partial tiles and tile counters) and
the device error word that a bounded wait sets when it runs out."""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p, POINTER, byref

import torch

from . import ops

_P = c_void_p
ops.register_signatures("sm100", {
    "rllm_tc_gemm": [c_int, _P, c_longlong, _P, _P, c_longlong, c_int, c_int, c_int, _P, c_longlong, _P,
                     c_int, _P, c_int, _P],
    "rllm_tc_gemm_plan": [c_int, c_int, c_int, c_int, c_int, c_longlong, c_int, POINTER(c_int), POINTER(c_int)],
})

WS_BYTES = 64 << 20
MAX_COUNTERS = 8192


class _State:
    def __init__(self, device):
        self.device = device
        self.ws = torch.empty(WS_BYTES // 4, dtype=torch.float32, device=device)
        self.counters = torch.zeros(MAX_COUNTERS, dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
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
    code = int(st.err.item())
    if code:
        st.err.zero_()
        raise ops.KernelError(f"a tcgen05 kernel gave up waiting (role {code}); its output is not valid")


def gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1]
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.shape[0] > 0)


def plan(epilogue: int, T: int, N: int, K: int, device="cuda:0") -> tuple[int, int]:
    st = init(device)
    bn, sp = c_int(), c_int()
    ops._fn("sm100", "rllm_tc_gemm_plan")(epilogue, T, N, K, st.sm_count, WS_BYTES, MAX_COUNTERS,
                                          byref(bn), byref(sp))
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
    rc = ops._fn("sm100", "rllm_tc_gemm")(
        epilogue, x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), T, N, K,
        st.ws.data_ptr() if split else None, WS_BYTES, st.counters.data_ptr() if split else None,
        MAX_COUNTERS, st.err.data_ptr(), st.sm_count, ops._stream())
    ops._check(rc, "tc_gemm")
    return out


def attention(q, cache, ctx, nh, scale, window):
    return None
