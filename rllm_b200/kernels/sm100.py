"""Python face of the tcgen05 / TMA kernels (library "sm100"). Placeholder until built."""
from __future__ import annotations


def init(device) -> None:
    return None


def gemm_supported(x, w) -> bool:
    return False


def gemm(x, w, epilogue, out=None):
    raise NotImplementedError


def attention(q, cache, ctx, nh, scale, window):
    return None
