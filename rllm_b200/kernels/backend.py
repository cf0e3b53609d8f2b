"""Chooses the kernel for each operation of a run.

`Backend(torch.float32)` is the true 32-bit path: float storage everywhere and
FMA kernels only. `Backend(torch.bfloat16)` is the serving path: bfloat16
weights, activations and cache, float residual stream and logits; it sends
matrix products to the tcgen05 kernel and attention to the tiled kernels when
those take the sizes at hand, and to the generic CUDA-core kernels otherwise.
Both are hand-written CUDA; there is nothing else to fall back to.
"""
from __future__ import annotations

import os

import torch

from . import ops


class Normed:
    """An RMSNorm that has not run yet: rows of the float residual stream, the norm's weight and
    eps. A product that can take the norm in front of it in one kernel consumes it as it is;
    everything else calls `tensor()`, which runs the norm kernel once and keeps the result."""

    def __init__(self, backend, h, weight, eps, rows=None):
        self.backend, self.h, self.weight, self.eps, self.rows = backend, h, weight, float(eps), rows
        self._tensor = None

    @property
    def shape(self):
        return (self.h.shape[0] if self.rows is None else self.rows.numel(), self.h.shape[1])

    def tensor(self):
        if self._tensor is None:
            self._tensor = self.backend.rmsnorm(self.h, self.weight, self.eps, rows=self.rows)
        return self._tensor


class Backend:
    def __init__(self, dtype: torch.dtype, device: torch.device | str = "cuda:0"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError("the engine runs on a CUDA device only (there is no CPU path)")
        self.fast = dtype == torch.bfloat16 and os.environ.get("RLLM_B200_GENERIC_ONLY") != "1"
        self._sm100 = None
        if self.fast:
            from . import sm100          # builds/loads the tcgen05 library, or raises
            self._sm100 = sm100
            sm100.init(self.device)

    # ---- element-wise / row-wise
    def embed(self, ids, table, err=None):
        return ops.embed(ids, table, err=err)

    def rmsnorm(self, x, w, eps, out_dtype=None, rows=None):
        return ops.rmsnorm(x, w, eps, out_dtype or self.dtype, rows=rows)

    def normed(self, h, weight, eps, rows=None):
        """rmsnorm(h[rows]) for a consumer that may fuse it: deferred on the serving path, computed
        at once on the 32-bit path."""
        n = Normed(self, h, weight, eps, rows)
        return n if self._sm100 is not None else n.tensor()

    def _fused_norm(self, x, w, gate_up=False):
        """Take the norm into the product? Every CTA of the product then normalises its own slice of
        the rows, which pays while the weight has no more 128-row tiles than the GPU has SMs; a
        wider weight (the output head) gets the norm from its own kernel, once. So does a gate/up
        pair from 33 tokens on: its faster kernel there (tokens on the accumulator's rows, no ranges
        of K to merge) takes no norm in front (64 tokens: 14.8 us + the norm's 2 against 19.4)."""
        if gate_up and isinstance(x, Normed) and x.shape[0] > 32:
            return False
        if not (isinstance(x, Normed) and x._tensor is None and self._sm100 is not None
                and os.environ.get("RLLM_B200_NO_NORM_FUSION") != "1"
                and self._sm100.norm_supported(x.h, x.weight, w, x.rows)):
            return False
        # the kernel for steps of at most 8 tokens builds the normalised rows once per CTA whatever
        # the width (a CTA walks many slabs of the weight)
        return (w.shape[0] + 127) // 128 <= self._sm100.init(self.device).sm_count or \
            self._sm100.stream_supported(ops.EPI_STORE_F32, True, x.shape[0], w.shape[0], w.shape[1])

    def gather_rows(self, x, rows):
        return ops.gather_rows(x, rows)

    def add_into(self, residual, delta):
        return ops.add_into(residual, delta)

    # ---- matrix products: y = x W^T
    def _tc(self, x, w):
        return self._sm100 is not None and self._sm100.gemm_supported(x, w)

    def linear(self, x, w, bias=None):
        if bias is None and self._fused_norm(x, w):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w, ops.EPI_STORE, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            # a bias is added after the product (a small kernel): the product stays on the tensor cores
            y = self._sm100.gemm(x, w, ops.EPI_STORE)
            return y if bias is None else ops.add_bias(y, bias)
        return ops.gemm_simt(x, w, ops.EPI_STORE, bias=bias)

    def linear_f32(self, x, w):
        if self._fused_norm(x, w):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w, ops.EPI_STORE_F32, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            return self._sm100.gemm(x, w, ops.EPI_STORE_F32)
        return ops.gemm_simt(x, w, ops.EPI_STORE_F32)

    def linear_residual(self, x, w, residual):
        """residual (float32, in place) += x W^T"""
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w):
            return self._sm100.gemm(x, w, ops.EPI_ACCUM_F32, out=residual)
        return ops.gemm_simt(x, w, ops.EPI_ACCUM_F32, out=residual)

    def linear_swiglu(self, x, w_gate_up):
        """silu(x Wg^T) * (x Wu^T) with w_gate_up = [Wg; Wu]"""
        if self._fused_norm(x, w_gate_up, gate_up=True):
            return self._sm100.gemm_norm(x.h, x.weight, x.eps, w_gate_up, ops.EPI_SWIGLU, rows=x.rows)
        x = x.tensor() if isinstance(x, Normed) else x
        if self._tc(x, w_gate_up):
            return self._sm100.gemm(x, w_gate_up, ops.EPI_SWIGLU)
        return ops.gemm_simt(x, w_gate_up, ops.EPI_SWIGLU)

    # ---- position encoding + cache write, attention
    def rope_table(self, ctx, positions, inv_freq, rot_dim, key=None):
        """The step's (cos, sin) table for one rotation rule, made at its first use in a forward
        pass and shared by the layers with the same rule (`key`)."""
        if ctx is None:
            return None
        tables = ctx.per_forward.setdefault("rope_tables", {})
        key = key if key is not None else (inv_freq.data_ptr(), rot_dim)
        t = tables.get(key)
        if t is None:
            t = tables[key] = ops.rope_table(positions, inv_freq[: rot_dim // 2].contiguous(), ctx.num_tokens)
        return t

    def qkv_rope_cache_write(self, x, w_qkv, bias, positions, inv_freq, cache, nh, nkv, hd, rot_dim=None,
                             ctx=None, key=None):
        """qkv = x w_qkv^T (+ bias), q and k rotated, k and v written to the cache. One kernel when
        the tensor-core product takes the sizes, else the product followed by the rotation kernel."""
        rot_dim = hd if rot_dim is None else rot_dim
        table = self.rope_table(ctx, positions, inv_freq, rot_dim, key)
        kc = cache.k if cache.writes else None
        if bias is None and self._fused_norm(x, w_qkv) and x.rows is None and 128 % hd == 0 and \
                (kc is None or kc.dtype == torch.bfloat16):
            writes = cache.writes
            return self._sm100.gemm_qkv_rope(None, w_qkv, positions, inv_freq, cache.slots if writes else None,
                                             kc, cache.v if writes else None, nh, nkv, hd, cache.page_size,
                                             rot_dim, norm=(x.h, x.weight, x.eps), table=table)
        x = x.tensor() if isinstance(x, Normed) else x
        if bias is None and self._sm100 is not None and \
                self._sm100.qkv_rope_supported(x, w_qkv, cache.k if cache.writes else None, hd, rot_dim):
            writes = cache.writes
            return self._sm100.gemm_qkv_rope(x, w_qkv, positions, inv_freq, cache.slots if writes else None,
                                             cache.k if writes else None, cache.v if writes else None,
                                             nh, nkv, hd, cache.page_size, rot_dim, table=table)
        qkv = self.linear(x, w_qkv, bias=bias)
        self.rope_cache_write(qkv, positions, inv_freq, cache, nh, nkv, hd, rot_dim, ctx=ctx, key=key)
        return qkv

    def rope_cache_write(self, qkv, positions, inv_freq, cache, nh, nkv, hd, rot_dim=None, ctx=None, key=None):
        writes = cache.writes
        rot_dim = hd if rot_dim is None else rot_dim
        table = self.rope_table(ctx, positions, inv_freq, rot_dim, key)
        ops.rope_cache_write(qkv, positions, inv_freq, cache.slots if writes else None,
                             cache.k if writes else None, cache.v if writes else None,
                             nh, nkv, hd, cache.page_size, rot_dim, table=table)

    def attention(self, q, cache, ctx, nh, scale, window):
        if self._sm100 is not None:
            out = self._sm100.attention(q, cache, ctx, nh, scale, window)
            if out is not None:
                return out
        return ops.paged_attention_simt(q, cache.k, cache.v, ctx.token_seq, ctx.positions,
                                        cache.block_table, nh, scale, window)

    # ---- selection
    def argmax(self, logits):
        return ops.argmax(logits)

    def add_at(self, logits, rows, cols, vals):
        return ops.add_at(logits, rows, cols, vals)

    def logprobs(self, logits, temperature, top_k, chosen, rows, n_top):
        return ops.logprobs(logits, temperature, top_k, chosen, rows, n_top)

    def sample(self, logits, temperature, uniform, top_k=None, top_p=None, min_p=None, out=None):
        return ops.sample(logits, temperature, uniform, top_k, top_p, min_p, out=out)
