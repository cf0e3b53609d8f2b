"""The allocation-free attention entry point, called the way its users call it: through the
exported C symbol `rllm_attention_fa_noalloc`, with raw pointers and a stream, no Python
wrapper in between.

It serves callers that cannot call cudaMalloc (a host that owns all device memory through its
own pool, a plug-in running inside another program's capture or memory-pool scope, a loop that
must not take the allocator's lock): the scratch for the partial sums of the key ranges is a
fixed array inside the library instead of two buffers from the caller. The test runs the same
batch through it and through the ordinary entry point `rllm_attention_fa` (which gets its
scratch from the caller) and requires equal output, and output equal to the plain formula of
tests/plain_llama.py, twice in a row with different data, because the fixed array keeps what
the previous call left in it. It also checks that a problem
beyond the fixed array is refused before anything runs.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_gpu_kernels import scattered_cache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 8e-3      # the tolerance of the tiled attention's own tests; the two paths are in fact bit-equal

_P = c_void_p
_COMMON = [_P, c_int, _P, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
           c_int, c_float, c_int, c_int]


def _symbols():
    from rllm_b200.kernels import build
    lib = build.load_library("sm100")
    plain = lib.rllm_attention_fa
    plain.restype = c_int
    plain.argtypes = _COMMON + [_P, _P, _P]           # ..., part_o, part_ml, stream
    noalloc = lib.rllm_attention_fa_noalloc
    noalloc.restype = c_int
    noalloc.argtypes = _COMMON + [_P]                 # ..., stream
    return plain, noalloc


def _batch(seed, lens, q_lens, nh, nkv, hd, page):
    S = len(lens)
    kc, vc, bt, ks, vs = scattered_cache(S, lens, nkv, hd, page, torch.bfloat16, seed=seed)
    g = torch.Generator().manual_seed(seed)
    T = sum(q_lens)
    q = torch.randn(T, nh * hd, generator=g).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return dict(q=q.to(DEV), kc=kc.to(DEV), vc=vc.to(DEV), bt=bt.to(DEV).contiguous(), cu=i32(cu), lens=i32(lens),
                S=S, T=T, max_q=max(q_lens), q_host=q, ks=ks, vs=vs, lens_host=lens, q_lens=q_lens, cu_host=cu)


def _args(b, out, nh, nkv, hd, page, splits, window=0):
    return [b["q"].data_ptr(), b["q"].stride(0), b["kc"].data_ptr(), b["vc"].data_ptr(), out.data_ptr(),
            out.stride(0), b["cu"].data_ptr(), b["lens"].data_ptr(), b["bt"].data_ptr(), b["bt"].stride(0),
            b["S"], b["T"], b["max_q"], nh, nkv, hd, page, float(hd ** -0.5), window, splits]


def _plain(b, nh, hd, window):
    """The plain formula over whole sequences (tests/plain_llama.py), the step's rows cut out."""
    import plain_llama as P
    rows = []
    for s, (L, n) in enumerate(zip(b["lens_host"], b["q_lens"])):
        qf = torch.zeros(L, nh, hd)
        qf[L - n:] = b["q_host"][b["cu_host"][s]: b["cu_host"][s + 1]].float().view(n, nh, hd)
        rows.append(P.attention(qf, b["ks"][s].float(), b["vs"][s].float(), hd ** -0.5, window or None)[L - n:])
    return torch.cat(rows).reshape(b["T"], nh * hd)


# two calls in a row per case, with different data: single tokens; portions beside single tokens; a
# window; and sequences so short that some of the key ranges are empty
CASES = [
    (32, 8, 64, 16, 4, 0, [([1, 63, 300, 129, 700], [1, 1, 1, 1, 1]), ([640, 2, 65, 64, 257], [1, 1, 1, 1, 1])]),
    (8, 2, 128, 8, 3, 0, [([1, 63, 300, 129, 700], [1, 1, 1, 1, 1]), ([640, 2, 65, 64, 257], [1, 1, 1, 1, 1])]),
    (8, 2, 64, 16, 3, 0, [([40, 300, 9, 130], [40, 7, 1, 2]), ([200, 64, 33], [3, 1, 33])]),
    (4, 1, 128, 8, 4, 50, [([150, 97, 23, 64], [1, 1, 1, 1]), ([300, 51, 50, 49], [5, 1, 2, 1])]),
    (16, 4, 64, 16, 8, 0, [([65, 1, 2, 130], [1, 1, 1, 1]), ([64, 66, 1, 1], [1, 1, 1, 1])]),
]


@pytest.mark.parametrize("nh,nkv,hd,page,splits,window,calls", CASES)
def test_noalloc_entry_equals_the_ordinary_one_twice_in_a_row(nh, nkv, hd, page, splits, window, calls):
    """Against the ordinary entry point (same kernels, scratch from the caller) and against the plain
    formula, which shares nothing with either."""
    plain, noalloc = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lens, q_lens) in enumerate(calls):
        b = _batch(11 + call, lens, q_lens, nh, nkv, hd, page)
        T = b["T"]
        want = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
        part_o = torch.empty(T * nh * splits * hd, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(T * nh * splits * 2, dtype=torch.float32, device=DEV)
        rc = plain(*_args(b, want, nh, nkv, hd, page, splits, window), part_o.data_ptr(), part_ml.data_ptr(), stream)
        assert rc == 0
        got = torch.zeros_like(want)
        rc = noalloc(*_args(b, got, nh, nkv, hd, page, splits, window), stream)
        assert rc == 0, f"call {call}: refused or failed with {rc}"
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max()) / max(float(want.float().abs().max()), 1e-30)
        assert err <= TOL, f"call {call}: differs from the ordinary entry point by {err:.3e}"
        ref = _plain(b, nh, hd, window)
        err = float((got.float().cpu() - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
        assert err <= TOL, f"call {call}: differs from the plain formula by {err:.3e}"


def test_noalloc_entry_refuses_what_its_array_cannot_hold():
    _, noalloc = _symbols()
    nh, nkv, hd, page, splits = 32, 8, 128, 16, 64
    b = _batch(3, [40] * 40, [1] * 40, nh, nkv, hd, page)          # 40 * 32 * 64 * 128 floats > 2 Mi
    out = torch.full((b["S"], nh * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = noalloc(*_args(b, out, nh, nkv, hd, page, splits), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -4                                      # "problem too large", nothing was launched
    assert float((out.float() - 7.0).abs().max()) == 0.0
