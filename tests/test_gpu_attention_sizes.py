"""The attention kernels at the sizes the benchmark runs, which the other kernel tests stay far
below: decode over 4,096, 8,192 and some 20,000 keys with the number of key ranges left to the
kernel's own choice and the largest key count given as a CUDA graph gives it (the block table's
capacity, not the real lengths); prefill on tcgen05 over 4,096 and 8,192 keys, with a portion that
starts after 3,000 keys already in the cache. Against the plain formula for the rows of the step."""
import pytest
import torch

import plain_llama as P
from test_gpu_kernels import scattered_cache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 8e-3


def rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max()) / max(float(b.abs().max()), 1e-30)


def capacity(longest, page):
    """What a decode graph passes as the largest key count: pages rounded up to a power of two (from 8)."""
    pages, p = (longest + page - 1) // page, 8
    while p < pages:
        p *= 2
    return p * page


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("longest", [4096, 8192, 20000])
def test_decode_at_benchmark_sizes(hd, longest):
    from rllm_b200.kernels import sm100
    nh, nkv, page = 32, 8, 16
    lens = [longest, longest - 96, 37, longest // 2 + 1, longest - 1, 1, (3 * longest) // 4, 512]
    S = len(lens)
    kc, vc, bt, ks, vs = scattered_cache(S, lens, nkv, hd, page, torch.bfloat16, seed=hd + longest)
    g = torch.Generator().manual_seed(4)
    q = torch.randn(S, nh, hd, generator=g).to(torch.bfloat16)
    # a far key that must dominate: sequence 0, key 5 (it lies in the first of the key ranges)
    ks[0][5] = 0
    ks[0][5, :, 0] = 30.0
    q[0, :, 0] = 30.0
    kc[int(bt[0, 5 // page]), :, 5 % page] = ks[0][5]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    cap = capacity(longest, page)
    wide = torch.full((S, cap // page), -1, dtype=torch.int32)       # the table as wide as the graph's
    wide[:, : bt.shape[1]] = bt
    st = sm100.init(DEV)
    chosen = sm100.decode_splits(S, nkv, cap, st.sm_count)
    assert chosen >= 2                                               # ranges are in play at these lengths
    out = sm100.attention_decode(q.reshape(S, nh * hd).to(DEV), kc.to(DEV), vc.to(DEV), i32(lens), wide.to(DEV), nh,
                                 hd ** -0.5, None, cap)              # splits: the kernel's own choice
    sm100.check_error(DEV)
    for s in range(S):
        ref = P.attention_tail(q[s: s + 1].float(), ks[s].float(), vs[s].float(), hd ** -0.5)[0]
        got = out[s].float().cpu().view(nh, hd)
        assert torch.isfinite(got).all()
        assert rel(got, ref) <= TOL, f"sequence {s} (len {lens[s]})"
    assert rel(out[0].float().cpu().view(nh, hd), vs[0][5].float().repeat_interleave(nh // nkv, 0)) <= TOL


@pytest.mark.parametrize("hd,nh,nkv", [(64, 8, 2), (128, 4, 1)])
@pytest.mark.parametrize("keys,cached", [(4096, 0), (4096, 3000), (8192, 3000)])
def test_prefill_on_tcgen05_at_benchmark_sizes(hd, nh, nkv, keys, cached):
    """One long portion (rows cached .. keys-1) beside a short sequence; a far key among the cached
    ones dominates the last row."""
    from rllm_b200.kernels import sm100
    page = 16
    lens, q_lens = [keys, 200], [keys - cached, 200]
    kc, vc, bt, ks, vs = scattered_cache(2, lens, nkv, hd, page, torch.bfloat16, seed=hd + keys + cached)
    g = torch.Generator().manual_seed(9)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(torch.bfloat16)
    j = 11
    ks[0][j] = 0
    ks[0][j, :, 0] = 30.0
    q[q_lens[0] - 1, :, 0] = 30.0
    kc[int(bt[0, j // page]), :, j % page] = ks[0][j]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    out = sm100.attention_prefill_tc(q.reshape(T, nh * hd).to(DEV), kc.to(DEV), vc.to(DEV), i32([0, q_lens[0], T]),
                                     i32(lens), bt.to(DEV), max(q_lens), nh, hd ** -0.5, None)
    sm100.check_error(DEV)
    row = 0
    for s in range(2):
        n = q_lens[s]
        ref = P.attention_tail(q[row: row + n].float(), ks[s].float(), vs[s].float(), hd ** -0.5)
        got = out[row: row + n].float().cpu().view(n, nh, hd)
        assert torch.isfinite(got).all()
        assert rel(got, ref) <= TOL, f"sequence {s}"
        row += n
    assert rel(out[q_lens[0] - 1].float().cpu().view(nh, hd), vs[0][j].float().repeat_interleave(nh // nkv, 0)) <= TOL
