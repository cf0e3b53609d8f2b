"""Each CUDA kernel alone against its plain float32 formula, at sizes other than the
engine's: widths and vocabularies that are no power of two, odd head counts, head sizes in
steps of 16, pages of odd size, scattered pages. Inputs are shaped so that a fault shows:
one far key made to dominate, a window's edge, a tie for the maximum."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative to the largest reference magnitude; bfloat16 inputs are identical in both,
# so only the single rounding of the output (2^-9) and accumulation order remain
TOL = {"float32": 2e-6, "bfloat16": 6e-3}


def ops():
    from rllm_b200.kernels import ops as o
    return o


def rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max()) / max(float(b.abs().max()), 1e-30)


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", list(DT))
def test_embed(dtype):
    table = rnd(1000, 200, dtype=DT[dtype])
    ids = torch.tensor([0, 999, 17, 17, 503], dtype=torch.int32)
    out = ops().embed(ids.to(DEV), table.to(DEV))
    assert out.dtype == torch.float32 and torch.equal(out.cpu(), P.embedding(table.float(), ids))
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = ops().embed(torch.tensor([3, 1000, -1], dtype=torch.int32, device=DEV), table.to(DEV), err=err)
    assert int(err) == 1 and float(out[1:].abs().sum()) == 0.0      # flagged, nothing read outside


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("T,H,eps", [(1, 48, 1e-5), (7, 1000, 1e-6), (3, 4100, 3e-2)])
def test_rmsnorm(dtype, T, H, eps):
    x = rnd(T, H, seed=1, scale=3.0)
    w = (1 + rnd(H, seed=2, scale=0.3)).to(DT[dtype])
    out = ops().rmsnorm(x.to(DEV), w.to(DEV), eps, DT[dtype])
    assert rel(out, P.rms_norm(x, w.float(), eps)) <= TOL[dtype]
    out32 = ops().rmsnorm(x.to(DEV), w.float().to(DEV), eps, torch.float32)   # weight kept in 32-bit
    assert rel(out32, P.rms_norm(x, w.float(), eps)) <= 2e-6
    # chosen rows only (the output head normalises the wanted rows): the same values, row by row
    rows = torch.tensor([T - 1, 0, T - 1], dtype=torch.int32)
    picked = ops().rmsnorm(x.to(DEV), w.float().to(DEV), eps, torch.float32, rows=rows.to(DEV))
    assert torch.equal(picked, out32[rows.long()])


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("T,N,K", [(1, 100, 72), (70, 130, 200), (5, 64, 16), (129, 66, 1030)])
def test_gemm_simt_all_epilogues(dtype, T, N, K):
    o = ops()
    a = rnd(T, K, dtype=DT[dtype], seed=3)
    w = rnd(2 * N, K, dtype=DT[dtype], seed=4, scale=K ** -0.5)
    ref = P.linear(a.float(), w[:N].float())
    ad, wd = a.to(DEV), w.to(DEV)
    assert rel(o.gemm_simt(ad, wd[:N].contiguous(), o.EPI_STORE), ref) <= TOL[dtype]
    out32 = o.gemm_simt(ad, wd[:N].contiguous(), o.EPI_STORE_F32)
    assert out32.dtype == torch.float32 and rel(out32, ref) <= 2e-6
    res = rnd(T, N, seed=5)
    got = o.gemm_simt(ad, wd[:N].contiguous(), o.EPI_ACCUM_F32, out=res.to(DEV).clone())
    assert rel(got, res + ref) <= 2e-6
    g, u = ref, P.linear(a.float(), w[N:].float())
    assert rel(o.gemm_simt(ad, wd, o.EPI_SWIGLU), g / (1 + torch.exp(-g)) * u) <= TOL[dtype]
    bias = rnd(N, dtype=DT[dtype], seed=6)
    assert rel(o.gemm_simt(ad, wd[:N].contiguous(), o.EPI_STORE, bias=bias.to(DEV)), ref + bias.float()) <= TOL[dtype]
    # a row's result does not depend on the rows beside it
    one = o.gemm_simt(ad[T // 2: T // 2 + 1], wd[:N].contiguous(), o.EPI_STORE_F32)
    assert torch.equal(one[0], out32[T // 2])


def scattered_cache(n_seqs, lens, nkv, hd, page, dtype, seed=0, extra_pages=5):
    """Random K/V for sequences of the given lengths in a cache whose pages are scattered."""
    g = torch.Generator().manual_seed(seed)
    per = [math.ceil(l / page) for l in lens]
    total = sum(per) + extra_pages
    perm = torch.randperm(total, generator=g).tolist()
    kc = torch.full((total, nkv, page, hd), 7.0).to(dtype)      # junk in unused slots
    vc = torch.full((total, nkv, page, hd), -7.0).to(dtype)
    bt = torch.full((n_seqs, max(per)), -1, dtype=torch.int32)
    ks, vs = [], []
    for s, l in enumerate(lens):
        k = (torch.randn(l, nkv, hd, generator=g)).to(dtype)
        v = (torch.randn(l, nkv, hd, generator=g)).to(dtype)
        ks.append(k); vs.append(v)
        for i in range(per[s]):
            pg = perm.pop()
            bt[s, i] = pg
            n = min(page, l - i * page)
            kc[pg, :, :n] = k[i * page: i * page + n].transpose(0, 1)
            vc[pg, :, :n] = v[i * page: i * page + n].transpose(0, 1)
    return kc, vc, bt, ks, vs


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nh,nkv,hd,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 5, 24), (8, 8, 80, 16, None),
    (5, 5, 128, 32, 100), (2, 1, 256, 16, None)])
def test_paged_attention_simt(dtype, nh, nkv, hd, page, window):
    """Mixed batch: a whole prompt, a late portion of a long sequence, single decode tokens."""
    lens = [37, 300, 1, 130, 64]         # keys visible to each sequence's last token
    q_lens = [37, 9, 1, 1, 2]            # of which this step brings the last q_len
    kc, vc, bt, ks, vs = scattered_cache(5, lens, nkv, hd, page, DT[dtype], seed=hd)
    g = torch.Generator().manual_seed(99)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(DT[dtype])
    # one far key dominates: query row of sequence 1 points at key 11 of 300
    far_row = q_lens[0] + 4
    if window is None:
        ks[1][11, :] = 0
        ks[1][11, :, 0] = 30.0
        q[far_row, :, 0] = 30.0
        pg = int(bt[1, 11 // page]); kc[pg, :, 11 % page] = ks[1][11]
    token_seq = torch.tensor([s for s, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32)
    positions = torch.tensor([lens[s] - q_lens[s] + i for s in range(5) for i in range(q_lens[s])],
                             dtype=torch.int32)
    scale = hd ** -0.5
    out = ops().paged_attention_simt(q.reshape(T, nh * hd).to(DEV), kc.to(DEV), vc.to(DEV),
                                     token_seq.to(DEV), positions.to(DEV), bt.to(DEV), nh, scale, window)
    row = 0
    for s in range(5):
        L, n = lens[s], q_lens[s]
        qf = torch.zeros(L, nh, hd); qf[L - n:] = q[row: row + n].float()
        ref = P.attention(qf, ks[s].float(), vs[s].float(), scale, window)[L - n:]
        got = out[row: row + n].float().cpu().view(n, nh, hd)
        assert rel(got, ref) <= TOL[dtype], f"sequence {s}"
        row += n
    if window is None:
        got = out[far_row].float().cpu().view(nh, hd)
        want = vs[1][11].float().repeat_interleave(nh // nkv, 0)
        assert rel(got, want) <= TOL[dtype]          # the far key's value comes through alone


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nh,nkv,hd,page,rot", [(4, 2, 16, 16, None), (3, 1, 32, 8, None),
                                                (5, 5, 48, 4, None), (2, 1, 64, 16, 32)])
def test_rope_and_cache_write(dtype, nh, nkv, hd, page, rot):
    o = ops()
    T = 11
    rot_dim = rot or hd
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=DT[dtype], seed=7)
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 31, 32, 33, 4095, 7], dtype=torch.int32)
    inv_freq = P.rope_inv_freq(rot_dim, 500000.0, {"rope_type": "llama3", "factor": 8.0,
                               "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 32})
    pages = 9
    slots = torch.tensor([5 * page + 0, 5 * page + 1, 2 * page + page - 1, 0, 8 * page + 2,
                          8 * page + 3, 1 * page + 1, 7 * page, -1, 3 * page + 1, 4 * page],
                         dtype=torch.int32)
    kc = torch.zeros(pages, nkv, page, hd, dtype=DT[dtype], device=DEV)
    vc = torch.zeros_like(kc)
    buf = qkv.to(DEV).clone()
    o.rope_cache_write(buf, positions.to(DEV), inv_freq.to(DEV), slots.to(DEV), kc, vc, nh, nkv, hd,
                       page, rot_dim)
    q = qkv[:, : nh * hd].float().view(T, nh, hd)
    k = qkv[:, nh * hd: (nh + nkv) * hd].float().view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)

    def rope(x):
        r = P.rope(x[..., :rot_dim], positions, inv_freq)
        return torch.cat([r, x[..., rot_dim:]], -1)

    assert rel(buf[:, : nh * hd].view(T, nh, hd), rope(q)) <= TOL[dtype]
    assert torch.equal(buf[:, nh * hd:].cpu(), qkv[:, nh * hd:])            # k, v rows untouched
    kr = rope(k)
    written = torch.zeros(pages, page, dtype=torch.bool)
    for t in range(T):
        if slots[t] < 0:
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        written[pg, off] = True
        assert rel(kc[pg, :, off], kr[t]) <= TOL[dtype]
        assert torch.equal(vc[pg, :, off].cpu(), v[t])
    assert float(kc.float().cpu()[~written[:, None, :].expand(-1, nkv, -1)].abs().sum()) == 0.0
    # with the step's table of angles instead of angles computed in the kernel: the same bits
    table = o.rope_table(positions.to(DEV), inv_freq[: rot_dim // 2].contiguous().to(DEV), T)
    ang = positions.float()[:, None] * inv_freq[: rot_dim // 2].float()[None, :]
    assert rel(table[..., 0], torch.cos(ang.double()).float()) <= 2e-6
    assert rel(table[..., 1], torch.sin(ang.double()).float()) <= 2e-6
    kc2, vc2, buf2 = torch.zeros_like(kc), torch.zeros_like(vc), qkv.to(DEV).clone()
    o.rope_cache_write(buf2, positions.to(DEV), inv_freq.to(DEV), slots.to(DEV), kc2, vc2, nh, nkv, hd,
                       page, rot_dim, table=table)
    assert torch.equal(buf2, buf) and torch.equal(kc2, kc) and torch.equal(vc2, vc)


def test_argmax_lowest_index_wins_and_large_vocab():
    V = 128256
    x = rnd(3, V, seed=8)
    x[0, 77] = x[0, 90000] = 50.0                  # a tie: the lower index
    x[1, V - 1] = 60.0
    x[2] = -5.0                                    # all equal: index 0
    assert ops().argmax(x.to(DEV)).tolist() == [77, V - 1, 0]
    y = rnd(5, 777, seed=9)
    assert ops().argmax(y.to(DEV)).tolist() == torch.argmax(y, -1).tolist()


@pytest.mark.parametrize("V", [256, 1000, 50257, 128256, 300000])
@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [
    (1.0, 0, 1.0, 0.0), (0.8, 0, 1.0, 0.0), (1.3, 40, 1.0, 0.0), (1.0, 0, 0.9, 0.0),
    (0.7, 0, 1.0, 0.05), (1.1, 50, 0.8, 0.02), (1.0, 1, 1.0, 0.0)])
def test_sample_follows_the_reference_pipeline(V, temperature, top_k, top_p, min_p):
    R = 64
    logits = rnd(1, V, seed=V, scale=2.5).repeat(R, 1)
    us = torch.linspace(0.0, 0.999, R)
    f = lambda v, dt: torch.full((R,), v, dtype=dt, device=DEV)
    got = ops().sample(logits.to(DEV), f(temperature, torch.float32), us.to(DEV),
                       f(top_k, torch.int32) if top_k else None,
                       f(top_p, torch.float32) if top_p < 1 else None,
                       f(min_p, torch.float32) if min_p > 0 else None).tolist()
    p = P.sample_probs(logits[0], temperature, top_k, top_p, min_p).double()
    cdf = torch.cumsum(p, 0)
    eps = 2e-5      # float rounding of the running sums; a draw this close to an edge may go either way
    for u, tok in zip(us.tolist(), got):
        assert p[tok] > 0, f"token {tok} has no mass after filtering (u={u})"
        lo = float(cdf[tok - 1]) if tok else 0.0
        assert lo - eps <= u <= float(cdf[tok]) + eps, (u, tok, lo, float(cdf[tok]))
    if top_k == 1:
        assert set(got) == {int(torch.argmax(logits[0]))}


def test_sample_rows_have_their_own_parameters():
    V = 500
    logits = rnd(4, V, seed=11, scale=3.0)
    temp = torch.tensor([0.5, 1.0, 1.5, 1.0])
    top_k = torch.tensor([0, 5, 0, 0], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.5, 1.0])
    u = torch.tensor([0.3, 0.6, 0.9, 0.1])
    got = ops().sample(logits.to(DEV), temp.to(DEV), u.to(DEV), top_k.to(DEV), top_p.to(DEV), None).tolist()
    for r in range(4):
        p = P.sample_probs(logits[r], float(temp[r]), int(top_k[r]), float(top_p[r]), 0.0).double()
        cdf = torch.cumsum(p, 0)
        lo = float(cdf[got[r] - 1]) if got[r] else 0.0
        assert p[got[r]] > 0 and lo - 2e-5 <= float(u[r]) <= float(cdf[got[r]]) + 2e-5


@pytest.mark.parametrize("V", [200, 1000, 128256])
def test_logprobs_of_the_chosen_token_and_of_the_most_probable(V):
    """Rows with their own temperature (0 among them), top-k and chosen token; only some rows are
    listed; a tie among the largest goes by rising index; top-k leaves fewer tokens than asked for."""
    import math
    R = 6
    logits = rnd(R, V, seed=V + 1, scale=3.0)
    logits[2, 7] = logits[2, 150] = logits[2].max() + 1.0        # two equal at the top
    temp = torch.tensor([1.0, 0.0, 0.7, 1.5, 1.0, 0.9])
    top_k = torch.tensor([0, 0, 0, 3, 50, 0], dtype=torch.int32)
    chosen = torch.tensor([int(torch.argmax(logits[0])), int(torch.argmax(logits[1])), 150, 5, 11, V - 1], dtype=torch.int32)
    chosen[3] = int(torch.topk(logits[3], 2).indices[1])         # inside its top-k of 3; row 4's token 11 is outside
    rows = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32)
    for n_top in (0, 5, 20):
        lp, ids = ops().logprobs(logits.to(DEV), temp.to(DEV), top_k.to(DEV), chosen.to(DEV), rows.to(DEV), n_top)
        assert lp.shape == (5, 1 + n_top) and ids.shape == (5, n_top)
        lp, ids = lp.cpu(), ids.cpu()
        for i, r in enumerate(rows.tolist()):
            want_lp, want_top = P.logprobs(logits[r], float(temp[r]), int(top_k[r]), int(chosen[r]), n_top)
            if want_lp == float("-inf"):
                assert float(lp[i, 0]) == float("-inf")
            else:
                assert abs(float(lp[i, 0]) - want_lp) <= 1e-4
            got = [(int(t), float(v)) for t, v in zip(ids[i], lp[i, 1:]) if int(t) >= 0]
            assert [t for t, _ in got] == [t for t, _ in want_top], (r, n_top)
            assert all(abs(a[1] - b[1]) <= 1e-4 for a, b in zip(got, want_top))
            assert all(int(t) == -1 and float(v) == float("-inf")
                       for t, v in zip(ids[i, len(got):], lp[i, 1 + len(got):]))
        if n_top >= 5:
            assert ids[2, :2].tolist() == [7, 150] and len([t for t in ids[3] if t >= 0]) == 3
        assert float(lp[4, 0]) == float("-inf") or int(chosen[4]) in torch.topk(logits[4], 50).indices.tolist()
    # probabilities of a whole small row add up to 1
    small = rnd(1, 19, seed=3)
    lp, ids = ops().logprobs(small.to(DEV), torch.ones(1, device=DEV), None, torch.zeros(1, dtype=torch.int32, device=DEV),
                             torch.zeros(1, dtype=torch.int32, device=DEV), 19)
    assert sorted(ids[0].tolist()) == list(range(19))
    assert abs(sum(math.exp(v) for v in lp[0, 1:].tolist()) - 1.0) <= 1e-5


def test_kernels_refuse_what_they_cannot_take():
    o = ops()
    with pytest.raises(o.KernelError):
        o.embed(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4))            # CPU tensors
    with pytest.raises(o.KernelError):
        o.gemm_simt(torch.zeros(2, 8, device=DEV), torch.zeros(4, 9, device=DEV), o.EPI_STORE)
    with pytest.raises(o.KernelError):
        o.rmsnorm(torch.zeros(2, 8, device=DEV, dtype=torch.float16), torch.ones(8, device=DEV), 1e-5,
                  torch.float32)
    q = torch.zeros(1, 2 * 24, device=DEV)
    kc = torch.zeros(2, 1, 4, 24, device=DEV)                                      # head size 24: no
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(o.KernelError):
        o.paged_attention_simt(q, kc, kc, z, z, z.view(1, 1), 2, 1.0, None)


@pytest.mark.parametrize("dtype", list(DT))
def test_add_bias_in_place_on_a_strided_view(dtype):
    from rllm_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    big = torch.randn(9, 150, generator=g).to(DT[dtype])
    b = torch.randn(70, generator=g).to(DT[dtype])
    d = big.to(DEV)
    ops.add_bias(d[:, 40:110], b.to(DEV))
    want = big.clone()
    want[:, 40:110] = (big[:, 40:110].float() + b.float()).to(DT[dtype])
    assert torch.equal(d.cpu(), want)
    with pytest.raises(ops.KernelError):
        ops.add_bias(d[:, :70], b.float().to(DEV) if dtype != "float32" else b.to(torch.bfloat16).to(DEV))


def test_check_meta_makes_bad_entries_harmless_and_names_the_first():
    from rllm_b200.kernels import ops
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    table = i32([[0, 5, -1, 9], [3, 10, -2, 1]])                 # 10 pages: entries 10 and -2 are out
    slots = i32([0, 159, 160, -1, -7])                            # 10 pages of 16: slots 160 and -7 are out
    err = i32([0])
    ops.check_meta(table, slots, 10, 16, err)
    assert table.tolist() == [[0, 5, -1, 9], [3, -1, -1, 1]] and slots.tolist() == [0, 159, -1, -1, -1]
    code = int(err.item())
    assert code in (1 + 5, 1 + 6, 0x40000000 | 2, 0x40000000 | 4)           # one of the offenders, whichever came first
    err.zero_()
    ops.check_meta(table, slots, 10, 16, err)
    assert int(err.item()) == 0
