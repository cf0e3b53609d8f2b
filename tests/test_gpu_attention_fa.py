"""The tiled tensor-core attention alone against the plain formula: head sizes 64 and 128,
group sizes 1 to 8, pages of 16, 8, 5 and 32 positions scattered over the pool, windows,
prompt portions beside decode tokens, and the keys of a sequence cut into 1 to 7 ranges."""
import pytest
import torch

import plain_llama as P
from test_gpu_kernels import scattered_cache

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 8e-3      # bf16 probabilities and output; inputs are the same bf16 values on both sides


def rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max()) / max(float(b.abs().max()), 1e-30)


def run(nh, nkv, hd, page, window, lens, q_lens, splits, far=None, kernel="fa"):
    from rllm_b200.kernels import sm100
    S = len(lens)
    kc, vc, bt, ks, vs = scattered_cache(S, lens, nkv, hd, page, torch.bfloat16, seed=hd + nh)
    g = torch.Generator().manual_seed(5)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    if far is not None:          # (sequence, key index): that key dominates the sequence's last query
        s_, j = far
        ks[s_][j] = 0
        ks[s_][j, :, 0] = 30.0
        q[cu[s_ + 1] - 1, :, 0] = 30.0
        kc[int(bt[s_, j // page]), :, j % page] = ks[s_][j]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    # the q rows sit inside a wider buffer, as in the engine's qkv tensor
    buf = torch.zeros(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16)
    buf[:, : nh * hd] = q.reshape(T, nh * hd)
    bufd = buf.to(DEV)
    if kernel == "tc":
        out = sm100.attention_prefill_tc(bufd[:, : nh * hd], kc.to(DEV), vc.to(DEV), i32(cu), i32(lens), bt.to(DEV),
                                         max(q_lens), nh, hd ** -0.5, window)
        sm100.check_error(DEV)
    else:
        out = sm100.attention_fa(bufd[:, : nh * hd], kc.to(DEV), vc.to(DEV), i32(cu), i32(lens), bt.to(DEV), T,
                                 max(q_lens), max(lens), nh, hd ** -0.5, window, splits=splits)
    row = 0
    for s in range(S):
        L, n = lens[s], q_lens[s]
        qf = torch.zeros(L, nh, hd); qf[L - n:] = q[row: row + n].float()
        ref = P.attention(qf, ks[s].float(), vs[s].float(), hd ** -0.5, window)[L - n:]
        got = out[row: row + n].float().cpu().view(n, nh, hd)
        assert torch.isfinite(got).all()
        assert rel(got, ref) <= TOL, f"sequence {s} (len {L}, q {n})"
        row += n
    if far is not None:
        s_, j = far
        got = out[cu[s_ + 1] - 1].float().cpu().view(nh, hd)
        assert rel(got, vs[s_][j].float().repeat_interleave(nh // nkv, 0)) <= TOL
    return out


@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 64, 16), (4, 2, 64, 8), (3, 1, 64, 5), (8, 8, 128, 16),
                                            (24, 8, 128, 32), (16, 2, 64, 16), (6, 2, 128, 8)])
def test_mixed_batch(nh, nkv, hd, page):
    run(nh, nkv, hd, page, None, lens=[37, 300, 1, 130, 64, 200], q_lens=[37, 9, 1, 1, 2, 200], splits=1,
        far=(1, 11))


@pytest.mark.parametrize("window", [24, 64, 100])
@pytest.mark.parametrize("hd", [64, 128])
def test_window(window, hd):
    run(8, 2, hd, 8, window, lens=[150, 97, 23, 64], q_lens=[150, 1, 23, 5], splits=1)


@pytest.mark.parametrize("splits", [1, 2, 3, 7])
@pytest.mark.parametrize("nh,nkv,hd,page", [(32, 8, 64, 16), (8, 1, 128, 8), (3, 1, 64, 5)])
def test_decode_with_split_keys(splits, nh, nkv, hd, page):
    run(nh, nkv, hd, page, None, lens=[1, 63, 64, 65, 700, 129], q_lens=[1, 1, 1, 1, 1, 1], splits=splits,
        far=(4, 5))
    run(nh, nkv, hd, page, 50, lens=[1, 63, 64, 65, 700, 129], q_lens=[1, 1, 1, 1, 1, 1], splits=splits)


@pytest.mark.parametrize("splits", [1, 2, 3, 8, 12, 16])
@pytest.mark.parametrize("nh,nkv,hd,page,window", [
    (32, 8, 64, 16, None), (8, 1, 128, 8, None), (3, 1, 64, 32, None), (16, 1, 64, 64, 100),
    (4, 4, 128, 16, 70), (12, 4, 64, 8, None), (6, 2, 128, 32, None), (6, 2, 64, 5, None), (2, 1, 128, 3, 40)])
def test_decode_kernel_with_cluster_merge(splits, nh, nkv, hd, page, window):
    """The TMA-fed decode kernel against the plain formula: lengths on both sides of a tile and
    of a page, one sequence of a single key, scattered pages, windows, and a far key that must
    dominate (it lies in another range than the query's own position)."""
    from rllm_b200.kernels import sm100
    lens = [1, 63, 64, 65, 700, 129, 1000, 17]
    S = len(lens)
    kc, vc, bt, ks, vs = scattered_cache(S, lens, nkv, hd, page, torch.bfloat16, seed=hd + nh + page)
    g = torch.Generator().manual_seed(6)
    q = torch.randn(S, nh, hd, generator=g).to(torch.bfloat16)
    far = None
    if window is None:
        far = (4, 5)
        ks[4][5] = 0
        ks[4][5, :, 0] = 30.0
        q[4, :, 0] = 30.0
        kc[int(bt[4, 5 // page]), :, 5 % page] = ks[4][5]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    buf = torch.zeros(S, (nh + 2 * nkv) * hd, dtype=torch.bfloat16)
    buf[:, : nh * hd] = q.reshape(S, nh * hd)
    bufd = buf.to(DEV)
    out = sm100.attention_decode(bufd[:, : nh * hd], kc.to(DEV), vc.to(DEV), i32(lens), bt.to(DEV), nh,
                                 hd ** -0.5, window, max(lens), splits=splits)
    sm100.check_error(DEV)
    for s in range(S):
        L = lens[s]
        qf = torch.zeros(L, nh, hd); qf[L - 1] = q[s].float()
        ref = P.attention(qf, ks[s].float(), vs[s].float(), hd ** -0.5, window)[L - 1]
        got = out[s].float().cpu().view(nh, hd)
        assert torch.isfinite(got).all()
        assert rel(got, ref) <= TOL, f"sequence {s} (len {L})"
    if far is not None:
        got = out[4].float().cpu().view(nh, hd)
        assert rel(got, vs[4][5].float().repeat_interleave(nh // nkv, 0)) <= TOL
    # the same call again: same bits (the merge order is fixed)
    again = sm100.attention_decode(bufd[:, : nh * hd], kc.to(DEV), vc.to(DEV), i32(lens), bt.to(DEV), nh,
                                   hd ** -0.5, window, max(lens), splits=splits)
    assert torch.equal(out, again)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv,page,window", [(32, 8, 16, None), (6, 2, 8, None), (3, 1, 5, None), (8, 8, 16, 200),
                                                (4, 1, 32, 70), (8, 2, 128, None), (4, 2, 256, 300)])
def test_prefill_on_tcgen05(nh, nkv, page, window, hd):
    """The tcgen05 prefill kernel (head sizes 64 and 128) against the plain formula: portions that
    start in the middle of what the cache holds, lengths on both sides of the 128-row and the
    key tiles, a decode token and a two-token portion in the same launch, windows, and a far key
    that must dominate its row."""
    run(nh, nkv, hd, page, window, lens=[300, 517, 1, 130, 128, 700, 40], q_lens=[300, 260, 1, 2, 128, 129, 40],
        splits=1, far=(1, 11) if window is None else None, kernel="tc")


@pytest.mark.parametrize("seed", range(8))
def test_prefill_on_tcgen05_random_shapes(seed):
    """Random batches for the tcgen05 prefill kernel against the plain formula: group sizes 1 to 8,
    pages of 4 to 64 keys (tensor copies from 8 up, cp.async below and for sizes that are no power
    of two), portions that end a row tile, a pair of row tiles or a key tile exactly or one short
    or one over, contexts before the portion of 0 to 300 keys, and windows on some."""
    import random
    r = random.Random(100 + seed)
    nkv = r.choice([1, 2, 3])
    G = r.choice([1, 2, 4, 8])
    page = r.choice([4, 8, 16, 64, 12, 32])
    window = r.choice([None, None, 40, 200])
    edges = [128 // G, 256 // G, 128, 256, 384]
    q_lens, lens = [], []
    for _ in range(r.randint(2, 5)):
        q = max(1, r.choice(edges) * r.randint(1, 2) + r.choice([-1, 0, 1]) if r.random() < 0.7 else r.randint(1, 300))
        q = min(q, 520)
        q_lens.append(q)
        lens.append(q + r.choice([0, 0, 1, 127, 128, r.randint(0, 300)]))
    run(nkv * G, nkv, r.choice([64, 128]), page, window, lens=lens, q_lens=q_lens, splits=1, kernel="tc")


def test_long_prompt_whole_and_chosen_splits():
    from rllm_b200.kernels import sm100
    run(8, 2, 64, 16, None, lens=[1500], q_lens=[1500], splits=1, far=(0, 3))
    assert sm100.attention_splits(8, 8, 4, 4096, 148) >= 8       # decode: cut until the GPU is full
    assert sm100.attention_splits(8, 8, 2048 * 4, 4096, 148) == 1  # prefill: tiles fill it already
    assert sm100.attention_splits(1, 8, 4, 100, 148) == 1          # too short to cut


@pytest.mark.parametrize("kernel", ["fa", "decode", "tc"])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("edge", ["in", "out"])
@pytest.mark.parametrize("gave_back", [False, True])
def test_window_edge_with_a_key_that_would_dominate(kernel, hd, edge, gave_back):
    """The window's edge, made visible: the key at j = pos - window + 1 (the oldest the query may see)
    is given a score that dominates, so the output must be its value; the key one further back gets
    the same treatment and must leave no trace. Random scores would hide one key too many or too few
    (it moves the output by about 1 / window). Single tokens for the decode kernels, and a portion
    whose rows straddle the edge inside one key tile for the two prefill kernels; with `gave_back` the
    pages that lie wholly before the window are gone from the block table (-1), as after the cache
    manager has taken them back."""
    from rllm_b200.kernels import sm100
    nh, nkv, page, W = 8, 2, 8, 100
    decode = kernel == "decode"
    # (keys, rows of this step, row from the end whose query dominates)
    seqs = [(300, 1, 0), (257, 1, 0)] if decode else [(400, 200, 89), (300, 1, 0), (700, 130, 5)]
    lens, q_lens = [s[0] for s in seqs], [s[1] for s in seqs]
    S = len(seqs)
    kc, vc, bt, ks, vs = scattered_cache(S, lens, nkv, hd, page, torch.bfloat16, seed=hd + W)
    g = torch.Generator().manual_seed(8)
    T = sum(q_lens)
    q = torch.randn(T, nh, hd, generator=g).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    marks = []
    for s, (L, n, back) in enumerate(seqs):
        pos = L - 1 - back
        j = pos - W + 1 if edge == "in" else pos - W
        ks[s][j] = 0
        ks[s][j, :, 0] = 30.0
        q[cu[s + 1] - 1 - back, :, 0] = 30.0
        kc[int(bt[s, j // page]), :, j % page] = ks[s][j]
        marks.append((cu[s + 1] - 1 - back, j))
        if gave_back:
            first_needed = max(0, (L - n) - W + 1)       # the oldest key the step's first row sees
            bt[s, : first_needed // page] = -1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    qd = q.reshape(T, nh * hd).to(DEV)
    if kernel == "decode":
        out = sm100.attention_decode(qd, kc.to(DEV), vc.to(DEV), i32(lens), bt.to(DEV), nh, hd ** -0.5, W, max(lens),
                                     splits=2)
    elif kernel == "tc":
        out = sm100.attention_prefill_tc(qd, kc.to(DEV), vc.to(DEV), i32(cu), i32(lens), bt.to(DEV), max(q_lens), nh,
                                         hd ** -0.5, W)
    else:
        out = sm100.attention_fa(qd, kc.to(DEV), vc.to(DEV), i32(cu), i32(lens), bt.to(DEV), T, max(q_lens), max(lens),
                                 nh, hd ** -0.5, W, splits=1)
    sm100.check_error(DEV)
    for s, (L, n, back) in enumerate(seqs):
        qf = torch.zeros(L, nh, hd); qf[L - n:] = q[cu[s]: cu[s + 1]].float()
        ref = P.attention(qf, ks[s].float(), vs[s].float(), hd ** -0.5, W)[L - n:]
        got = out[cu[s]: cu[s + 1]].float().cpu().view(n, nh, hd)
        assert torch.isfinite(got).all()
        assert rel(got, ref) <= TOL, f"sequence {s} (len {L}, q {n})"
        row, j = marks[s]
        mine = out[row].float().cpu().view(nh, hd)
        vj = vs[s][j].float().repeat_interleave(nh // nkv, 0)
        if edge == "in":
            assert rel(mine, vj) <= TOL, f"sequence {s}: the oldest visible key was not seen"
        else:
            assert rel(mine, vj) > 0.1, f"sequence {s}: a key beyond the window was seen"
