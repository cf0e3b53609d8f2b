"""The plain implementation itself: closed-form cases in the manner of the reference's CPU
kernel tests (src/gpu/cpu/mod.rs:2344-2631), and that no cache or batching hides in it."""
import math
import os

import pytest

import torch

import plain_llama as P
import tiny


def test_rms_norm_of_a_uniform_vector_is_the_weight():
    x = torch.full((2, 8), 3.0)
    w = torch.arange(8, dtype=torch.float32)
    assert torch.allclose(P.rms_norm(x, w, 0.0), w.expand(2, 8), atol=1e-6)
    y = P.rms_norm(torch.tensor([[3.0, 4.0]]), torch.ones(2), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 4.0]]) / math.sqrt(12.5))


def test_linear_is_row_times_column():
    w = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert torch.equal(P.linear(torch.tensor([[1.0, 1.0]]), w), torch.tensor([[3.0, 7.0, 11.0]]))
    assert torch.equal(P.linear(torch.eye(2), w), w.t())


def test_rope_at_position_zero_is_identity_and_keeps_length():
    f = P.rope_inv_freq(8, 10000.0, None)
    x = torch.randn(3, 2, 8)
    y = P.rope(x, torch.tensor([0, 5, 9]), f)
    assert torch.equal(y[0], x[0]) and not torch.allclose(y[1], x[1])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # pair (0, 4) turns by the position itself (f_0 = 1)
    e = torch.zeros(1, 1, 8); e[0, 0, 0] = 1.0
    r = P.rope(e, torch.tensor([2]), f)[0, 0]
    assert abs(float(r[0]) - math.cos(2.0)) < 1e-6 and abs(float(r[4]) - math.sin(2.0)) < 1e-6


def test_llama3_bands():
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 32}
    base, f = P.rope_inv_freq(32, 500000.0, None), P.rope_inv_freq(32, 500000.0, sc)
    wl = 2 * math.pi / base
    hi, lo = wl < 32 / 4.0, wl > 32 / 1.0
    assert hi.any() and lo.any() and (~hi & ~lo).any()         # all three bands occur
    assert torch.equal(f[hi], base[hi]) and torch.allclose(f[lo], base[lo] / 8.0)
    mid = ~hi & ~lo
    assert ((f[mid] < base[mid]) & (f[mid] > base[mid] / 8.0)).all()


def test_attention_single_key_returns_v_and_is_causal_and_windowed():
    q, k, v = torch.randn(1, 4, 8), torch.randn(1, 2, 8), torch.randn(1, 2, 8)
    o = P.attention(q, k, v, 8 ** -0.5)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 3], v[0, 1])   # heads 0,1 -> kv 0
    q, k, v = torch.randn(6, 2, 8), torch.randn(6, 1, 8), torch.randn(6, 1, 8)
    o = P.attention(q, k, v, 1.0)
    k2, v2 = k.clone(), v.clone(); k2[4:] += 1.0; v2[4:] -= 2.0                    # later keys changed
    assert torch.allclose(P.attention(q, k2, v2, 1.0)[:4], o[:4])
    ow = P.attention(q, k, v, 1.0, window=2)
    assert torch.allclose(ow[:2], o[:2]) and not torch.allclose(ow[5], o[5])
    assert torch.allclose(ow[5], P.attention(q[4:], k[4:], v[4:], 1.0)[1], atol=1e-6)


def test_swiglu_formula():
    x = torch.tensor([[1.0, -2.0]])
    wg, wu, wd = torch.tensor([[1.0, 0.0]]), torch.tensor([[0.0, 1.0]]), torch.tensor([[2.0]])
    g, u = 1.0, -2.0
    assert torch.allclose(P.swiglu(x, wg, wu, wd), torch.tensor([[2.0 * (g / (1 + math.exp(-g))) * u]]))


def test_forward_is_causal_and_greedy_takes_the_lowest_index(tmp_path):
    d = tiny.make_model_dir(tmp_path, "B")
    cfg, w = P.read_model_dir(d)
    ids = tiny.random_prompt(20, cfg["vocab_size"], 3)
    full = P.forward(cfg, w, ids)
    assert torch.allclose(P.forward(cfg, w, ids[:11]), full[:11], atol=1e-5)
    out = P.greedy(cfg, w, ids[:5], 3)
    assert out[0] == int(torch.argmax(P.forward(cfg, w, ids[:5])[-1]))
    assert int(torch.argmax(torch.tensor([1.0, 3.0, 3.0]))) == 1


def test_sampling_distribution_rules():
    lg = torch.log(torch.tensor([0.5, 0.25, 0.125, 0.125]))
    assert torch.allclose(P.sample_probs(lg, 1.0), torch.tensor([0.5, 0.25, 0.125, 0.125]))
    assert torch.allclose(P.sample_probs(lg, 1.0, top_k=2), torch.tensor([2 / 3, 1 / 3, 0, 0]))
    assert torch.allclose(P.sample_probs(lg, 1.0, top_p=0.7), torch.tensor([2 / 3, 1 / 3, 0, 0]))
    assert torch.allclose(P.sample_probs(lg, 1.0, min_p=0.3), torch.tensor([2 / 3, 1 / 3, 0, 0]))
    assert torch.allclose(P.sample_probs(lg, 0.5), torch.tensor([16 / 22, 4 / 22, 1 / 22, 1 / 22]))
    p = torch.tensor([0.5, 0.25, 0.25])
    assert [P.sample_from_probs(p, u) for u in (0.0, 0.49, 0.5, 0.76, 0.9999999)] == [0, 0, 1, 2, 2]


def test_plain_bias_and_logprobs():
    import math
    g = torch.Generator().manual_seed(4)
    x = torch.randn(30, generator=g) * 2
    lp, top = P.logprobs(x, 0.5, 0, 3, 30)
    assert abs(sum(math.exp(v) for _, v in top) - 1.0) < 1e-9 and dict(top)[3] == lp
    assert [t for t, _ in top] == sorted(range(30), key=lambda i: (-float(x[i]), i))
    lp0, top0 = P.logprobs(x, 0.0, 0, 3, 2)                   # a greedy row: the raw logits' softmax
    assert abs(lp0 - float(torch.log_softmax(x.double(), -1)[3])) < 1e-12 and len(top0) == 2
    _, top_k = P.logprobs(x, 1.0, 4, int(torch.argmax(x)), 10)
    assert len(top_k) == 4 and abs(sum(math.exp(v) for _, v in top_k) - 1.0) < 1e-9
    assert P.logprobs(x, 1.0, 4, int(torch.argmin(x)), 0)[0] == float("-inf")
    y = P.adjust_logits(x, [2, 2, 5], frequency_penalty=0.5, presence_penalty=1.0, logit_bias={5: 3.0, 99: 1.0})
    want = x.clone(); want[2] -= 2.0; want[5] += 3.0 - 1.5
    assert torch.allclose(y, want)


def test_attention_tail_is_the_whole_formula_cut_to_its_last_rows():
    g = torch.Generator().manual_seed(3)
    L, nh, nkv, hd = 45, 6, 2, 16
    q, k, v = (torch.randn(L, h, hd, generator=g) for h in (nh, nkv, nkv))
    for window in (None, 7, 100):
        full = P.attention(q, k, v, 0.3, window)
        for n in (1, 5, L):
            assert torch.allclose(P.attention_tail(q[L - n:], k, v, 0.3, window), full[L - n:], atol=1e-6)


@pytest.mark.parametrize("name", ["a", "g"])
def test_plain_against_the_reference_projects_own_kernels(name, tmp_path):
    """The outside anchor: tests/golden/golden_<name>.npz holds logits of a tiny random Llama computed
    token by token by the reference project's own CUDA kernels (tests/golden/make_golden.py built and
    ran them, unmodified). The plain implementation, whole sequence, must agree to the rounding the
    reference's bfloat16 activations cost, and pick the same greedy token wherever the golden's best
    two logits are clearly apart. A wrong rotary pairing, scale, mask or norm is off by far more."""
    import hashlib
    import json
    import numpy as np
    from rllm_b200.weights import write_random_model
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"golden_{name}.npz")
    z = np.load(path)
    cfg = json.loads(str(z["config"]))
    d = write_random_model(cfg, int(z["seed"]), str(tmp_path / name), std=float(z["std"]), norm_std=float(z["norm_std"]))
    with open(os.path.join(d, "model.safetensors"), "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    assert digest == str(z["weights_sha256"]), "the random weights are no longer those the golden was made from: " \
        "run tests/golden/make_golden.py again"
    pcfg, w = P.read_model_dir(d)
    ids = z["ids"].tolist()
    got = P.forward(pcfg, w, ids).numpy()
    want = z["logits"]
    assert got.shape == want.shape
    scale = float(np.abs(want).max())
    err = float(np.abs(got - want).max()) / scale
    assert err <= 3e-2, f"golden {name}: plain differs from the reference's kernels by {err:.3e} of the largest logit"
    decided = agree = 0
    for t in range(len(ids)):
        top2 = np.partition(want[t], -2)[-2:]
        if top2[1] - top2[0] > 6e-2 * scale:
            decided += 1
            agree += int(np.argmax(got[t]) == np.argmax(want[t]))
    assert decided > 0 and agree == decided
    # and the anchor bites: the other rotary pairing (neighbours instead of halves) is far outside
    real = P.rope

    def interleaved(x, positions, inv_freq):
        T, nh, hd = x.shape
        ang = positions[:, None].float() * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
        return out
    P.rope = interleaved
    try:
        wrong = P.forward(pcfg, w, ids).numpy()
    finally:
        P.rope = real
    assert float(np.abs(wrong - want).max()) / scale > 2 * err + 3e-2
