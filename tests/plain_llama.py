"""Plain, slow, whole-sequence Llama in float32 on the CPU: the tests' yardstick.

It restates the reference's formulas, each function citing the file and lines it restates (paths
relative to the reference project root), and it is anchored on the reference's own code: the
reference's host code is Rust (no `cargo`/`rustc` on the build machine) and cannot be imported or
compiled on the CPU here, but its CUDA kernels compile as they are, and `tests/golden/` holds the
logits of two tiny random models computed by those kernels (`tests/golden/make_golden.py`, run
once on a GPU). `tests/test_plain.py::test_plain_against_the_reference_projects_own_kernels`
compares this file with them (agreement to the reference's bfloat16 rounding, 5e-3 and 1e-2 of
the largest logit; equal greedy tokens); the llama3 rule and attention across prompt portions,
which the reference does not run, rest on the formulas alone.

Deliberate differences from what the reference *does*, all argued from what
it *states*:
  * the llama3 frequency rule is applied (the reference parses
    `rope_scaling` but passes only theta for Llama; the three-band rule is
    the one its "yarn" kernel computes, src/gpu/cuda/shaders/rope.cu:233-251);
  * every query attends all earlier keys of its sequence, not just the keys
    of its own prefill chunk (src/gpu/cuda/shaders/attention.cu:573-618 is
    chunk-local);
  * nothing is rounded to bfloat16 between operations.

No cache, no batching, no paging: one token list in, logits for every
position out. Shares no code with the `rllm_b200` package.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch


# ----------------------------------------------------------------------------
# reading a model folder (own tiny safetensors reader: nothing shared with the
# package's loader)
# ----------------------------------------------------------------------------

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        raw = bytearray(blob[8 + hlen + b: 8 + hlen + e])
        t = torch.frombuffer(raw, dtype=_ST_DTYPES[meta["dtype"]]).reshape(meta["shape"])
        out[name] = t.clone()
    return out


def read_model_dir(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    w = {k: (v.to(torch.float32) if v.is_floating_point() else v) for k, v in w.items()}
    return cfg, w


# ----------------------------------------------------------------------------
# one function per part
# ----------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x0[t] = E[id_t], a row copy with no scaling.
    src/gpu/cuda/shaders/embed.cu:24-59; src/model/primitives.rs:113-121."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, the weight used as stored (no 1+w).
    src/gpu/cuda/shaders/rms_norm.cu:78-115; src/gpu/cpu/mod.rs:188-202."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """y[o] = sum_i W[o,i] x[i], W row-major [out, in]; bias (Qwen-style only)
    added after the product. src/gpu/cuda/shaders/matmul.cu:63-76;
    src/model/registry/llama.rs:183-187."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    return y


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """f_i = theta^(-2i/hd) for i in [0, hd/2)  (src/gpu/cuda/shaders/rope.cu:62-66).
    llama3 rule in the shape of the reference's three-band kernel
    (src/gpu/cuda/shaders/rope.cu:233-251, src/gpu/cpu/mod.rs:1069-1084) with
    beta_fast -> high_freq_factor and beta_slow -> low_freq_factor:
      wavelength < orig/high -> f;  wavelength > orig/low -> f/factor;
      else s = (orig/wavelength - low)/(high - low), f' = (1-s) f/factor + s f.
    Computed in float64, returned as float32 (one table of hd/2 numbers)."""
    half = head_dim // 2
    out = []
    rtype = None
    if scaling:
        rtype = scaling.get("rope_type", scaling.get("type"))
    for i in range(half):
        f = float(theta) ** (-2.0 * i / head_dim)
        if rtype == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                pass
            elif wavelen > orig / low:
                f = f / factor
            else:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        elif rtype == "linear":
            f = f / float(scaling["factor"])
        elif rtype in (None, "default"):
            pass
        else:
            raise ValueError(f"plain implementation: rope_type {rtype!r} not covered")
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, hd]. Pair (i, i+hd/2): a' = a cos - b sin, b' = a sin + b cos,
    angle = p * f_i with p the token's absolute position.
    src/gpu/cuda/shaders/rope.cu:62-77, 126-146; src/gpu/cpu/mod.rs:958-989."""
    half = x.shape[-1] // 2
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]       # [T, half]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: int | None = None) -> torch.Tensor:
    """q: [T, nh, hd]; k, v: [T, nkv, hd]. Query head h uses KV head h // (nh/nkv);
    s_j = (q . k_j) * scale for j <= p (causal), and j > p - window when a
    window is set (the last `window` keys, the query's own included:
    src/gpu/cuda/shaders/attention.cu:337-338); softmax with the maximum
    subtracted; o = sum_j a_j v_j.
    src/gpu/cuda/shaders/attention.cu:328-388; src/gpu/cpu/mod.rs:1283-1347."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(T)
    mask = pos[None, :] <= pos[:, None]
    if window:
        mask &= pos[None, :] > (pos[:, None] - window)
    for h in range(nh):
        kh, vh = k[:, h // g], v[:, h // g]
        s = (q[:, h] @ kh.t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        a = e / e.sum(dim=-1, keepdim=True)
        out[:, h] = a @ vh
    return out


def attention_tail(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   window: int | None = None) -> torch.Tensor:
    """The same formula for the last n positions only: q [n, nh, hd] are the queries at positions
    L-n .. L-1 of a sequence whose keys and values k, v [L, nkv, hd] are all given. Equal to
    `attention` over the whole sequence, cut to its last n rows, without the L x L scores (for
    sequences of many thousand keys). src/gpu/cuda/shaders/attention.cu:328-388."""
    n, nh, hd = q.shape
    L, nkv = k.shape[0], k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    qpos = torch.arange(L - n, L)
    kpos = torch.arange(L)
    mask = kpos[None, :] <= qpos[:, None]
    if window:
        mask &= kpos[None, :] > (qpos[:, None] - window)
    for h in range(nh):
        kh, vh = k[:, h // g], v[:, h // g]
        s = (q[:, h] @ kh.t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        e = torch.exp(s)
        out[:, h] = (e / e.sum(dim=-1, keepdim=True)) @ vh
    return out


def swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """g = Wg x, u = Wu x, a = g/(1+exp(-g)) * u, y = Wd a.
    src/gpu/cuda/shaders/moe.cu:141-146; src/gpu/cuda/shaders/elementwise.cu:36-49;
    src/model/primitives.rs:557-585."""
    g = linear(x, wg)
    u = linear(x, wu)
    a = g / (1.0 + torch.exp(-g)) * u
    return linear(a, wd)


# ----------------------------------------------------------------------------
# the model: layer order of src/model/registry/llama.rs:163-245
# ----------------------------------------------------------------------------

def layer_windows(cfg: dict) -> list[int | None]:
    """Which layers look at a window of keys: `sliding_window` with optional
    `layer_types` (src/model/config.rs:553-558, 970-985: "sliding_attention" /
    "full_attention"); none for stock Llama."""
    L = cfg["num_hidden_layers"]
    win = cfg.get("sliding_window") or None
    types = cfg.get("layer_types")
    if not win:
        return [None] * L
    if not types:
        return [win] * L
    return [win if t == "sliding_attention" else None for t in types]


def forward(cfg: dict, w: dict[str, torch.Tensor], ids) -> torch.Tensor:
    """Logits [T, vocab] (float32) for the token list `ids`, whole sequence."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.numel()
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or H // nh          # src/model/config.rs:966-968
    eps = cfg.get("rms_norm_eps", cfg.get("norm_eps", 1e-5))
    theta = cfg.get("rope_theta", 10000.0)
    inv_freq = rope_inv_freq(hd, theta, cfg.get("rope_scaling"))
    scale = hd ** -0.5                             # src/gpu/cuda/shaders/attention.cu:336
    positions = torch.arange(T)
    windows = layer_windows(cfg)

    h = embedding(w["model.embed_tokens.weight"], ids)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        n = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        q = linear(n, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias"))
        k = linear(n, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias"))
        v = linear(n, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias"))
        q = rope(q.view(T, nh, hd), positions, inv_freq)
        k = rope(k.view(T, nkv, hd), positions, inv_freq)
        a = attention(q, k, v.view(T, nkv, hd), scale, windows[l])
        h = h + linear(a.reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        n = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    n = rms_norm(h, w["model.norm.weight"], eps)
    # tied output: src/model/primitives.rs:135, 1467; src/model/loader/mod.rs:693-702
    wout = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return linear(n, wout)


def greedy(cfg, w, prompt, n_new: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token;
    ties go to the lowest index."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, w, ids)[-1]
        ids.append(int(torch.argmax(logits)))   # torch.argmax returns the first maximal index
    return ids[len(prompt):]


# ----------------------------------------------------------------------------
# sampling, restated from src/model/sampler.rs:328-547
# ----------------------------------------------------------------------------

def sample_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                 min_p: float = 0.0) -> torch.Tensor:
    """The distribution the reference draws from: x/T -> top-k mask (ties at the
    threshold kept) -> softmax -> min-p (p < min_p * max p dropped, renormalised)
    -> top-p (sorted descending, kept until the cumulative mass reaches top_p,
    renormalised). src/model/sampler.rs:361-482."""
    x = logits.to(torch.float32) / temperature
    V = x.numel()
    if 0 < top_k < V:
        thr = torch.topk(x, top_k).values[-1]
        x = torch.where(x < thr, torch.full_like(x, float("-inf")), x)
    p = torch.softmax(x, dim=-1)
    if min_p > 0.0:
        p = torch.where(p < min_p * p.max(), torch.zeros_like(p), p)
        p = p / p.sum()
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True, stable=True)
        cum = torch.cumsum(sp, 0)
        cut = int((cum >= top_p).nonzero()[0]) + 1 if bool((cum >= top_p).any()) else V
        keep = torch.zeros(V, dtype=torch.bool)
        keep[si[:cut]] = True
        p = torch.where(keep, p, torch.zeros_like(p))
        p = p / p.sum()
    return p


def sample_from_probs(p: torch.Tensor, u: float) -> int:
    """First index whose cumulative probability exceeds u, in vocabulary order;
    the last index with mass if rounding leaves none. src/model/sampler.rs:489-499."""
    cum = torch.cumsum(p.to(torch.float64), 0)
    idx = (cum > u).nonzero()
    if idx.numel():
        return int(idx[0])
    return int((p > 0).nonzero()[-1])


def adjust_logits(logits: torch.Tensor, history: list[int], frequency_penalty: float = 0.0,
                  presence_penalty: float = 0.0, logit_bias: dict[int, float] | None = None) -> torch.Tensor:
    """Penalties for tokens already generated, then the per-token bias, on the raw logits
    (before the temperature). src/model/sampler.rs:341-358."""
    x = logits.to(torch.float32).clone()
    V = x.numel()
    if frequency_penalty != 0.0 or presence_penalty != 0.0:
        for t in set(history):
            if t < V:
                x[t] -= frequency_penalty * history.count(t) + presence_penalty
    for t, b in (logit_bias or {}).items():
        if t < V:
            x[t] += b
    return x


def logprobs(logits: torch.Tensor, temperature: float, top_k: int, chosen: int, n_top: int):
    """ln p of the chosen token and of the n_top most probable ones under the distribution
    before min-p and top-p: softmax of x/T (of x when T is 0) over what top-k keeps; tokens of
    probability 0 are not listed. src/model/sampler.rs:372-428, 501-541."""
    x = logits.to(torch.float64)
    if temperature != 0.0:
        x = x / temperature
    V = x.numel()
    if 0 < top_k < V:
        thr = torch.topk(x, top_k).values[-1]
        x = torch.where(x < thr, torch.full_like(x, float("-inf")), x)
    lp = torch.log_softmax(x, dim=-1)
    order = sorted(range(V), key=lambda i: (-float(lp[i]), i))[:n_top]
    return float(lp[chosen]), [(i, float(lp[i])) for i in order if lp[i] > float("-inf")]
