#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/: tiny random Llama models run token by token through
the reference project's OWN CUDA kernels (JonCooperWorks/rLLM, src/gpu/cuda/shaders/: embed_lookup,
rms_norm, matvec_bf16, rotary_embedding, copy_to_kv_cache, attention, silu_mul, add_tensors),
compiled unmodified and launched by `ref_kernels.cu`, in the layer order of
src/model/registry/llama.rs:163-245. `tests/test_plain.py` compares the plain implementation with
these files, which anchors its formulas (the rotary pairing, the attention scale and mask, the
norm's rounding, SiLU) on code that is not this repository's.

    python tests/golden/make_golden.py --shaders <reference>/src/gpu/cuda/shaders [--out tests/golden]

Needs nvcc and a GPU (the kernels are device code; the reference's host code is Rust and does not
build here). The reference keeps every activation in bfloat16, so the goldens agree with a float32
computation to bfloat16 rounding only (about 1e-2 of the largest logit). The models have no
`rope_scaling` (the reference applies none for Llama) and decode one token a step (its prefill
kernel sees its own chunk only). Weights come from `rllm_b200.weights.write_random_model` with the
seeds below; the .npz records the SHA-256 of the weight file it was made from.
"""
import argparse
import ctypes
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))            # tests/ (plain_llama's reader)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

# name -> (config, seed, weight std, norm std, tokens)
GOLDEN = {
    "a": ({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 64, "num_hidden_layers": 2,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
           "vocab_size": 256, "max_position_embeddings": 128, "rope_theta": 10000.0, "rope_scaling": None,
           "rms_norm_eps": 1e-5, "tie_word_embeddings": True}, 0, 0.05, 0.1, 24),
    "g": ({"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 96, "num_hidden_layers": 3,
           "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 160,
           "vocab_size": 200, "max_position_embeddings": 256, "rope_theta": 500000.0, "rope_scaling": None,
           "rms_norm_eps": 1e-6, "tie_word_embeddings": False}, 7, 0.08, 0.2, 40),
}
SHADERS = {"EMBED": "embed.cu", "RMS_NORM": "rms_norm.cu", "MATMUL": "matmul.cu", "ROPE": "rope.cu",
           "ATTENTION": "attention.cu", "ELEMENTWISE": "elementwise.cu"}


def build(shaders: str, tmp: str) -> ctypes.CDLL:
    objs = []
    for name in SHADERS:
        obj = os.path.join(tmp, f"{name.lower()}.o")
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-Xcompiler", "-fPIC",
                        f"-DWRAP_{name}", "-I", shaders, "-c", os.path.join(HERE, "ref_kernels.cu"), "-o", obj], check=True)
        objs.append(obj)
    so = os.path.join(tmp, "libref_kernels.so")
    subprocess.run(["nvcc", "-shared", "-o", so, *objs], check=True)
    lib = ctypes.CDLL(so)
    u, f, p = ctypes.c_uint, ctypes.c_float, ctypes.c_void_p
    lib.ref_embed.argtypes = [u, u, p, p]
    lib.ref_rms_norm.argtypes = [u, f, p, p, p]
    lib.ref_matvec.argtypes = [u, u, p, p, p]
    lib.ref_rope.argtypes = [u, f, u, u, u, p, p]
    lib.ref_copy_kv.argtypes = [u, u, u, p, p]
    lib.ref_attention.argtypes = [u, u, u, u, u, p, p, p, p]
    lib.ref_silu_mul.argtypes = [u, p, p, p]
    lib.ref_add.argtypes = [u, p, p, p]
    return lib


def run_reference(lib, cfg, w, ids):
    """Logits [T, vocab] from the reference's kernels, one token a step, flat caches."""
    dev = "cuda:0"
    W = {k: v.to(torch.bfloat16).to(dev).contiguous() for k, v in w.items()}
    H, L, nh = cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"]
    nkv, hd, I, V = cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    buf = lambda n: torch.zeros(n, dtype=torch.bfloat16, device=dev)
    h, n, q, k, v, a, o = buf(H), buf(H), buf(nh * hd), buf(nkv * hd), buf(nkv * hd), buf(nh * hd), buf(H)
    g, u, act, d, lg = buf(I), buf(I), buf(I), buf(H), buf(V)
    kc = [buf(len(ids) * nkv * hd) for _ in range(L)]
    vc = [buf(len(ids) * nkv * hd) for _ in range(L)]
    P = lambda t: t.data_ptr()
    head = W["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else W["lm_head.weight"]
    out = []
    for pos, tok in enumerate(ids):
        lib.ref_embed(tok, H, P(W["model.embed_tokens.weight"]), P(h))
        for l in range(L):
            pre = f"model.layers.{l}."
            lib.ref_rms_norm(H, eps, P(h), P(W[pre + "input_layernorm.weight"]), P(n))
            lib.ref_matvec(nh * hd, H, P(W[pre + "self_attn.q_proj.weight"]), P(n), P(q))
            lib.ref_matvec(nkv * hd, H, P(W[pre + "self_attn.k_proj.weight"]), P(n), P(k))
            lib.ref_matvec(nkv * hd, H, P(W[pre + "self_attn.v_proj.weight"]), P(n), P(v))
            lib.ref_rope(pos, theta, nh, nkv, hd, P(q), P(k))
            lib.ref_copy_kv(pos, nkv, hd, P(k), P(kc[l]))
            lib.ref_copy_kv(pos, nkv, hd, P(v), P(vc[l]))
            lib.ref_attention(pos + 1, nh, nkv, hd, 0, P(q), P(kc[l]), P(vc[l]), P(a))
            lib.ref_matvec(H, nh * hd, P(W[pre + "self_attn.o_proj.weight"]), P(a), P(o))
            lib.ref_add(H, P(h), P(o), P(h))
            lib.ref_rms_norm(H, eps, P(h), P(W[pre + "post_attention_layernorm.weight"]), P(n))
            lib.ref_matvec(I, H, P(W[pre + "mlp.gate_proj.weight"]), P(n), P(g))
            lib.ref_matvec(I, H, P(W[pre + "mlp.up_proj.weight"]), P(n), P(u))
            lib.ref_silu_mul(I, P(g), P(u), P(act))
            lib.ref_matvec(H, I, P(W[pre + "mlp.down_proj.weight"]), P(act), P(d))
            lib.ref_add(H, P(h), P(d), P(h))
        lib.ref_rms_norm(H, eps, P(h), P(W["model.norm.weight"]), P(n))
        lib.ref_matvec(V, H, P(head), P(n), P(lg))
        rc = lib.ref_sync()
        if rc:
            raise RuntimeError(f"a reference kernel failed (cudaError {rc}) at position {pos}")
        out.append(lg.float().cpu().numpy().copy())
    return np.stack(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shaders", required=True, help="the reference's src/gpu/cuda/shaders folder")
    ap.add_argument("--out", default=HERE)
    a = ap.parse_args()
    import plain_llama
    from rllm_b200.weights import write_random_model
    with tempfile.TemporaryDirectory() as tmp:
        lib = build(a.shaders, tmp)
        for name, (cfg, seed, std, norm_std, T) in GOLDEN.items():
            d = write_random_model(cfg, seed, os.path.join(tmp, name), std=std, norm_std=norm_std, dtype=torch.bfloat16)
            with open(os.path.join(d, "model.safetensors"), "rb") as f:
                digest = hashlib.sha256(f.read()).hexdigest()
            pcfg, w = plain_llama.read_model_dir(d)
            ids = torch.randint(0, cfg["vocab_size"], (T,), generator=torch.Generator().manual_seed(1000 + seed)).tolist()
            logits = run_reference(lib, pcfg, w, ids)
            np.savez_compressed(os.path.join(a.out, f"golden_{name}.npz"), logits=logits.astype(np.float32),
                                ids=np.array(ids, dtype=np.int32), weights_sha256=digest,
                                config=json.dumps(cfg), seed=seed, std=std, norm_std=norm_std)
            print(f"golden_{name}.npz: {logits.shape}, largest |logit| {np.abs(logits).max():.3f}, weights {digest[:12]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
