"""Random-weights mode: from a configuration and a seed, either write a model folder
(config.json + model.safetensors) that the ordinary loader reads, or fill a model's
tensors on the device directly (for sizes where a file round trip is a waste).
The reference has no such mode; it exists for tests and measurement without checkpoints."""
from __future__ import annotations

import json
import os

import torch

from ..config.base import config_from_dict
from .loader import expected_tensors, storage_dtype
from .safetensors_io import write_safetensors


def _fill(source, gen, std, norm_std, device):
    if source.init == "zeros":
        return torch.zeros(source.shape, dtype=torch.float32, device=device)
    if source.init == "norm":
        t = torch.ones(source.shape, dtype=torch.float32, device=device)
        if norm_std > 0:
            t += torch.randn(source.shape, generator=gen, dtype=torch.float32, device=device) * norm_std
        return t
    return torch.randn(source.shape, generator=gen, dtype=torch.float32, device=device) * std


def random_tensors(model, seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """Checkpoint-named tensors, drawn in the order the model lists them (CPU generator)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, source, param, _ in expected_tensors(model):
        t = _fill(source, gen, std, norm_std, "cpu")
        out[name] = t.to(torch.int32) if param.role == "table" else t.to(dtype)
    return out


def write_random_model(config: dict, seed: int, out_dir: str, std: float = 0.02,
                       norm_std: float = 0.0, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors` for the raw config dict."""
    arch, cfg = config_from_dict(config)
    model = arch.build(cfg)
    os.makedirs(out_dir, exist_ok=True)
    raw = dict(config)
    raw.setdefault("architectures", [arch.name])
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      random_tensors(model, seed, std, norm_std, dtype))
    return out_dir


def init_random_weights(model, seed: int, dtype: torch.dtype, device, std: float = 0.02,
                        norm_std: float = 0.0) -> None:
    """Fill the model's tensors on `device` without touching the disk."""
    device = torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    for part in model.parts():
        for p in part.params():
            pieces = []
            for s in p.sources:
                t = _fill(s, gen, std, norm_std, device)
                pieces.append(t.to(storage_dtype(p.role, torch.bfloat16, dtype)))
            setattr(part, p.attr, (pieces[0] if len(pieces) == 1 else torch.cat(pieces, 0)).contiguous())
    model.finalize(device, dtype)
