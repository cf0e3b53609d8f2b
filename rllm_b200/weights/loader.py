"""Binds checkpoint tensors to a model's parts, by name.

Every `Param` of every part names the checkpoint tensors it is assembled from
(prefix + source name). All problems are collected and raised once: tensors the
model needs but the folder lacks, tensors the folder holds but the model does not
know, and tensors of the wrong shape. Storage rule: matrices take the run dtype
(bfloat16, or float32 in the 32-bit run); vectors stay as stored when stored in
32-bit, otherwise bfloat16 (everything floating becomes float32 in the 32-bit
run); integer tables become int32.
Parity: src/model/loader/store.rs:48-59, upload.rs:85-95 (by-name lookup, shape check).
"""
from __future__ import annotations

import fnmatch

import torch

from .safetensors_io import TensorStore

# Names that may sit in a checkpoint without belonging to any part: the rotary tables some exporters
# store, and the output matrix of a model that ties it to the embedding (a redundant copy; the
# reference never looks for it then, src/model/loader/mod.rs:693-702). Where a model does own
# `lm_head.weight` the name is expected and this list is not asked.
IGNORABLE = ("*.rotary_emb.inv_freq", "lm_head.weight")


class WeightError(RuntimeError):
    """One error for the whole folder: `.missing`, `.unexpected`, `.wrong_shape`, `.wrong_dtype`."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = [f"weights in {model_dir!r} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(g)}" for n, e, g in wrong_shape))
        if wrong_dtype:
            lines.append(f"  unsupported dtype ({len(wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in wrong_dtype))
        super().__init__("\n".join(lines))


def expected_tensors(model):
    """[(full checkpoint name, Source, Param, part)] for the whole model."""
    out = []
    for part in model.parts():
        for p in part.params():
            for s in p.sources:
                out.append((part.prefix + s.name, s, p, part))
    return out


def storage_dtype(role: str, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if role == "table":
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if role == "matrix":
        return run_dtype
    return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16


def load_weights(model, model_dir: str, dtype: torch.dtype, device) -> None:
    store = TensorStore(model_dir)
    try:
        exp = expected_tensors(model)
        names = {n for n, *_ in exp}
        missing = sorted(n for n in names if n not in store.entries)
        unexpected = sorted(n for n in store.names() if n not in names
                            and not any(fnmatch.fnmatch(n, pat) for pat in IGNORABLE))
        wrong_shape, wrong_dtype = [], []
        for n, s, p, _ in exp:
            ent = store.entries.get(n)
            if ent is None:
                continue
            if tuple(ent.shape) != tuple(s.shape):
                wrong_shape.append((n, s.shape, ent.shape))
            floating = ent.dtype in ("F32", "BF16", "F16", "F64")
            if (p.role == "table") == floating:
                wrong_dtype.append((n, ent.dtype))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
        for part in model.parts():
            for p in part.params():
                pieces = [store.read(part.prefix + s.name) for s in p.sources]
                target = storage_dtype(p.role, pieces[0].dtype, dtype)
                pieces = [t.to(target) for t in pieces]
                t = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=0)
                setattr(part, p.attr, t.to(device).contiguous())
    finally:
        store.close()
    model.finalize(torch.device(device), dtype)
