"""Reading and writing safetensors files without any model library: an 8-byte
little-endian header length, a JSON header (name -> dtype, shape, data_offsets), then
the raw little-endian tensor bytes. Single file `model.safetensors`, or
`model.safetensors.index.json` naming shards (all of which must exist), as the
reference's loader accepts (src/model/loader/store.rs:141-217)."""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
           "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "I8": torch.int8,
           "F64": torch.float64, "BOOL": torch.bool, "I16": torch.int16}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightFileError(RuntimeError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    file: str
    dtype: str
    shape: tuple[int, ...]
    begin: int      # absolute byte offsets in the file
    end: int


class TensorStore:
    """All tensors of a model folder, by name, read lazily through mmap."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.entries: dict[str, TensorEntry] = {}
        self._maps: dict[str, mmap.mmap] = {}
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(single):
            files = [single]
        elif os.path.isfile(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map", {})
            shards = sorted(set(wm.values()))
            missing = [s for s in shards if not os.path.isfile(os.path.join(model_dir, s))]
            if missing:
                raise WeightFileError(f"{index} names shards that are absent: {missing}")
            files = [os.path.join(model_dir, s) for s in shards]
        else:
            raise WeightFileError(f"{model_dir!r} has neither model.safetensors nor "
                                  f"model.safetensors.index.json")
        for path in files:
            self._read_header(path)

    def _read_header(self, path: str) -> None:
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise WeightFileError(f"{path}: too short for a safetensors header")
            (hlen,) = struct.unpack("<Q", head)
            if hlen > size - 8:
                raise WeightFileError(f"{path}: header length {hlen} exceeds the file")
            try:
                header = json.loads(f.read(hlen))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise WeightFileError(f"{path}: header is not valid JSON ({e})") from e
        base = 8 + hlen
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            b, e = meta["data_offsets"]
            if meta["dtype"] not in _DTYPES:
                raise WeightFileError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
            if base + e > size or b > e:
                raise WeightFileError(f"{path}: tensor {name!r} lies outside the file")
            self.entries[name] = TensorEntry(path, meta["dtype"], tuple(meta["shape"]), base + b, base + e)

    def names(self):
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        """The tensor as stored (a copy on the host)."""
        ent = self.entries[name]
        mm = self._maps.get(ent.file)
        if mm is None:
            with open(ent.file, "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[ent.file] = mm
        dtype = _DTYPES[ent.dtype]
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=dtype)
        buf = bytearray(mm[ent.begin:ent.end])
        return torch.frombuffer(buf, dtype=dtype, count=n).reshape(ent.shape)

    def close(self):
        for mm in self._maps.values():
            mm.close()
        self._maps.clear()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor]) -> None:
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store dtype {t.dtype}")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
