"""Model folders: `config.json` + `model.safetensors`, read without any third-party reader.

A safetensors file is an 8-byte little-endian header length, that many bytes of JSON (tensor name -> dtype, shape,
data_offsets relative to the end of the header), then the raw little-endian tensor data."""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Mapping

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, np.uint16), "F16": (torch.float16, np.float16), "F32": (torch.float32, np.float32),
           "I32": (torch.int32, np.int32), "I64": (torch.int64, np.int64), "U8": (torch.uint8, np.uint8)}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file as CPU tensors (copied out of the mapping, so the file can go away)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
    raw = np.memmap(path, dtype=np.uint8, mode="r", offset=base) if os.path.getsize(path) > base else np.zeros(0, np.uint8)
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        tdt, ndt = _DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(bytes(raw[lo:hi]), dtype=ndt).copy()
        t = torch.from_numpy(arr)
        if tdt is torch.bfloat16:
            t = t.view(torch.bfloat16)
        out[name] = t.reshape(meta["shape"])
    return out


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor {name}: unsupported dtype {t.dtype}")
        b = (t.view(torch.int16) if t.dtype is torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json"), "r") as f:
        return json.load(f)
