"""Safetensors checkpoints, byte-compatible with the reference.

The reference saves every tensor as little-endian F32 with no metadata through the Rust
``safetensors`` crate (rumus/src/nn/io.rs:27-81) and refuses anything but F32 on load
(io.rs:102-107).  That crate's serializer orders entries by (dtype alignment descending, name
ascending), writes a compact JSON header ``{"name":{"dtype":..,"shape":..,"data_offsets":..}}``
padded with spaces to a multiple of 8 bytes, preceded by its length as a little-endian u64.
This module reproduces that byte stream directly (no dependency on the Python package; a test
compares both), writes atomically (tmp + rename), and loads F32 files.
"""
from __future__ import annotations

import json
import os
import struct
from collections import OrderedDict
from typing import Dict, Mapping

import numpy as np
import torch


def _to_f32_bytes(t: torch.Tensor) -> bytes:
    a = t.detach().to(device="cpu", dtype=torch.float32).contiguous().numpy()
    if a.dtype.byteorder == ">":  # pragma: no cover - big-endian hosts
        a = a.byteswap()
    return a.tobytes()


def serialize(state: Mapping[str, torch.Tensor]) -> bytes:
    names = sorted(state.keys())  # single dtype (F32): order is by name
    header = OrderedDict()
    blobs = []
    off = 0
    for name in names:
        t = state[name]
        b = _to_f32_bytes(t)
        header[name] = OrderedDict([("dtype", "F32"), ("shape", [int(s) for s in t.shape]),
                                    ("data_offsets", [off, off + len(b)])])
        blobs.append(b)
        off += len(b)
    hjson = json.dumps(header, separators=(",", ":"), ensure_ascii=False).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    return struct.pack("<Q", len(hjson)) + hjson + b"".join(blobs)


def save_safetensors(state: Mapping[str, torch.Tensor], path: str) -> None:
    """Atomic write of ``state`` (any dtype/device; stored as F32)."""
    data = serialize(state)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def load_safetensors(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 8:
        raise ValueError("safetensors: file too short")
    (n,) = struct.unpack("<Q", raw[:8])
    if 8 + n > len(raw):
        raise ValueError("safetensors: header length exceeds file size")
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    base = 8 + n
    out: Dict[str, torch.Tensor] = OrderedDict()
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] != "F32":
            raise ValueError(f"safetensors: unsupported dtype {info['dtype']} for {name!r}, expected F32")
        b, e = info["data_offsets"]
        if (e - b) % 4 != 0:
            raise ValueError(f"safetensors: data length {e - b} of {name!r} is not a multiple of 4")
        arr = np.frombuffer(raw, dtype="<f4", count=(e - b) // 4, offset=base + b)
        shape = [int(s) for s in info["shape"]]
        if int(np.prod(shape)) != arr.size:
            raise ValueError(f"safetensors: shape {shape} does not match data of {name!r}")
        out[name] = torch.from_numpy(arr.copy()).view(*shape).to(device)
    return out


def load_into(module: torch.nn.Module, path: str, strict: bool = False) -> None:
    """Load a checkpoint into ``module``: missing keys are skipped, a shape mismatch is an error
    (rumus/src/nn/parameter.rs:72-100)."""
    sd = load_safetensors(path)
    target = module.state_dict()
    for k, v in sd.items():
        if k in target and tuple(target[k].shape) != tuple(v.shape):
            raise ValueError(f"shape mismatch for {k!r}: checkpoint {tuple(v.shape)} vs model {tuple(target[k].shape)}")
    conv = {k: v.to(target[k].dtype) if k in target else v for k, v in sd.items()}
    module.load_state_dict(conv, strict=strict)
