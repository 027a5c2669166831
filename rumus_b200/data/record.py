"""`.rrec` record files (rumus/src/data/record.rs): sequential writer, memory-mapped reader.

The reader is the C++ mmap reader (``csrc/runtime/rrec_reader.cpp``) when the host library is
built, with a pure-Python fallback that parses the same bytes."""
from __future__ import annotations

import ctypes
import mmap
import struct
from ctypes import c_int, c_longlong, c_void_p

import numpy as np
import torch

from ..ops import _lib
from .dataset import DataItem, Dataset

MAGIC, VERSION, HEADER = b"RREC", 1, 64
_TAG = {torch.float32: 0, torch.float16: 1}
_NP = {0: np.dtype("<f4"), 1: np.dtype("<f2")}


class RecordWriter:
    def __init__(self, path: str):
        self.f = open(path, "wb")
        self.f.write(b"\0" * HEADER)
        self.index = []

    @staticmethod
    def create(path: str) -> "RecordWriter":
        return RecordWriter(path)

    def _write_tensor(self, t: torch.Tensor) -> int:
        if t.dtype not in _TAG:
            raise ValueError(f".rrec stores f32/f16 tensors, got {t.dtype}")
        t = t.detach().cpu().contiguous()
        meta = struct.pack("<I", t.dim()) + b"".join(struct.pack("<I", int(s)) for s in t.shape) \
            + struct.pack("<I", _TAG[t.dtype])
        data = t.numpy().astype(_NP[_TAG[t.dtype]], copy=False).tobytes()
        pad = (4 - len(data) % 4) % 4
        self.f.write(meta + data + b"\0" * pad)
        return len(meta) + len(data) + pad

    def append(self, input: torch.Tensor, target: torch.Tensor) -> None:
        off = self.f.tell()
        n = self._write_tensor(input) + self._write_tensor(target)
        self.index.append((off, n))

    def finish(self) -> None:
        index_off = self.f.tell()
        for off, n in self.index:
            self.f.write(struct.pack("<QQ", off, n))
        self.f.seek(0)
        self.f.write(MAGIC + struct.pack("<IQQ", VERSION, len(self.index), index_off))
        self.f.close()


class RecordDataset(Dataset):
    def __init__(self, path: str, force_python: bool = False):
        self.path = path
        self._h = None
        if _lib.have_host_lib() and not force_python:
            L = _lib.host_lib()
            L.rrec_open.restype = c_void_p
            L.rrec_open.argtypes = [ctypes.c_char_p]
            L.rrec_close.argtypes = [c_void_p]
            L.rrec_len.restype = c_longlong
            L.rrec_len.argtypes = [c_void_p]
            L.rrec_tensor.restype = c_longlong
            L.rrec_tensor.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            h = L.rrec_open(path.encode())
            if not h:
                raise IOError(f"not a valid .rrec file: {path}")
            self._L, self._h = L, c_void_p(h)
            self._n = int(L.rrec_len(self._h))
        else:
            self._f = open(path, "rb")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
            if self._mm[:4] != MAGIC or struct.unpack("<I", self._mm[4:8])[0] != VERSION:
                raise IOError(f"not a valid .rrec file: {path}")
            self._n, self._index_off = struct.unpack("<QQ", self._mm[8:24])

    @staticmethod
    def open(path: str) -> "RecordDataset":
        return RecordDataset(path)

    def __len__(self):
        return self._n

    def __del__(self):
        try:
            if self._h is not None:
                self._L.rrec_close(self._h)
        except Exception:
            pass

    def _native_tensor(self, idx: int, which: int) -> torch.Tensor:
        nd, dt = c_int(0), c_int(0)
        shape = (c_int * 8)()
        data = c_void_p(0)
        nbytes = self._L.rrec_tensor(self._h, idx, which, ctypes.byref(nd), shape, ctypes.byref(dt),
                                     ctypes.byref(data))
        if nbytes < 0:
            raise IndexError(f"bad record {idx}")
        buf = (ctypes.c_char * nbytes).from_address(data.value) if nbytes else b""
        arr = np.frombuffer(buf, dtype=_NP[dt.value]).reshape([shape[i] for i in range(nd.value)])
        return torch.from_numpy(arr.copy())

    def _py_tensor(self, p: int):
        mm = self._mm
        nd = struct.unpack("<I", mm[p:p + 4])[0]
        shape = struct.unpack(f"<{nd}I", mm[p + 4:p + 4 + 4 * nd]) if nd else ()
        tag = struct.unpack("<I", mm[p + 4 + 4 * nd:p + 8 + 4 * nd])[0]
        numel = int(np.prod(shape)) if nd else 1
        nbytes = numel * _NP[tag].itemsize
        d = p + 8 + 4 * nd
        arr = np.frombuffer(mm, dtype=_NP[tag], count=numel, offset=d).reshape(shape)
        return torch.from_numpy(arr.copy()), d + ((nbytes + 3) & ~3)

    def get(self, index: int) -> DataItem:
        if index < 0 or index >= self._n:
            raise IndexError(index)
        if self._h is not None:
            return DataItem(self._native_tensor(index, 0), self._native_tensor(index, 1))
        off, _ = struct.unpack("<QQ", self._mm[self._index_off + 16 * index:self._index_off + 16 * index + 16])
        x, p = self._py_tensor(off)
        y, _ = self._py_tensor(p)
        return DataItem(x, y)
