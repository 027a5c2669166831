"""Native (C++) batch loader over a `.rrec` file of fixed-shape records.

Worker threads of ``csrc/runtime/batch_loader.cpp`` copy records from the memory-mapped file into
a ring of pinned host batches; iteration yields views of the ring (valid until the next item is
requested), ready for ``tensor.to(device, non_blocking=True)``.  Order, shuffling and ``drop_last``
match ``DataLoader`` over a ``RecordDataset`` of the same file (the reference's loader:
rumus/src/data/dataloader.rs:16-274, rumus/src/data/record.rs).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p
from typing import Iterator

import torch

from ..ops import _lib
from .dataset import DataItem

_DT = {0: torch.float32, 1: torch.float16}


def _bind(L):
    L.rbl_probe.argtypes = [c_char_p] + [POINTER(c_longlong)] * 3 + [POINTER(c_int)] * 6
    L.rbl_create.restype = c_void_p
    L.rbl_create.argtypes = [c_char_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    L.rbl_num_batches.restype = c_longlong
    L.rbl_num_batches.argtypes = [c_void_p]
    L.rbl_start_epoch.argtypes = [c_void_p, c_int]
    L.rbl_next.argtypes = [c_void_p, POINTER(c_int)]
    L.rbl_release.argtypes = [c_void_p, c_int]
    L.rbl_destroy.argtypes = [c_void_p]


class NativeBatchLoader:
    def __init__(self, path: str, batch_size: int, shuffle: bool = False, drop_last: bool = False,
                 num_workers: int = 4, prefetch_batches: int = 4, pin_memory: bool = True):
        if not _lib.have_host_lib():
            raise RuntimeError("the host library is not built (python -m rumus_b200.build)")
        self._L = _lib.host_lib()
        _bind(self._L)
        n, ib, tb = c_longlong(), c_longlong(), c_longlong()
        ind, itd, ind2, itd2 = c_int(), c_int(), c_int(), c_int()
        ish, tsh = (c_int * 8)(), (c_int * 8)()
        rc = self._L.rbl_probe(path.encode(), ctypes.byref(n), ctypes.byref(ib), ctypes.byref(tb),
                               ctypes.byref(ind), ish, ctypes.byref(itd), ctypes.byref(ind2), tsh,
                               ctypes.byref(itd2))
        if rc != 0:
            raise IOError(f"not a valid .rrec file: {path}")
        self.num_records = int(n.value)
        in_shape = tuple(ish[i] for i in range(ind.value))
        tg_shape = tuple(tsh[i] for i in range(ind2.value))
        self.shuffle, self.batch_size = shuffle, batch_size
        pin = pin_memory and torch.cuda.is_available()
        self._in = torch.empty((prefetch_batches, batch_size) + in_shape, dtype=_DT[itd.value],
                               pin_memory=pin)
        self._tg = torch.empty((prefetch_batches, batch_size) + tg_shape, dtype=_DT[itd2.value],
                               pin_memory=pin)
        assert self._in[0, 0].numel() * self._in.element_size() == ib.value
        assert self._tg[0, 0].numel() * self._tg.element_size() == tb.value
        h = self._L.rbl_create(path.encode(), batch_size, 1 if drop_last else 0, num_workers,
                               prefetch_batches, self._in.data_ptr(), self._tg.data_ptr())
        if not h:
            raise IOError(f"could not start the loader on {path}")
        self._h = c_void_p(h)

    def __len__(self) -> int:
        return int(self._L.rbl_num_batches(self._h))

    def __iter__(self) -> Iterator[DataItem]:
        self._L.rbl_start_epoch(self._h, 1 if self.shuffle else 0)
        held = -1
        rows = c_int()
        while True:
            if held >= 0:
                self._L.rbl_release(self._h, held)
                held = -1
            s = self._L.rbl_next(self._h, ctypes.byref(rows))
            if s == -1:
                return
            if s < 0:
                raise IOError("a record does not have the shape of record 0")
            held = s
            yield DataItem(self._in[s, :rows.value], self._tg[s, :rows.value])

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.rbl_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass
