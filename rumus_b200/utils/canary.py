"""Bounds-guard mode for kernel outputs: canary-padded allocations checked on the host.

Inside ``with canary_guard():`` every tensor that Python code allocates with ``torch.empty`` /
``empty_like`` / ``zeros`` / ``zeros_like`` / ``empty_strided`` (dense strides) — which is how every
kernel wrapper in ``rumus_b200.ops`` makes its outputs and scratch buffers — is carved out of a
larger buffer with a guard band of a known byte pattern on both sides.  When the block ends (after a
device synchronisation) the bands are compared on the host; a kernel that wrote outside its output
raises ``CanaryError`` naming the allocation (shape, dtype, which side, first damaged byte offset,
and the Python line that allocated it).

This stands in for a memory checker on machines where none can be run, and needs no change in the
kernels or their wrappers: the interception is a ``TorchFunctionMode``.  The guard bands are 4 KiB,
so payloads keep the 512-byte alignment the allocator gives them (TMA base addresses, 16-byte vector
accesses).  An overrun that jumps further than 4 KiB is not seen.

The reference relies on wgpu's robust-buffer-access bounds clamping and has no counterpart
(rumus/src/backend/gpu/compute.rs:296-345 only asserts uniform-struct sizes at compile time).
"""
from __future__ import annotations

import math
import traceback
from typing import List

import torch
from torch.overrides import TorchFunctionMode

GUARD_BYTES = 4096
PATTERN = 0xA5


class CanaryError(RuntimeError):
    pass


class _Record:
    __slots__ = ("buf", "nbytes", "shape", "dtype", "where")

    def __init__(self, buf, nbytes, shape, dtype, where):
        self.buf, self.nbytes, self.shape, self.dtype, self.where = buf, nbytes, shape, dtype, where


def _dense_strides(shape, strides) -> bool:
    expect = 1
    for n, s in zip(reversed(shape), reversed(strides)):
        if n != 1 and s != expect:
            return False
        expect *= n
    return True


class canary_guard(TorchFunctionMode):
    """Context manager; ``check()`` can also be called inside the block (it synchronises)."""

    def __init__(self, devices=("cuda",), guard_bytes: int = GUARD_BYTES):
        super().__init__()
        self.devices = tuple(devices)
        self.guard = int(guard_bytes)
        self.records: List[_Record] = []

    # ------------------------------------------------------------------ allocation
    def _alloc(self, shape, dtype, device, zero: bool):
        shape = tuple(int(s) for s in shape)
        dtype = dtype or torch.get_default_dtype()
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = math.prod(shape) * esz
        payload = (nbytes + 511) // 512 * 512          # the back band starts on an aligned address too
        buf = torch.empty(self.guard + payload + self.guard, dtype=torch.uint8, device=device)
        buf[: self.guard].fill_(PATTERN)
        buf[self.guard + nbytes:].fill_(PATTERN)
        body = buf[self.guard: self.guard + nbytes]
        if zero:
            body.zero_()
        frame = traceback.extract_stack(limit=6)
        where = next((f"{f.filename}:{f.lineno}" for f in reversed(frame)
                      if "canary.py" not in f.filename and "torch/" not in f.filename), "?")
        self.records.append(_Record(buf, nbytes, shape, dtype, where))
        return body.view(dtype).view(shape)

    def _wanted(self, device) -> bool:
        if device is None:
            return False
        return torch.device(device).type in self.devices

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        try:
            if func in (torch.empty, torch.zeros) and not kwargs.get("pin_memory") and kwargs.get("out") is None \
                    and kwargs.get("layout", torch.strided) == torch.strided and self._wanted(kwargs.get("device")):
                shape = args[0] if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)) else args
                if all(isinstance(s, int) for s in shape):
                    return self._alloc(shape, kwargs.get("dtype"), kwargs["device"], func is torch.zeros)
            elif func in (torch.empty_like, torch.zeros_like):
                src = args[0]
                dev = kwargs.get("device", src.device)
                fmt = kwargs.get("memory_format", torch.preserve_format)
                if self._wanted(dev) and src.layout == torch.strided and (
                        fmt == torch.contiguous_format or src.is_contiguous()):
                    return self._alloc(src.shape, kwargs.get("dtype", src.dtype), dev, func is torch.zeros_like)
            elif func is torch.empty_strided and self._wanted(kwargs.get("device")):
                shape, strides = args[0], args[1]
                if _dense_strides(shape, strides):
                    return self._alloc(shape, kwargs.get("dtype"), kwargs["device"], False)
        except CanaryError:
            raise
        return func(*args, **kwargs)

    # ------------------------------------------------------------------ checking
    def check(self) -> int:
        """Compares every guard band with the pattern; returns the number of allocations checked."""
        if torch.cuda.is_available() and "cuda" in self.devices:
            torch.cuda.synchronize()
        problems = []
        for r in self.records:
            front = r.buf[: self.guard]
            back = r.buf[self.guard + r.nbytes:]
            for side, band in (("before", front), ("after", back)):
                bad = (band != PATTERN).nonzero()
                if bad.numel():
                    off = int(bad[0]) if side == "after" else int(bad[-1]) - self.guard
                    problems.append(f"{tuple(r.shape)} {r.dtype} allocated at {r.where}: {bad.numel()} byte(s) "
                                    f"damaged {side} the tensor (first at byte offset {off:+d} from its "
                                    f"{'end' if side == 'after' else 'start'})")
        if problems:
            raise CanaryError("out-of-bounds write(s) detected:\n  " + "\n  ".join(problems))
        return len(self.records)

    def __exit__(self, exc_type, exc, tb):
        out = super().__exit__(exc_type, exc, tb)
        if exc_type is None:
            self.check()
        self.records.clear()
        return out
