"""Symmetric arena: one peer-mapped allocation per rank, sub-allocated by byte offset.

``torch.distributed._symmetric_memory`` does the plumbing (allocation, handle exchange over the
process group's store, peer mappings, NVLS multicast binding where the fabric supports it); the
kernels in ``csrc/comm`` only ever see the table of arena base pointers plus byte offsets, which
are identical on every rank because every rank performs the same sequence of ``alloc`` calls.

The first ``FLAG_BYTES`` of the arena hold 32-bit epoch flags (zeroed once at creation; they only
ever grow, see ``csrc/comm/comm_common.cuh``).

This replaces the reference's host-staged rendezvous (rumus-distributed/src/collective.rs:16-79,
rumus/src/nn/parallel.rs:134-250): "WebGPU has no peer-to-peer DMA"
(rumus/src/tensor/core.rs:1175) — NVLink does.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

FLAG_BYTES = 4 << 20


class SymmArena:
    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + FLAG_BYTES + 4095) // 4096 * 4096
        self.buf = symm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.hdl = symm.rendezvous(self.buf, self.group)
        self.base_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        assert self.base_ptrs[self.rank] == self.buf.data_ptr()
        mc = 0
        try:
            if os.environ.get("RB_MULTIMEM", "0") == "1" and self.hdl.has_multicast_support(
                    self.device.type, self.device.index):
                mc = int(self.hdl.multicast_ptr)
        except Exception:
            mc = 0
        self.mc_ptr = mc
        self.buf[:FLAG_BYTES].zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self._off = FLAG_BYTES
        self._flag_off = 0
        self._bases_c = (ctypes.c_void_p * 8)(*([ctypes.c_void_p(p) for p in self.base_ptrs]
                                                + [ctypes.c_void_p(0)] * (8 - self.world)))
        # small local (non-symmetric) scratch ints: counters that kernels reset themselves
        self.local_ints = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        self._local_int_off = 0

    # ------------------------------------------------------------------ allocation
    def alloc_bytes(self, nbytes: int, align: int = 1024) -> Tuple[torch.Tensor, int]:
        off = (self._off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {nbytes} at {off}, size {self.nbytes}")
        self._off = off + nbytes
        return self.buf[off:off + nbytes], off

    def alloc(self, numel: int, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        esz = torch.empty((), dtype=dtype).element_size()
        raw, off = self.alloc_bytes(numel * esz)
        t = raw.view(dtype)
        return t, off

    def alloc_flat(self, numel: int, dtype: torch.dtype, device=None) -> torch.Tensor:
        """Allocator signature used by ``flat.FlatUnit`` (zero-filled)."""
        t, off = self.alloc(numel, dtype)
        t.zero_()
        t.arena_offset = off
        return t

    def alloc_flags(self, n: int) -> int:
        """Returns the byte offset of ``n`` zero-initialised int32 flags."""
        off = self._flag_off
        if off + 4 * n > FLAG_BYTES:
            raise MemoryError("flag region exhausted")
        self._flag_off = (off + 4 * n + 127) // 128 * 128
        return off

    def alloc_local_ints(self, n: int) -> torch.Tensor:
        off = self._local_int_off
        assert off + n <= self.local_ints.numel()
        self._local_int_off = off + n
        return self.local_ints[off:off + n]

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.buf.data_ptr()
        assert 0 <= off < self.nbytes, "tensor is not inside the arena"
        return off

    # ------------------------------------------------------------------ access
    def bases(self):
        return self._bases_c

    def flag_view(self, off: int, n: int) -> torch.Tensor:
        return self.buf[off:off + 4 * n].view(torch.int32)

    def peer_tensor(self, rank: int, off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return self.hdl.get_buffer(rank, (numel,), dtype, storage_offset=off // torch.empty((), dtype=dtype).element_size())

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(self.group)
