"""Symmetric arena: one peer-mapped allocation per rank, sub-allocated by byte offset.

Two implementations of the plumbing: by default ``torch.distributed._symmetric_memory``
(allocation, handle exchange over the process group's store, peer mappings, NVLS multicast binding
where the fabric supports it); with ``RB_NATIVE_ARENA=1`` the framework's own allocator
(``NativeSymmArena`` below: driver VMM allocation, file-descriptor exchange over Unix sockets, peer
mappings, no multicast).  Either way the
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
    def __new__(cls, *args, **kwargs):
        # RB_NATIVE_ARENA=1 swaps in the framework's own allocator at every construction site
        if cls is SymmArena and os.environ.get("RB_NATIVE_ARENA", "0") == "1":
            return object.__new__(NativeSymmArena)
        return object.__new__(cls)

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + FLAG_BYTES + 4095) // 4096 * 4096
        self._map()
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

    def _map(self) -> None:
        """Allocate this rank's arena and map every peer's: sets ``buf``, ``base_ptrs``, ``mc_ptr``."""
        if self.world == 1:
            # a group of one has no peer to map: plain device memory serves (this is how the fused
            # collective kernels run on a single GPU, e.g. under a profiler)
            self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            self.hdl = None
            self.base_ptrs = [self.buf.data_ptr()]
            self.mc_ptr = 0
            return
        import torch.distributed._symmetric_memory as symm
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


class _RawDeviceBytes:
    """Lets ``torch.as_tensor`` wrap device memory that torch did not allocate."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner   # keeps the mapping alive as long as a tensor views it
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class NativeSymmArena(SymmArena):
    """The same arena on the framework's own allocator (``csrc/comm/symm_arena.cu``): physical
    memory from the driver's virtual-memory-management API, exported as a file descriptor, passed to
    the peers of the node over Unix sockets (``csrc/runtime/fd_exchange.cpp``) and mapped by each.
    Plain peer loads / stores only — no multicast object is bound (``mc_ptr`` is 0).
    Selected with ``RB_NATIVE_ARENA=1`` wherever a ``SymmArena`` is constructed."""

    def _map(self) -> None:
        import shutil
        import tempfile
        from ctypes import byref, c_int, c_longlong, c_ulonglong, c_void_p
        from ..ops import _lib, native
        L = native.lib()
        L.rb_arena_base.restype = c_ulonglong
        L.rb_arena_bytes.restype = c_longlong
        h = c_void_p(0)
        _lib.check(L.rb_arena_create(c_longlong(self.nbytes), c_int(self.device.index), c_int(self.rank),
                                     c_int(self.world), byref(h)), "rb_arena_create")
        self._h, self._L = h, L
        fd = c_int(-1)
        _lib.check(L.rb_arena_export_fd(h, byref(fd)), "rb_arena_export_fd")
        box = [tempfile.mkdtemp(prefix="rb-arena-") if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
        fds = (c_int * self.world)()
        rc = _lib.host_lib().rb_fd_exchange(box[0].encode(), c_int(self.rank), c_int(self.world), fd,
                                            fds, c_int(30000))
        if rc:
            raise RuntimeError(f"file-descriptor exchange between ranks failed (code {rc})")
        try:
            for r in range(self.world):
                if r != self.rank:
                    _lib.check(L.rb_arena_import_peer(h, c_int(r), c_int(fds[r])), "rb_arena_import_peer")
        finally:
            for r in range(self.world):
                if fds[r] >= 0:
                    os.close(fds[r])      # the mappings keep the memory alive; fds[rank] is the exported fd
        dist.barrier(self.group)
        if self.rank == 0:
            shutil.rmtree(box[0], ignore_errors=True)
        self.mapped_bytes = int(L.rb_arena_bytes(h))
        self.base_ptrs = [int(L.rb_arena_base(h, c_int(r))) for r in range(self.world)]
        assert all(self.base_ptrs)
        self.buf = torch.as_tensor(_RawDeviceBytes(self.base_ptrs[self.rank], self.nbytes, self),
                                   device=self.device)
        self.mc_ptr = 0
        self.hdl = None

    def peer_tensor(self, rank: int, off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        raw = torch.as_tensor(_RawDeviceBytes(self.base_ptrs[rank] + off, numel * esz, self), device=self.device)
        return raw.view(dtype)

    def close(self) -> None:
        """Collective: every rank calls it once no kernel uses the arena any more.  Tensors that
        view the arena must not be used afterwards."""
        if getattr(self, "_h", None):
            self.barrier()
            self._L.rb_arena_destroy(self._h)
            self._h = None
