"""Python launchers for the fused collective kernels in ``csrc/comm`` (symmetric-arena based)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..ops import native
from ..ops._lib import check, count_launch, ptr, stream_ptr
from .symm import SymmArena

P, LL, I, F = c_void_p, c_longlong, c_int, c_float
native.register_signature("rb_rs_adam", [I, P, P, I, I, LL, LL, LL, LL, P, P, P, F, F, F, F, F, F, F,
                                         I, P, P, LL, LL, I, P, I, I, P])
native.register_signature("rb_signal_peers", [P, I, I, LL, I, P])
native.register_signature("rb_group_barrier", [P, I, I, LL, I, P])
native.register_signature("rb_all_gather", [P, I, I, LL, LL, LL, P, LL, I, I, P])
native.register_signature("rb_shard_gather", [P, I, I, LL, P, LL, LL, I, I, P])
native.register_signature("rb_allreduce_unscale", [I, P, P, I, I, LL, LL, LL, LL, LL, I, P, F, P, P,
                                                   I, I, P])
native.register_signature("rb_gemm_rs_push", [I, P, I, I, P, LL, P, LL, I, I, I, I, LL, LL, P, I, P, P, P, P])
native.register_signature("rb_oneshot_allreduce", [I, P, P, I, I, LL, LL, I, LL, P, P, I, I, P, P])
native.register_signature("rb_ag_gemm", [I, P, I, I, LL, LL, LL, P, LL, I, I, LL, P, LL, I, I, I, I,
                                         P, LL, P, P, LL, I, P, I, P])
native.register_signature("rb_gemm_rs", [I, P, I, I, P, LL, P, LL, I, I, I, I, LL, LL, P, I, P, P, P,
                                         I, P])


def rs_adam(arena: SymmArena, dtype, grad_off, param_off, shard_lo, shard_n, master, m, v, *, lr,
            beta1, beta2, eps, weight_decay, step, adamw, grad_flags_off, param_flags_off, epoch,
            done_counter, grad_scale=None, skip=None, ctas: int = 32):
    L = native.lib()
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    rc = L.rb_rs_adam(native.dtype_code(dtype), arena.bases(), c_void_p(arena.mc_ptr), arena.world,
                      arena.rank, grad_off, param_off, shard_lo, shard_n, ptr(master), ptr(m), ptr(v),
                      lr, beta1, beta2, eps, weight_decay, bc1, bc2, 1 if adamw else 0,
                      ptr(grad_scale), ptr(skip), grad_flags_off, param_flags_off, epoch,
                      ptr(done_counter), 1 if arena.mc_ptr else 0, ctas, stream_ptr())
    check(rc, "rb_rs_adam")
    count_launch(2)   # flag gate + worker


def signal_peers(arena: SymmArena, flags_off: int, epoch: int):
    """Stream-ordered: write ``epoch`` into slot ``[rank]`` of every peer's flag array."""
    check(native.lib().rb_signal_peers(arena.bases(), arena.world, arena.rank, flags_off, epoch,
                                       stream_ptr()), "rb_signal_peers")
    count_launch()


def group_barrier(arena: SymmArena, flags_off: int, epoch: int):
    """Stream-ordered barrier over the arena's ranks (one-warp kernel: signal, then bounded wait)."""
    check(native.lib().rb_group_barrier(arena.bases(), arena.world, arena.rank, flags_off, epoch,
                                        stream_ptr()), "rb_group_barrier")
    count_launch()


def all_gather(arena: SymmArena, buf_off: int, shard_bytes: int, *, src_flags_off: int = -1,
               chunk_flags: Optional[torch.Tensor] = None, chunk_bytes: int = 0, epoch: int = 1,
               ctas: int = 16):
    L = native.lib()
    rc = L.rb_all_gather(arena.bases(), arena.world, arena.rank, buf_off, shard_bytes, src_flags_off,
                         ptr(chunk_flags), chunk_bytes, epoch, ctas, stream_ptr())
    check(rc, "rb_all_gather")
    count_launch(2 if src_flags_off >= 0 else 1)


def shard_gather(arena: SymmArena, src_off: int, dst: torch.Tensor, shard_bytes: int, *,
                 src_flags_off: int = -1, epoch: int = 0, ctas: int = 16):
    """Every rank's shard buffer (arena offset ``src_off``) -> local ``dst`` (world * shard_bytes)."""
    assert dst.is_contiguous() and dst.numel() * dst.element_size() >= arena.world * shard_bytes
    rc = native.lib().rb_shard_gather(arena.bases(), arena.world, arena.rank, src_off, ptr(dst), shard_bytes,
                                      src_flags_off, epoch, ctas, stream_ptr())
    check(rc, "rb_shard_gather")
    count_launch(2 if src_flags_off >= 0 else 1)


def allreduce_unscale(arena: SymmArena, buf: torch.Tensor, *, enter_flags_off, exit_flags_off,
                      inf_flags_off, epoch, inv_scale=None, extra_scale: float = 1.0, found_inf=None,
                      done_counter=None, ctas: int = 32):
    """In-place all-reduce of an arena-resident flat buffer: ``buf = sum_r buf_r * inv_scale *
    extra_scale`` with a job-wide non-finite flag."""
    L = native.lib()
    rc = L.rb_allreduce_unscale(native.dtype_code(buf.dtype), arena.bases(), c_void_p(arena.mc_ptr),
                                arena.world, arena.rank, arena.offset_of(buf), buf.numel(),
                                enter_flags_off, exit_flags_off, inf_flags_off, epoch, ptr(inv_scale),
                                float(extra_scale), ptr(found_inf), ptr(done_counter),
                                1 if arena.mc_ptr else 0, ctas, stream_ptr())
    check(rc, "rb_allreduce_unscale")
    count_launch()


def ag_gemm(arena: SymmArena, *, buf_off: int, shard_bytes: int, chunk_flags: torch.Tensor,
            chunk_bytes: int, epoch: int, gather_a: bool, operand_off: int, other: torch.Tensor,
            M: int, N: int, K: int, out: torch.Tensor, src_flags_off: int = -1, bias=None,
            residual=None, act: Optional[str] = None, aux_out=None, n_copy_ctas: int = 16):
    """All-gather -> GEMM in one launch; see ``csrc/comm/tp_comm.cu``.

    ``other`` is the operand that is NOT gathered: B (``[K,N]`` or a ``.t()`` view of ``[N,K]``)
    when ``gather_a``, else A ``[M,K]`` row-major.
    """
    L = native.lib()
    if gather_a:
        bt, ld_other = native._mat_major(other)
        assert bt is not None
        b_mn = 0 if bt else 1
    else:
        assert other.stride(1) == 1
        ld_other = other.stride(0) if other.shape[0] > 1 else K
        b_mn = 1
    rc = L.rb_ag_gemm(native.dtype_code(out.dtype), arena.bases(), arena.world, arena.rank, buf_off,
                      shard_bytes, src_flags_off, ptr(chunk_flags), chunk_bytes, epoch,
                      1 if gather_a else 0, operand_off, ptr(other), ld_other, b_mn, M, N, K,
                      ptr(out), out.stride(0) if M > 1 else N, ptr(bias), ptr(residual),
                      (residual.stride(0) if residual is not None else 0),
                      native.ACT_CODES[act], ptr(aux_out), n_copy_ctas, stream_ptr())
    check(rc, "rb_ag_gemm")
    count_launch()
    return out


def gemm_rs(arena: SymmArena, a: torch.Tensor, b: torch.Tensor, *, partial_off: int,
            tile_flags_off: int, tile_counters: torch.Tensor, epoch: int, out: torch.Tensor,
            bias=None, residual=None, n_reduce_ctas: int = 0):
    """GEMM -> reduce-scatter in one launch: ``out [M/W, N]`` = this rank's rows of ``sum_r a_r @ b_r``."""
    L = native.lib()
    M, K = a.shape
    _, N = b.shape
    assert a.stride(1) == 1
    bt, ldb = native._mat_major(b)
    assert bt is not None
    rc = L.rb_gemm_rs(native.dtype_code(a.dtype), arena.bases(), arena.world, arena.rank, ptr(a),
                      a.stride(0) if M > 1 else K, ptr(b), ldb, 0 if bt else 1, M, N, K, partial_off,
                      tile_flags_off, ptr(tile_counters), epoch, ptr(out), ptr(bias), ptr(residual),
                      n_reduce_ctas, stream_ptr())
    check(rc, "rb_gemm_rs")
    count_launch()
    return out


def gemm_rs_push(arena: SymmArena, a: torch.Tensor, b: torch.Tensor, *, slots_off: int, done_flags_off: int,
                 owner_counters: torch.Tensor, epoch: int, out: torch.Tensor, bias=None, residual=None):
    """GEMM -> reduce-scatter with the transfer pushed from the GEMM's epilogue: every tile is stored,
    in the compute dtype, into the OWNER rank's slot for this source rank (plain stores over NVLink, no
    atomics: slots of different sources are disjoint), and each rank ends with a local pass
    ``out = sum of its slots + bias + residual``.  ``out [M/W, N]``; ``slots_off`` is the arena offset of a
    ``[W][M/W, N]`` slot set and the caller alternates between two sets (``csrc/comm/tp_comm.cu``)."""
    L = native.lib()
    M, K = a.shape
    _, N = b.shape
    assert a.stride(1) == 1 and out.is_contiguous()
    bt, ldb = native._mat_major(b)
    assert bt is not None
    if residual is not None:
        assert residual.is_contiguous() and residual.shape == out.shape
    rc = L.rb_gemm_rs_push(native.dtype_code(a.dtype), arena.bases(), arena.world, arena.rank, ptr(a),
                           a.stride(0) if M > 1 else K, ptr(b), ldb, 0 if bt else 1, M, N, K, slots_off,
                           done_flags_off, ptr(owner_counters), epoch, ptr(out), ptr(bias), ptr(residual),
                           stream_ptr())
    check(rc, "rb_gemm_rs_push")
    count_launch()
    return out


def oneshot_allreduce(arena: SymmArena, partial: torch.Tensor, out: torch.Tensor, *, flags_off: int, epoch: int,
                      residual: Optional[torch.Tensor] = None, ctas: int = 32,
                      epoch_base: Optional[torch.Tensor] = None):
    """``out = residual + sum over ranks of partial`` for a small arena-resident ``partial`` (decode
    activations): one flag round and one pass of peer loads (``csrc/comm/oneshot_allreduce.cu``).  The
    caller alternates ``partial`` between two arena buffers from one call to the next.  ``epoch_base``
    (an int32 device tensor) is added to ``epoch`` on the device: a launch captured in a CUDA graph keeps
    its arguments, so the caller moves the epochs forward through that word between replays."""
    assert partial.is_contiguous() and out.is_contiguous() and out.numel() == partial.numel()
    if residual is not None:
        assert residual.is_contiguous() and residual.numel() == partial.numel() and residual.dtype == partial.dtype
    rc = native.lib().rb_oneshot_allreduce(native.dtype_code(partial.dtype), arena.bases(), c_void_p(arena.mc_ptr),
                                           arena.world, arena.rank, arena.offset_of(partial), flags_off, epoch,
                                           partial.numel(), ptr(residual), ptr(out), 1 if arena.mc_ptr else 0,
                                           ctas, ptr(epoch_base), stream_ptr())
    check(rc, "rb_oneshot_allreduce")
    count_launch()
    return out
