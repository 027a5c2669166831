"""CUDA paths of the quantised matmuls (kernels: ``csrc/kernels/quant.cu``).

INT4: small batches (decode) run the split-K GEMV that streams the packed weights once; larger
``M`` expand the weight to a dense 16-bit matrix and run the tcgen05 GEMM; batches up to 128 rows
can instead take the fused W4A16 tcgen05 kernel (opt-in, see ``w4a16_enabled``).
INT8 blocks: quantise / dequantise kernels; the matmul dequantises then uses the GEMM.
"""
from __future__ import annotations

import os
from ctypes import c_int, c_longlong, c_void_p

import torch

from . import native
from ._lib import check, count_launch, ptr, stream_ptr

P, I = c_void_p, c_int
native.register_signature("rb_int4_gemv_splits", [I, I])
native.register_signature("rb_int4_gemv", [I, I, P, P, P, P, P, P, P, I, I, I, I, I, P])
native.register_signature("rb_int4_dequant", [I, I, P, P, P, P, I, I, I, P])
native.register_signature("rb_w4a16_slices", [I, I])
native.register_signature("rb_w4a16_gemm", [I, I, P, c_longlong, P, P, P, P, P, P, P, I, I, I, I, I, P])
native.register_signature("rb_w8a16_slices", [I, I])
native.register_signature("rb_w8a16_gemm", [I, P, c_longlong, P, I, P, P, P, P, I, I, I, P])
native.register_signature("rb_q8_quantize", [I, P, P, I, I, I, P])
native.register_signature("rb_q8_dequantize", [I, P, P, I, I, I, P])

GEMV_MAX_M = 32            # rows one GEMV launch handles (accumulators in registers)
GEMV_CHUNKED_MAX_M = 8     # batches up to this size use the GEMV; larger ones dequantise + tcgen05 GEMM
                           # (measured crossover on K 4096 x N 12288: GEMV 81 us at 8 rows, 118 us at 16;
                           # dequantise + GEMM 85-97 us for any batch up to 128)


def int4_dequant(qw, dtype: torch.dtype) -> torch.Tensor:
    dense = torch.empty((qw.k, qw.n), dtype=dtype, device=qw.packed.device)
    check(native.lib().rb_int4_dequant(native.dtype_code(dtype), native.dtype_code(qw.scales.dtype),
                                       ptr(qw.packed), ptr(qw.scales), ptr(qw.zero_points), ptr(dense),
                                       qw.n, qw.k, qw.group_size, stream_ptr()), "rb_int4_dequant")
    count_launch()
    return dense


# Batches of GEMV_CHUNKED_MAX_M+1 .. W4A16_MAX_M rows take the fused W4A16 tcgen05 kernel
# (csrc/kernels/w4a16_gemm.cu), which expands the packed weight inside shared memory instead of
# writing a dense 16-bit copy (RB_W4A16=0 switches back to dequantise + GEMM).
W4A16_MAX_M = 128
W4A16_ROUTE_MAX_M = 48     # above this the split-K additions of the fused kernel cost more than a dense copy


def w4a16_enabled() -> bool:
    return os.environ.get("RB_W4A16", "1") == "1"


def int4_matmul_fused(x: torch.Tensor, qw, bias=None, out=None):
    """The fused W4A16 kernel; returns ``None`` when the shape / alignment is outside what it covers.
    ``out``: contiguous ``[M, N]`` tensor to write into (for instance a peer-visible buffer)."""
    L = native.lib()
    M, K = x.shape
    if M > W4A16_MAX_M or x.dtype not in (torch.bfloat16, torch.float16):
        return None
    x = x.contiguous()
    y = out if out is not None else torch.empty((M, qw.n), dtype=x.dtype, device=x.device)
    ws = counters = None
    split = L.rb_w4a16_slices(qw.n, qw.padded_k) > 1
    if split:
        if os.environ.get("RB_W4A16_TWO_PASS", "0") == "1":
            ws = torch.empty((M, qw.n), dtype=torch.float32, device=x.device)     # cleared / converted by extra launches
        else:
            ws, counters = _w4_workspace(x.device, M * qw.n, (qw.n + 127) // 128)
    rc = L.rb_w4a16_gemm(native.dtype_code(x.dtype), native.dtype_code(qw.scales.dtype), ptr(x),
                         c_longlong(x.stride(0)), ptr(qw.packed), ptr(qw.scales), ptr(qw.zero_points),
                         ptr(bias), ptr(y), ptr(ws), ptr(counters), M, qw.n, K, qw.padded_k, qw.group_size,
                         stream_ptr())
    if rc == 51:
        return None
    check(rc, "rb_w4a16_gemm")
    count_launch(1 if (not split or counters is not None) else 3)
    return y


_W4_WS = {}


def _w4_workspace(device, numel: int, tiles: int):
    """Per-device, per-stream fp32 accumulation buffer and per-tile counters for split-K launches.
    Both are zero between launches (the kernel that finishes a tile puts them back), so consecutive
    launches on one stream share them; they only grow.  Launches on different streams may overlap, so
    each stream has its own pair; a kernel that gave up on a wait leaves them dirty, so they are
    dropped when a non-zero status word is read (``native.on_bad_status``)."""
    key = (device.type, device.index, int(torch.cuda.current_stream(device).cuda_stream))
    ws, cnt = _W4_WS.get(key, (None, None))
    if ws is None or ws.numel() < numel:
        ws = torch.zeros(max(numel, 1 << 22), dtype=torch.float32, device=device)
    if cnt is None or cnt.numel() < tiles:
        cnt = torch.zeros(max(tiles, 1024), dtype=torch.int32, device=device)
    _W4_WS[key] = (ws, cnt)
    return ws, cnt


native.on_bad_status(_W4_WS.clear)

_GEMV_SCRATCH = {}


def _gemv_scratch(device, numel: int) -> torch.Tensor:
    """Per-device split-K partial-sum buffer of the GEMV, reused by every call on the decode loop
    (the launches of one stream run in order; the buffer is fully rewritten by each launch before
    its reduction pass reads it).  It only grows."""
    key = (device.type, device.index)
    buf = _GEMV_SCRATCH.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1 << 20), dtype=torch.float32, device=device)
        _GEMV_SCRATCH[key] = buf
    return buf


def int4_matmul(x: torch.Tensor, qw, bias=None, out=None) -> torch.Tensor:
    """x [M, K] @ dequant(qw) [K, N]; ``out`` (optional): contiguous ``[M, N]`` destination."""
    L = native.lib()
    M, K = x.shape
    assert K == qw.k
    x = x.contiguous()
    if out is not None:
        assert out.shape == (M, qw.n) and out.dtype == x.dtype and out.is_contiguous()
    if GEMV_CHUNKED_MAX_M < M <= W4A16_ROUTE_MAX_M and w4a16_enabled():
        y = int4_matmul_fused(x, qw, bias, out)
        if y is not None:
            return y
    if M <= GEMV_CHUNKED_MAX_M:
        # decode batches: the packed weights are streamed once per 32 rows
        splits = L.rb_int4_gemv_splits(qw.padded_k, qw.n)
        y = out if out is not None else torch.empty((M, qw.n), dtype=x.dtype, device=x.device)
        scratch = _gemv_scratch(x.device, splits * min(M, GEMV_MAX_M) * qw.n)
        for r0 in range(0, M, GEMV_MAX_M):
            rows = min(GEMV_MAX_M, M - r0)
            check(L.rb_int4_gemv(native.dtype_code(x.dtype), native.dtype_code(qw.scales.dtype),
                                 ptr(x[r0:r0 + rows]), ptr(qw.packed), ptr(qw.scales),
                                 ptr(qw.zero_points), ptr(bias), ptr(y[r0:r0 + rows]), ptr(scratch),
                                 rows, qw.n, K, qw.padded_k, qw.group_size, stream_ptr()),
                  "rb_int4_gemv")
            count_launch(2)
        return y
    dense = int4_dequant(qw, x.dtype)
    return native.gemm(x, dense, bias=bias, out=out)


class QMatmulInt4Fn(torch.autograd.Function):
    """Frozen INT4 weight: only the activation gets a gradient, ``dX = dY @ dequant(W)^T``
    (reference: rumus-vision/src/shaders/qmatmul_int4_transpose.wgsl:38)."""

    @staticmethod
    def forward(ctx, x, qw):
        ctx.qw = qw
        return int4_matmul(x, qw)

    @staticmethod
    def backward(ctx, dy):
        dense = int4_dequant(ctx.qw, dy.dtype)
        return native.gemm(dy.contiguous(), dense.t()), None


def quantize_q8_cuda(weight: torch.Tensor, block_size: int):
    from ..nn.quant import Q8Tensor
    k, n = weight.shape
    w = weight.detach().contiguous()
    nb = (k * n + block_size - 1) // block_size
    out = torch.empty(nb * (4 + block_size), dtype=torch.uint8, device=w.device)
    check(native.lib().rb_q8_quantize(native.dtype_code(w.dtype), ptr(w), ptr(out), k, n, block_size,
                                      stream_ptr()), "rb_q8_quantize")
    count_launch()
    return Q8Tensor(k, n, block_size, out)


def dequantize_q8_cuda(q, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty((q.k, q.n), dtype=dtype, device=q.data.device)
    check(native.lib().rb_q8_dequantize(native.dtype_code(dtype), ptr(q.data), ptr(out), q.k, q.n,
                                        q.block_size, stream_ptr()), "rb_q8_dequantize")
    count_launch()
    return out


W8A16_MAX_M = 128          # rows one fused launch covers (the batch is the MMA's N dimension)
W8A16_MAX_CHUNKS = 4       # larger batches would re-read the weight more often than dequantising it once


def q8_matmul_fused(x: torch.Tensor, q, bias=None):
    """The fused W8A16 kernel (``csrc/kernels/w8a16_gemm.cu``): the quantised blocks are expanded in
    shared memory inside the GEMM.  Returns ``None`` when the shape / dtype is outside what it covers."""
    L = native.lib()
    M, K = x.shape
    if x.dtype not in (torch.bfloat16, torch.float16) or M > W8A16_MAX_M * W8A16_MAX_CHUNKS:
        return None
    if K % 8 or q.block_size % 8 or K != q.k:
        return None
    x = x.contiguous()
    y = torch.empty((M, q.n), dtype=x.dtype, device=x.device)
    ws = counters = None
    if L.rb_w8a16_slices(q.n, K) > 1:
        ws, counters = _w4_workspace(x.device, min(M, W8A16_MAX_M) * q.n, (q.n + 127) // 128)
    for r0 in range(0, M, W8A16_MAX_M):
        rows = min(W8A16_MAX_M, M - r0)
        rc = L.rb_w8a16_gemm(native.dtype_code(x.dtype), ptr(x[r0:r0 + rows]), c_longlong(x.stride(0)),
                             ptr(q.data), q.block_size, ptr(bias), ptr(y[r0:r0 + rows]), ptr(ws), ptr(counters),
                             rows, q.n, K, stream_ptr())
        if rc == 53:
            return None
        check(rc, "rb_w8a16_gemm")
        count_launch()
    return y


def matmul_q8_cuda(x: torch.Tensor, q, bias=None) -> torch.Tensor:
    """``x [M, K] @ dequant(q) [K, N]`` (+ bias): 16-bit batches of up to 512 rows run the fused
    dequantise-in-shared-memory kernel; fp32 activations and larger batches expand the weight once
    and use the dense GEMM."""
    y = q8_matmul_fused(x, q, bias)
    if y is not None:
        return y
    return native.gemm(x.contiguous(), dequantize_q8_cuda(q, x.dtype), bias=bias)
