"""Typed ctypes wrappers over the ``extern "C"`` launchers of the CUDA library.

Each wrapper takes torch tensors, validates what the kernel assumes (device,
dtype, contiguity), allocates outputs with torch, launches on the current CUDA
stream and returns tensors.  No autograd here — see ``functional.py``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p, c_uint
from typing import Optional

import torch

from . import _lib
from ._lib import check, count_launch, ptr, stream_ptr

DT_F32, DT_F16, DT_BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3
ACT_CODES = {None: 0, "none": 0, "relu": 1, "gelu": 2, "silu": 3}
UN_CODES = {"relu": 1, "gelu": 2, "silu": 3, "sigmoid": 4, "tanh": 5, "leaky_relu": 6, "scale": 7,
            "copy": 8}
BIN_CODES = {"add": 1, "sub": 2, "mul": 3}

_sig_done = False


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return DT_F32
    if dt == torch.float16:
        return DT_F16
    if dt == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"unsupported dtype {dt}")


def _L():
    global _sig_done
    lib = _lib.cuda_lib()
    if not _sig_done:
        _declare(lib)
        _sig_done = True
    return lib


def _declare(lib) -> None:
    P, LL, I, F = c_void_p, c_longlong, c_int, c_float
    lib.rb_gemm.argtypes = [I, I, I, P, LL, P, LL, I, I, I, P, LL, I, P, P, LL, P, LL, P, LL, I, I,
                            F, I, I, I, I, P, P]
    lib.rb_gemm_2cta.argtypes = [I, I, I, P, LL, P, LL, I, I, I, P, LL, I, P, P, LL, P, LL, P, LL, I, I,
                                 F, I, I, P]
    lib.rb_gemm_2cta_set_debug.argtypes = [P]
    lib.rb_gemm_2cta_set_debug.restype = None
    lib.rb_bmm_simt.argtypes = [I, I, I, P, LL, LL, P, LL, LL, I, I, I, I, P, LL, LL, I, F, P]
    lib.rb_norm_fwd.argtypes = [I, I, P, P, P, P, P, P, P, LL, I, F, P]
    lib.rb_norm_bwd_partials.argtypes = [LL]
    lib.rb_norm_bwd.argtypes = [I, I, P, P, P, P, P, P, P, P, P, LL, I, P]
    lib.rb_softmax_fwd.argtypes = [I, P, P, LL, I, P]
    lib.rb_softmax_bwd.argtypes = [I, P, P, P, LL, I, P]
    lib.rb_cross_entropy.argtypes = [I, P, P, P, P, P, LL, I, LL, F, F, P]
    lib.rb_reduce_sum_f32.argtypes = [P, LL, F, P, P]
    lib.rb_unary.argtypes = [I, P, P, LL, I, F, P]
    lib.rb_unary_bwd.argtypes = [I, P, P, P, LL, I, F, P]
    lib.rb_binary.argtypes = [I, P, P, P, LL, I, F, P]
    lib.rb_cast.argtypes = [I, I, P, P, LL, F, P]
    lib.rb_swiglu_fwd.argtypes = [I, P, P, LL, I, LL, P]
    lib.rb_swiglu_bwd.argtypes = [I, P, P, P, LL, I, LL, P]
    lib.rb_dropout.argtypes = [I, P, P, LL, c_uint, F, P]
    lib.rb_embedding_fwd.argtypes = [I, P, P, P, P, LL, I, I, I, P]
    lib.rb_embedding_bwd.argtypes = [I, P, P, P, P, LL, I, I, I, P]
    lib.rb_rope.argtypes = [I, P, P, LL, I, I, I, LL, I, F, I, P]
    lib.rb_colsum_slabs.argtypes = [LL]
    lib.rb_colsum.argtypes = [I, P, P, P, LL, I, LL, P]
    lib.rb_adam_flat.argtypes = [I, P, P, P, P, P, LL, F, F, F, F, F, F, F, I, P, P, P, P]
    lib.rb_scaler_update.argtypes = [P, P, P, P, F, F, I, P]
    lib.rb_sumsq_partials.argtypes = [I, P, LL, P, I, P, P]
    lib.rb_norm_finalize.argtypes = [P, I, F, F, P, P, P]
    lib.rb_scale_check.argtypes = [I, P, LL, P, F, P, P]
    lib.rb_multi_tensor_adam.argtypes = [P, I, F, F, F, F, F, F, F, I, P, P, P, P]
    lib.rb_multi_tensor_sgd.argtypes = [P, I, F, F, F, P, P, P]
    for name in ("rb_read_status", "rb_sm_count", "rb_init_device"):
        getattr(lib, name).argtypes = []
    # optional symbols (present once the corresponding source is built)
    for name, sig in _OPTIONAL_SIGS.items():
        if hasattr(lib, name):
            getattr(lib, name).argtypes = sig


_OPTIONAL_SIGS: dict = {}


def register_signature(name: str, argtypes) -> None:
    """Lets other modules (attention, conv, comm, ...) declare their launchers."""
    _OPTIONAL_SIGS[name] = argtypes
    if _sig_done and _lib._cuda_lib is not None and hasattr(_lib._cuda_lib, name):
        getattr(_lib._cuda_lib, name).argtypes = argtypes


def lib():
    return _L()


_BAD_STATUS_HOOKS = []


def on_bad_status(fn) -> None:
    """Registers ``fn()`` to run whenever a non-zero device status word is read: a kernel that gave up
    on a bounded wait may have left shared scratch state (split-K workspaces, tile counters) half
    written, and whoever caches such state drops it here."""
    _BAD_STATUS_HOOKS.append(fn)


def read_status() -> int:
    """Synchronises and returns the device status word (0 = clean), clearing it."""
    s = int(_L().rb_read_status())
    if s != 0:
        for fn in _BAD_STATUS_HOOKS:
            fn()
    return s


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out (the kernel returned normally)."""


def raise_on_status(where: str = "") -> None:
    s = read_status()
    if s != 0:
        raise DeviceWaitTimeout(f"device status {s} after {where}")


# ----------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------
def _mat_major(t: torch.Tensor):
    """Returns (is_transposed_storage, leading_dim) for a 2-D tensor whose storage is row-major
    either as given (stride (ld,1)) or as its transpose (stride (1,ld))."""
    assert t.dim() == 2
    r, c = t.shape
    s0, s1 = t.stride()
    if s1 == 1 and (s0 >= c or r == 1):
        return False, max(s0, c) if r > 1 else max(c, 1)
    if s0 == 1 and (s1 >= r or c == 1):
        return True, max(s1, r) if c > 1 else max(r, 1)
    return None, None


_SM_COUNT = None


def sm_count() -> int:
    """SMs of the current device (cached)."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = int(_L().rb_sm_count())
    return _SM_COUNT


def _use_2cta(M: int, N: int) -> bool:
    """Large 16-bit GEMMs run on CTA pairs (256- or 512-row tiles, 256 columns): less operand traffic
    per FLOP, which is what the power-capped sustained rate follows.  Problems with fewer than half a
    wave of such tiles, or fewer than 256 columns, keep the one-CTA kernel's smaller tiles.
    ``RB_GEMM_2CTA=0`` switches the pair kernel off."""
    if os.environ.get("RB_GEMM_2CTA", "1") != "1" or N < 256 or M < 256:
        return False
    return ((M + 255) // 256) * ((N + 255) // 256) * 4 >= sm_count()


def gemm(a: torch.Tensor, b: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
         act: Optional[str] = None, residual: Optional[torch.Tensor] = None,
         aux_out: bool = False, aux_in: Optional[torch.Tensor] = None, dact: Optional[str] = None,
         out_dtype: Optional[torch.dtype] = None, alpha: float = 1.0,
         out: Optional[torch.Tensor] = None, path: int = 0, bn: int = 0, max_ctas: int = 0,
         split_k: int = 0, mt: int = 0):
    """``out = dact'(aux_in) * act(alpha * a @ b + bias) + residual``.

    ``a`` is logical [M,K], ``b`` logical [K,N]; either may be a transposed view
    (``x.t()``) — the storage order is passed to the kernel as the operand's
    "major", nothing is copied.  Returns ``out`` or ``(out, pre_activation)``
    when ``aux_out``.

    ``path``: 0 automatic, 1 force the one-CTA tcgen05 kernel, 2 force the SIMT kernel, 3 force the
    two-CTA tcgen05 kernel (taken automatically for large 16-bit problems); ``mt`` picks its tile:
    0 automatic, 1 = 256 x 256, 2 = 512 x 256.

    ``split_k`` (0 = automatic): when the output has far fewer tiles than the GPU has SMs and K
    is long (weight gradients of convolutions: M, N a few hundred, K = batch x pixels), K is cut
    into slices that run as separate work items adding into an fp32 buffer.
    """
    L = _L()
    assert a.is_cuda and b.is_cuda and a.dtype == b.dtype
    M, K = a.shape
    K2, N = b.shape
    assert K == K2, (a.shape, b.shape)
    at, lda = _mat_major(a)
    if at is None:
        a = a.contiguous()
        at, lda = False, K
    bt, ldb = _mat_major(b)
    if bt is None:
        b = b.contiguous()
        bt, ldb = False, N
    if a.dtype == torch.float32 and path != 2:
        # the tf32 tensor-core path takes K-major operands only: restage the other layouts
        if at:
            a = a.contiguous()
            at, lda = False, K
        if not bt:
            b = b.t().contiguous().t()
            bt, ldb = True, K
    # kernel convention: a_mn=1 when A is stored [K,M]; b_mn=1 when B is stored [K,N]
    a_mn = 1 if at else 0
    b_mn = 0 if bt else 1
    dt = dtype_code(a.dtype)
    odt = out_dtype or a.dtype
    out_f32 = 1 if (odt == torch.float32) else 0
    assert odt in (a.dtype, torch.float32)
    if out is None:
        out = torch.empty((M, N), dtype=odt, device=a.device)
    else:
        assert out.shape == (M, N) and out.dtype == odt and out.stride(1) == 1
    pre = torch.empty((M, N), dtype=odt, device=a.device) if aux_out else None
    if bias is not None:
        assert bias.dtype == a.dtype and bias.is_contiguous() and bias.numel() == N
    if residual is not None:
        assert residual.dtype == odt and residual.shape == (M, N) and residual.stride(1) == 1
    if aux_in is not None:
        assert aux_in.dtype == odt and aux_in.shape == (M, N) and aux_in.stride(1) == 1
    plain = bias is None and act is None and not aux_out and aux_in is None and dact is None
    if split_k == 0 and plain and path != 2 and K >= 4096:
        tiles = ((M + 127) // 128) * ((N + 127) // 128)
        sms = sm_count()
        if tiles * 2 <= sms:
            split_k = max(1, min(sms // tiles, K // 1024))
    if split_k > 1 and plain:
        ws = torch.zeros((M, N), dtype=torch.float32, device=a.device)
        used = c_int(0)
        rc = L.rb_gemm(dt, a_mn, b_mn, ptr(a), lda, ptr(b), ldb, M, N, K, ptr(ws), N, 1, None, None, 0,
                       None, N, None, 0, 0, 0, float(alpha), path, bn, max_ctas, split_k,
                       ctypes.addressof(used), stream_ptr())
        check(rc, "rb_gemm")
        count_launch()
        gemm.last_path = used.value
        if residual is not None:
            ws.add_(residual)
        out.copy_(ws)
        return out
    if path in (0, 3) and a.dtype != torch.float32 and M >= 256 and N >= 256 and (path == 3 or _use_2cta(M, N)):
        # two-CTA kernel (each SM stages half of the B tile), see gemm_pair.cuh
        rc = L.rb_gemm_2cta(dt, a_mn, b_mn, ptr(a), lda, ptr(b), ldb, M, N, K, ptr(out), out.stride(0),
                            out_f32, ptr(bias), ptr(residual),
                            residual.stride(0) if residual is not None else 0, ptr(pre), N, ptr(aux_in),
                            aux_in.stride(0) if aux_in is not None else 0, ACT_CODES[act], ACT_CODES[dact],
                            float(alpha), max_ctas, mt, stream_ptr())
        if rc != 13:
            check(rc, "rb_gemm_2cta")
            count_launch()
            gemm.last_path = 3
            return (out, pre) if aux_out else out
        if path == 3:
            raise ValueError("operands are outside what the two-CTA GEMM covers")
    used = c_int(0)
    rc = L.rb_gemm(dt, a_mn, b_mn, ptr(a), lda, ptr(b), ldb, M, N, K, ptr(out), out.stride(0) if M > 1 else N,
                   out_f32, ptr(bias), ptr(residual),
                   (residual.stride(0) if M > 1 else N) if residual is not None else 0,
                   ptr(pre), N, ptr(aux_in),
                   (aux_in.stride(0) if M > 1 else N) if aux_in is not None else 0,
                   ACT_CODES[act], ACT_CODES[dact], float(alpha), path, bn, max_ctas, 1,
                   ctypes.addressof(used), stream_ptr())
    check(rc, "rb_gemm")
    count_launch()
    gemm.last_path = used.value
    return (out, pre) if aux_out else out


gemm.last_path = 0


def bmm(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """Batched matmul [B,M,K] @ [B,K,N] (any inner strides via transposed views)."""
    L = _L()
    assert a.dim() == 3 and b.dim() == 3 and a.dtype == b.dtype
    B, M, K = a.shape
    _, _, N = b.shape
    if not (a.stride(2) == 1 or a.stride(1) == 1):
        a = a.contiguous()
    if not (b.stride(2) == 1 or b.stride(1) == 1):
        b = b.contiguous()
    a_mn = 0 if a.stride(2) == 1 else 1
    lda = a.stride(1) if a_mn == 0 else a.stride(2)
    b_mn = 1 if b.stride(2) == 1 else 0
    ldb = b.stride(1) if b_mn == 1 else b.stride(2)
    out = torch.empty((B, M, N), dtype=a.dtype, device=a.device)
    rc = L.rb_bmm_simt(dtype_code(a.dtype), a_mn, b_mn, ptr(a), max(lda, 1), a.stride(0), ptr(b),
                       max(ldb, 1), b.stride(0), B, M, N, K, ptr(out), N, M * N, 0, float(alpha),
                       stream_ptr())
    check(rc, "rb_bmm_simt")
    count_launch()
    return out


# ----------------------------------------------------------------------------
# norms
# ----------------------------------------------------------------------------
def norm_fwd(x, gamma, beta, eps, rms: bool, residual=None):
    L = _L()
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    rows = x2.shape[0]
    r2 = None
    h = None
    if residual is not None:
        r2 = residual.reshape(-1, D)
        if not r2.is_contiguous():
            r2 = r2.contiguous()
        h = torch.empty_like(x2)
    y = torch.empty_like(x2)
    stats = torch.empty((rows, 2), dtype=torch.float32, device=x.device)
    rc = L.rb_norm_fwd(dtype_code(x.dtype), 1 if rms else 0, ptr(x2), ptr(r2), ptr(gamma), ptr(beta),
                       ptr(y), ptr(h), ptr(stats), rows, D, float(eps), stream_ptr())
    check(rc, "rb_norm_fwd")
    count_launch()
    return y.view(x.shape), (h.view(x.shape) if h is not None else None), stats


def norm_bwd(xn, dy, gamma, stats, rms: bool, dres=None, want_beta=True):
    """xn: the tensor that was normalised (x, or x+residual)."""
    L = _L()
    D = xn.shape[-1]
    x2 = xn.reshape(-1, D)
    dy2 = dy.reshape(-1, D)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    rows = x2.shape[0]
    dr2 = None
    if dres is not None:
        dr2 = dres.reshape(-1, D)
        if not dr2.is_contiguous():
            dr2 = dr2.contiguous()
    dx = torch.empty_like(x2)
    dgamma = torch.empty_like(gamma)
    dbeta = torch.empty_like(gamma) if (want_beta and not rms) else None
    nparts = L.rb_norm_bwd_partials(rows)
    scratch = torch.empty((nparts, 2, D), dtype=torch.float32, device=xn.device)
    rc = L.rb_norm_bwd(dtype_code(xn.dtype), 1 if rms else 0, ptr(x2), ptr(dy2), ptr(gamma),
                       ptr(stats), ptr(dr2), ptr(dx), ptr(dgamma), ptr(dbeta), ptr(scratch), rows, D,
                       stream_ptr())
    check(rc, "rb_norm_bwd")
    count_launch(2)
    return dx.view(xn.shape), dgamma, dbeta


# ----------------------------------------------------------------------------
# softmax / cross entropy
# ----------------------------------------------------------------------------
def softmax_fwd(x):
    L = _L()
    n = x.shape[-1]
    x2 = x.reshape(-1, n).contiguous()
    y = torch.empty_like(x2)
    check(L.rb_softmax_fwd(dtype_code(x.dtype), ptr(x2), ptr(y), x2.shape[0], n, stream_ptr()),
          "rb_softmax_fwd")
    count_launch()
    return y.view(x.shape)


def softmax_bwd(y, dy):
    L = _L()
    n = y.shape[-1]
    y2 = y.reshape(-1, n).contiguous()
    d2 = dy.reshape(-1, n).contiguous()
    dx = torch.empty_like(y2)
    check(L.rb_softmax_bwd(dtype_code(y.dtype), ptr(y2), ptr(d2), ptr(dx), y2.shape[0], n,
                           stream_ptr()), "rb_softmax_bwd")
    count_launch()
    return dx.view(y.shape)


def cross_entropy(logits, targets, grad_scale: float, loss_scale: float, want_grad: bool,
                  inplace: bool = False):
    """Returns (loss scalar fp32 tensor, dlogits or None)."""
    L = _L()
    assert logits.dim() == 2 and logits.stride(1) == 1
    rows, n = logits.shape
    ld = logits.stride(0) if rows > 1 else n
    targets = targets.to(torch.int64).contiguous()
    loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss = torch.empty((), dtype=torch.float32, device=logits.device)
    d = None
    if want_grad:
        d = logits if inplace else torch.empty_strided(logits.shape, logits.stride(),
                                                       dtype=logits.dtype, device=logits.device)
    check(L.rb_cross_entropy(dtype_code(logits.dtype), ptr(logits), ptr(targets), ptr(loss_rows),
                             ptr(loss), ptr(d), rows, n, ld, float(grad_scale), float(loss_scale),
                             stream_ptr()), "rb_cross_entropy")
    count_launch(2)
    return loss, d


# ----------------------------------------------------------------------------
# pointwise
# ----------------------------------------------------------------------------
def unary(x, op: str, a: float = 0.0):
    L = _L()
    xc = x.contiguous()
    y = torch.empty_like(xc)
    check(L.rb_unary(dtype_code(x.dtype), ptr(xc), ptr(y), xc.numel(), UN_CODES[op], float(a),
                     stream_ptr()), "rb_unary")
    count_launch()
    return y


def unary_bwd(x, dy, op: str, a: float = 0.0):
    L = _L()
    xc, dc = x.contiguous(), dy.contiguous()
    dx = torch.empty_like(xc)
    check(L.rb_unary_bwd(dtype_code(x.dtype), ptr(xc), ptr(dc), ptr(dx), xc.numel(), UN_CODES[op],
                         float(a), stream_ptr()), "rb_unary_bwd")
    count_launch()
    return dx


def binary(a, b, op: str, alpha: float = 1.0):
    L = _L()
    assert a.shape == b.shape and a.dtype == b.dtype
    ac, bc = a.contiguous(), b.contiguous()
    y = torch.empty_like(ac)
    check(L.rb_binary(dtype_code(a.dtype), ptr(ac), ptr(bc), ptr(y), ac.numel(), BIN_CODES[op],
                      float(alpha), stream_ptr()), "rb_binary")
    count_launch()
    return y


def cast(x, dtype: torch.dtype, scale: float = 1.0, out=None):
    L = _L()
    xc = x.contiguous()
    y = out if out is not None else torch.empty(xc.shape, dtype=dtype, device=x.device)
    check(L.rb_cast(dtype_code(x.dtype), dtype_code(dtype), ptr(xc), ptr(y), xc.numel(), float(scale),
                    stream_ptr()), "rb_cast")
    count_launch()
    return y


def swiglu_fwd(gu):
    L = _L()
    F2 = gu.shape[-1]
    g2 = gu.reshape(-1, F2)
    assert g2.stride(1) == 1
    rows = g2.shape[0]
    y = torch.empty((rows, F2 // 2), dtype=gu.dtype, device=gu.device)
    check(L.rb_swiglu_fwd(dtype_code(gu.dtype), ptr(g2), ptr(y), rows, F2 // 2,
                          g2.stride(0) if rows > 1 else F2, stream_ptr()), "rb_swiglu_fwd")
    count_launch()
    return y.view(*gu.shape[:-1], F2 // 2)


def swiglu_bwd(gu, dy):
    L = _L()
    F2 = gu.shape[-1]
    g2 = gu.reshape(-1, F2).contiguous()
    d2 = dy.reshape(-1, F2 // 2).contiguous()
    dgu = torch.empty_like(g2)
    check(L.rb_swiglu_bwd(dtype_code(gu.dtype), ptr(g2), ptr(d2), ptr(dgu), g2.shape[0], F2 // 2, F2,
                          stream_ptr()), "rb_swiglu_bwd")
    count_launch()
    return dgu.view(gu.shape)


def dropout(x, p: float, seed: int):
    L = _L()
    xc = x.contiguous()
    y = torch.empty_like(xc)
    check(L.rb_dropout(dtype_code(x.dtype), ptr(xc), ptr(y), xc.numel(), seed & 0xFFFFFFFF, float(p),
                       stream_ptr()), "rb_dropout")
    count_launch()
    return y


def embedding_fwd(idx, weight, pos=None, seq_len: int = 1):
    L = _L()
    idx = idx.to(torch.int64).contiguous()
    tokens = idx.numel()
    vocab, D = weight.shape
    out = torch.empty((*idx.shape, D), dtype=weight.dtype, device=weight.device)
    check(L.rb_embedding_fwd(dtype_code(weight.dtype), ptr(idx), ptr(weight), ptr(pos), ptr(out),
                             tokens, D, seq_len, vocab, stream_ptr()), "rb_embedding_fwd")
    count_launch()
    return out


def embedding_bwd(idx, dout, vocab: int, seq_len: int = 1, want_pos: bool = False):
    L = _L()
    idx = idx.to(torch.int64).contiguous()
    D = dout.shape[-1]
    d2 = dout.reshape(-1, D).contiguous()
    dW = torch.zeros((vocab, D), dtype=torch.float32, device=dout.device)
    dpos = torch.zeros((seq_len, D), dtype=torch.float32, device=dout.device) if want_pos else None
    check(L.rb_embedding_bwd(dtype_code(dout.dtype), ptr(idx), ptr(d2), ptr(dW), ptr(dpos),
                             idx.numel(), D, seq_len, vocab, stream_ptr()), "rb_embedding_bwd")
    count_launch()
    return dW, dpos


def rope_(x2d, tokens: int, seq_len: int, heads: int, head_dim: int, col0: int, theta: float,
          backward: bool, pos_ids=None):
    """In-place rotary embedding on columns [col0, col0 + heads*head_dim) of a [tokens, ld] buffer."""
    L = _L()
    assert x2d.dim() == 2 and x2d.stride(1) == 1
    check(L.rb_rope(dtype_code(x2d.dtype), ptr(x2d), ptr(pos_ids), tokens, seq_len, heads, head_dim,
                    x2d.stride(0), col0, float(theta), 1 if backward else 0, stream_ptr()), "rb_rope")
    count_launch()
    return x2d


def colsum(x2d):
    """Column sums of a [rows, N] matrix (bias gradient)."""
    L = _L()
    assert x2d.dim() == 2 and x2d.stride(1) == 1
    rows, N = x2d.shape
    slabs = L.rb_colsum_slabs(rows)
    scratch = torch.empty((slabs, N), dtype=torch.float32, device=x2d.device)
    out = torch.empty(N, dtype=x2d.dtype, device=x2d.device)
    check(L.rb_colsum(dtype_code(x2d.dtype), ptr(x2d), ptr(out), ptr(scratch), rows, N,
                      x2d.stride(0) if rows > 1 else N, stream_ptr()), "rb_colsum")
    count_launch(2)
    return out


# ----------------------------------------------------------------------------
# optimizers
# ----------------------------------------------------------------------------
class _TensorList(ctypes.Structure):
    _fields_ = [("count", c_int), ("grad", ctypes.POINTER(c_void_p)),
                ("master", ctypes.POINTER(c_void_p)), ("m", ctypes.POINTER(c_void_p)),
                ("v", ctypes.POINTER(c_void_p)), ("model", ctypes.POINTER(c_void_p)),
                ("numel", ctypes.POINTER(c_longlong))]


def _mk_list(grads, masters, ms, vs, models):
    n = len(grads)
    Arr = c_void_p * n

    def arr(ts):
        if ts is None:
            return None
        return Arr(*[(t.data_ptr() if t is not None else 0) for t in ts])

    keep = [arr(grads), arr(masters), arr(ms), arr(vs), arr(models),
            (c_longlong * n)(*[g.numel() for g in grads])]
    tl = _TensorList()
    tl.count = n
    tl.grad = ctypes.cast(keep[0], ctypes.POINTER(c_void_p))
    tl.master = ctypes.cast(keep[1], ctypes.POINTER(c_void_p))
    tl.m = ctypes.cast(keep[2], ctypes.POINTER(c_void_p)) if keep[2] is not None else None
    tl.v = ctypes.cast(keep[3], ctypes.POINTER(c_void_p)) if keep[3] is not None else None
    tl.model = ctypes.cast(keep[4], ctypes.POINTER(c_void_p)) if keep[4] is not None else None
    tl.numel = ctypes.cast(keep[5], ctypes.POINTER(c_longlong))
    return tl, keep


def multi_tensor_adam(grads, masters, ms, vs, models, *, lr, beta1, beta2, eps, weight_decay, step,
                      adamw, grad_scale=None, skip=None, step_tensor=None):
    L = _L()
    tl, keep = _mk_list(grads, masters, ms, vs, models)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    rc = L.rb_multi_tensor_adam(ctypes.addressof(tl), dtype_code(grads[0].dtype), lr, beta1, beta2,
                                eps, weight_decay, bc1, bc2, 1 if adamw else 0, ptr(grad_scale),
                                ptr(skip), ptr(step_tensor), stream_ptr())
    if rc < 0:
        check(-rc, "rb_multi_tensor_adam")
    count_launch(rc)


def multi_tensor_sgd(grads, masters, moms, models, *, lr, momentum, weight_decay, grad_scale=None,
                     skip=None):
    L = _L()
    tl, keep = _mk_list(grads, masters, moms, None, models)
    rc = L.rb_multi_tensor_sgd(ctypes.addressof(tl), dtype_code(grads[0].dtype), lr, momentum,
                               weight_decay, ptr(grad_scale), ptr(skip), stream_ptr())
    if rc < 0:
        check(-rc, "rb_multi_tensor_sgd")
    count_launch(rc)


def adam_flat(grad, master, m, v, model, *, lr, beta1, beta2, eps, weight_decay, step, adamw,
              grad_scale=None, skip=None, step_tensor=None):
    L = _L()
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    check(L.rb_adam_flat(dtype_code(grad.dtype), ptr(grad), ptr(master), ptr(m), ptr(v), ptr(model),
                         grad.numel(), lr, beta1, beta2, eps, weight_decay, bc1, bc2,
                         1 if adamw else 0, ptr(grad_scale), ptr(skip), ptr(step_tensor),
                         stream_ptr()), "rb_adam_flat")
    count_launch()


def global_norm(tensors, max_norm: float = 0.0, extra_scale: float = 1.0, found_inf=None):
    """Two-stage L2 norm over a list of tensors.  Returns (norm, clip_coef) device scalars."""
    L = _L()
    dev = tensors[0].device
    per = 64
    partials = torch.zeros(per * len(tensors), dtype=torch.float32, device=dev)
    off = 0
    for t in tensors:
        tc = t if t.is_contiguous() else t.contiguous()
        n = L.rb_sumsq_partials(dtype_code(tc.dtype), ptr(tc), tc.numel(),
                                c_void_p(partials.data_ptr() + 4 * off), per, ptr(found_inf),
                                stream_ptr())
        if n < 0:
            check(-n, "rb_sumsq_partials")
        off += per
        count_launch()
    norm = torch.empty((), dtype=torch.float32, device=dev)
    coef = torch.empty((), dtype=torch.float32, device=dev)
    check(L.rb_norm_finalize(ptr(partials), off, float(max_norm), float(extra_scale), ptr(norm),
                             ptr(coef), stream_ptr()), "rb_norm_finalize")
    count_launch()
    return norm, coef


def scale_check_(x, scale_tensor=None, scale: float = 1.0, found_inf=None):
    L = _L()
    assert x.is_contiguous()
    check(L.rb_scale_check(dtype_code(x.dtype), ptr(x), x.numel(), ptr(scale_tensor), float(scale),
                           ptr(found_inf), stream_ptr()), "rb_scale_check")
    count_launch()
    return x
