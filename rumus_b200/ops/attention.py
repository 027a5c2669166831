"""FlashAttention autograd wrapper over the tcgen05 forward / backward kernels."""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import native
from ._lib import check, count_launch, ptr, stream_ptr

P, LL, I, F = c_void_p, c_longlong, c_int, c_float
native.register_signature("rb_flash_attn_fwd", [I, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P])
native.register_signature("rb_flash_attn_bwd", [I, I, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P,
                                                I, I, I, I, I, I, F, P])
native.register_signature("rb_fa_dq_cast", [I, P, P, P, I, I, I, P])


def _strides3(t: torch.Tensor):
    """{batch, seq, head} strides (elements) of a [B, S, H, D] view whose last dim is dense."""
    assert t.dim() == 4 and t.stride(3) == 1
    arr = (c_longlong * 3)(t.stride(0), t.stride(1), t.stride(2))
    return arr


def _tma_ok(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0
            and all((t.stride(i) * t.element_size()) % 16 == 0 for i in range(3)))


def fa_forward(q, k, v, causal: bool, scale: float):
    L = native.lib()
    B, Sq, H, D = q.shape
    _, Sk, Hkv, _ = k.shape
    q, k, v = (t if _tma_ok(t) else t.contiguous() for t in (q, k, v))
    o = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    qs, ks, vs = _strides3(q), _strides3(k), _strides3(v)
    rc = L.rb_flash_attn_fwd(native.dtype_code(q.dtype), D, ptr(q), ptr(k), ptr(v),
                             ctypes.addressof(qs), ctypes.addressof(ks), ctypes.addressof(vs),
                             ptr(o), ptr(lse), B, H, Hkv, Sq, Sk, 1 if causal else 0, float(scale),
                             stream_ptr())
    check(rc, "rb_flash_attn_fwd")
    count_launch()
    return o, lse, (q, k, v)


def fa_backward(q, k, v, o, lse, dout, causal: bool, scale: float, out=None):
    """dq, dk, dv.  ``out`` may give three preallocated [B,S,heads,128] views (e.g. slices of one
    packed d_qkv buffer): the kernels write straight into them."""
    L = native.lib()
    B, Sq, H, D = q.shape
    _, Sk, Hkv, _ = k.shape
    if not _tma_ok(dout):
        dout = dout.contiguous()
    dq32 = torch.empty((B, Sq, H, D), dtype=torch.float32, device=q.device)   # zeroed by the delta kernel
    if out is None:
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Sk, Hkv, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Sk, Hkv, D), dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = out
    assert dk.stride() == dv.stride() and dk.stride(3) == 1 and dq.stride(3) == 1
    sq_pad = (Sq + 63) // 64 * 64
    stats = torch.zeros((2, B, H, sq_pad), dtype=torch.float32, device=q.device)  # delta | lse*log2e
    qs, ks, vs, dos = _strides3(q), _strides3(k), _strides3(v), _strides3(dout)
    dkvs, dqs = _strides3(dk), _strides3(dq)
    rc = L.rb_flash_attn_bwd(native.dtype_code(q.dtype), D, ptr(q), ptr(k), ptr(v), ptr(o),
                             ptr(dout), ptr(lse), ctypes.addressof(qs), ctypes.addressof(ks),
                             ctypes.addressof(vs), ctypes.addressof(dos), ptr(stats), ptr(dq32),
                             ptr(dk), ptr(dv), ctypes.addressof(dkvs), B, H, Hkv, Sq, Sk,
                             1 if causal else 0, float(scale), stream_ptr())
    check(rc, "rb_flash_attn_bwd")
    rc = L.rb_fa_dq_cast(native.dtype_code(q.dtype), ptr(dq32), ptr(dq), ctypes.addressof(dqs),
                         B, Sq, H, stream_ptr())
    check(rc, "rb_fa_dq_cast")
    count_launch(3)
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse, (qc, kc, vc) = fa_forward(q, k, v, causal, scale)
        ctx.causal, ctx.scale = causal, scale
        ctx.save_for_backward(qc, kc, vc, o, lse)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        if q.shape[-1] == 128:
            dq, dk, dv = fa_backward(q, k, v, o, lse, dout, ctx.causal, ctx.scale)
        else:
            dq, dk, dv = _composed_backward(q, k, v, dout, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


class _FlashAttnPackedFn(torch.autograd.Function):
    """Attention on the packed projection output ``qkv [B, S, (H + 2*Hkv) * 128]``: the backward
    kernels write d_q, d_k, d_v into the three slices of one d_qkv buffer (no concatenation)."""

    @staticmethod
    def forward(ctx, qkv, heads, kv_heads, causal, scale):
        B, S, _ = qkv.shape
        hd = 128
        q, k, v = qkv.split([heads * hd, kv_heads * hd, kv_heads * hd], dim=-1)
        q, k, v = q.view(B, S, heads, hd), k.view(B, S, kv_heads, hd), v.view(B, S, kv_heads, hd)
        o, lse, _ = fa_forward(q, k, v, causal, scale)
        ctx.causal, ctx.scale, ctx.heads, ctx.kv_heads = causal, scale, heads, kv_heads
        ctx.save_for_backward(qkv, o, lse)
        return o

    @staticmethod
    def backward(ctx, dout):
        qkv, o, lse = ctx.saved_tensors
        B, S, _ = qkv.shape
        H, Hkv, hd = ctx.heads, ctx.kv_heads, 128
        sizes = [H * hd, Hkv * hd, Hkv * hd]
        q, k, v = qkv.split(sizes, dim=-1)
        q, k, v = q.view(B, S, H, hd), k.view(B, S, Hkv, hd), v.view(B, S, Hkv, hd)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv.split(sizes, dim=-1)
        out = (dq.view(B, S, H, hd), dk.view(B, S, Hkv, hd), dv.view(B, S, Hkv, hd))
        fa_backward(q, k, v, o, lse, dout, ctx.causal, ctx.scale, out=out)
        return dqkv, None, None, None, None


def flash_attention_packed(qkv, heads: int, kv_heads: int, causal: bool = True,
                           scale: Optional[float] = None):
    """``qkv`` is the fused projection output, head_dim 128, CUDA, 16-bit, 16-byte aligned rows."""
    if scale is None:
        scale = 1.0 / math.sqrt(128)
    return _FlashAttnPackedFn.apply(qkv, heads, kv_heads, causal, scale)


def _composed_backward(q, k, v, dout, causal, scale):
    """head_dim != 128: gradient through the batched-matmul + softmax kernels in fp32."""
    from . import functional as F
    with torch.enable_grad():
        qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
        if kf.shape[2] != qf.shape[2]:
            rep = qf.shape[2] // kf.shape[2]
            ke, ve = kf.repeat_interleave(rep, dim=2), vf.repeat_interleave(rep, dim=2)
        else:
            ke, ve = kf, vf
        o = F._sdpa_composed(qf, ke, ve, causal, scale)
        gq, gk, gv = torch.autograd.grad(o, (qf, kf, vf), dout.float())
    return gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype)


def flash_attention_cuda(q, k, v, causal: bool = True, scale: Optional[float] = None):
    """q: [B, Sq, H, D], k/v: [B, Sk, Hkv, D] (bf16/fp16, D in {64, 128}); returns [B, Sq, H, D]."""
    D = q.shape[-1]
    if D not in (64, 128):
        from . import functional as F
        return F._sdpa_composed(q.float(), k.float(), v.float(), causal, scale).to(q.dtype)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    return _FlashAttnFn.apply(q, k, v, causal, scale)
