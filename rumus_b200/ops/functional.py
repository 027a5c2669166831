"""Differentiable ops.

CUDA tensors run the hand-written sm_100a kernels through ``native`` (and raise
if the library is missing); CPU tensors use plain PyTorch math, which is also
the fp32 reference the GPU tests compare against.

Op surface mirrors the reference's tensor ops (rumus/src/tensor/ops.rs:404-2743):
matmul/bmm, add_bias, relu/sigmoid/tanh/gelu/leaky_relu, softmax, layer_norm,
embedding, cross_entropy_loss, mse_loss, dropout, flash_attention — plus the ops
the benchmark configs need that the reference lacks (rms_norm, rope, swiglu,
fused linear epilogues, fused MLP).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as TF

from . import native

_ACT_TORCH = {
    None: lambda x: x,
    "none": lambda x: x,
    "relu": torch.relu,
    "gelu": lambda x: TF.gelu(x, approximate="tanh"),
    "silu": TF.silu,
}


def _acc(t: torch.Tensor) -> torch.Tensor:
    """Accumulation dtype of the plain-math paths: fp32, except that fp64 inputs stay fp64 (so the
    formulas can be checked by finite differences)."""
    return t if t.dtype == torch.float64 else t.float()


def _is_native(t: torch.Tensor) -> bool:
    return t.is_cuda


# ----------------------------------------------------------------------------
# matmul / linear
# ----------------------------------------------------------------------------
class _MatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return native.gemm(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        da = native.gemm(dy, b.t()) if ctx.needs_input_grad[0] else None
        db = native.gemm(a.t(), dy) if ctx.needs_input_grad[1] else None
        return da, db


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """2-D matmul (reference: tensor/ops.rs:516)."""
    if not _is_native(a):
        return a @ b
    return _MatmulFn.apply(a, b)


class _BmmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return native.bmm(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        dy = dy.contiguous()
        return native.bmm(dy, b.transpose(1, 2)), native.bmm(a.transpose(1, 2), dy)


def bmm(a, b):
    """Batched matmul [B,M,K]@[B,K,N] (reference: tensor/ops.rs:1490)."""
    if not _is_native(a):
        return torch.bmm(a, b)
    return _BmmFn.apply(a, b)


def _main_grad(p):
    """Parameters managed by a flat gradient arena carry ``main_grad`` (a view into the arena)
    and ``grad_accumulate`` (add instead of overwrite).  Weight-gradient GEMMs then write
    straight into the arena and autograd sees ``None`` for that parameter."""
    if p is None:
        return None
    mg = getattr(p, "main_grad", None)
    if mg is None:
        return None
    return (mg, p)


def _wgrad(x2, dy2, mg):
    if mg is None:
        return native.gemm(x2.t(), dy2)
    buf, p = mg
    acc = getattr(p, "grad_accumulate", False)
    native.gemm(x2.t(), dy2, out=buf, residual=buf if acc else None)
    p.grad_accumulate = True
    return None


def _bgrad(dy2, mg):
    g = native.colsum(dy2)
    if mg is None:
        return g
    buf, p = mg
    if getattr(p, "grad_accumulate", False):
        buf.add_(g)
    else:
        buf.copy_(g)
    p.grad_accumulate = True
    return None


def _small_grad(g, mg):
    """Route a small parameter gradient (norm scale/shift, embeddings) into the arena."""
    if mg is None or g is None:
        return g
    buf, p = mg
    if getattr(p, "grad_accumulate", False):
        buf.add_(g.view(buf.shape))
    else:
        buf.copy_(g.view(buf.shape))
    p.grad_accumulate = True
    return None


class _LinearFn(torch.autograd.Function):
    """y = act(x @ W + b) (+ residual); W is [in, out]."""

    @staticmethod
    def forward(ctx, x, w, bias, residual, act):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, w.shape[1]) if residual is not None else None
        need_pre = act not in (None, "none") and (x.requires_grad or w.requires_grad)
        if need_pre:
            y, pre = native.gemm(x2, w, bias=bias, act=act, residual=res2, aux_out=True)
        else:
            y, pre = native.gemm(x2, w, bias=bias, act=act, residual=res2), None
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        ctx.w_main_grad = _main_grad(w)
        ctx.b_main_grad = _main_grad(bias)
        ctx.save_for_backward(x2, w, pre)
        return y.view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        if pre is not None:
            dy2 = native.unary_bwd(pre, dy2, ctx.act)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = native.gemm(dy2, w.t()).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(x2, dy2, ctx.w_main_grad)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _bgrad(dy2, ctx.b_main_grad)
        return dx, dw, db, dres, None


def linear(x: torch.Tensor, weight_io: torch.Tensor, bias: Optional[torch.Tensor] = None,
           act: Optional[str] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(x @ weight_io + bias) + residual`` with ``weight_io`` stored ``[in, out]``
    (reference Linear: rumus/src/nn/linear.rs:44-100; bias/activation are GEMM epilogues here)."""
    if not _is_native(x):
        y = x @ weight_io
        if bias is not None:
            y = y + bias
        y = _ACT_TORCH[act](y)
        if residual is not None:
            y = y + residual
        return y
    return _LinearFn.apply(x, weight_io, bias, residual, act)


class _MlpFn(torch.autograd.Function):
    """y = act(x W1 + b1) W2 + b2 (+ residual) with the activation derivative fused into the
    epilogue of the second layer's data-gradient GEMM."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, act):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        a, h = native.gemm(x2, w1, bias=b1, act=act, aux_out=True)
        res2 = residual.reshape(-1, w2.shape[1]) if residual is not None else None
        y = native.gemm(a, w2, bias=b2, residual=res2)
        ctx.act = act
        ctx.has_res = residual is not None
        ctx.has_b1 = b1 is not None
        ctx.has_b2 = b2 is not None
        ctx.x_shape = x.shape
        ctx.mg = (_main_grad(w1), _main_grad(b1), _main_grad(w2), _main_grad(b2))
        ctx.save_for_backward(x2, w1, w2, h, a)
        return y.view(*x.shape[:-1], w2.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, h, a = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        mg_w1, mg_b1, mg_w2, mg_b2 = ctx.mg
        dh = native.gemm(dy2, w2.t(), aux_in=h, dact=ctx.act)
        dw2 = _wgrad(a, dy2, mg_w2)
        db2 = _bgrad(dy2, mg_b2) if ctx.has_b2 else None
        dx = native.gemm(dh, w1.t()).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw1 = _wgrad(x2, dh, mg_w1)
        db1 = _bgrad(dh, mg_b1) if ctx.has_b1 else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None), None


def mlp(x, w1, b1, w2, b2, act: str = "gelu", residual=None):
    """Two-layer MLP block (reference TransformerBlock MLP: rumus/src/nn/transformer.rs:51-57)."""
    if not _is_native(x):
        h = _ACT_TORCH[act](x @ w1 + (b1 if b1 is not None else 0))
        y = h @ w2
        if b2 is not None:
            y = y + b2
        if residual is not None:
            y = y + residual
        return y
    return _MlpFn.apply(x, w1, b1, w2, b2, residual, act)


def add_bias(x, bias):
    """reference: tensor/ops.rs:885"""
    return x + bias


# ----------------------------------------------------------------------------
# activations
# ----------------------------------------------------------------------------
class _UnaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, a):
        ctx.op, ctx.a = op, a
        ctx.save_for_backward(x)
        return native.unary(x, op, a).view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return native.unary_bwd(x, dy, ctx.op, ctx.a).view(x.shape), None, None


def _unary(x, op, torch_fn, a=0.0):
    if not _is_native(x):
        return torch_fn(x)
    return _UnaryFn.apply(x, op, a)


def relu(x):
    return _unary(x, "relu", torch.relu)


def gelu(x):
    """tanh approximation, as the reference (backend/cpu.rs gelu)."""
    return _unary(x, "gelu", lambda t: TF.gelu(t, approximate="tanh"))


def silu(x):
    return _unary(x, "silu", TF.silu)


def sigmoid(x):
    return _unary(x, "sigmoid", torch.sigmoid)


def tanh(x):
    return _unary(x, "tanh", torch.tanh)


def leaky_relu(x, negative_slope: float = 0.01):
    return _unary(x, "leaky_relu", lambda t: TF.leaky_relu(t, negative_slope), negative_slope)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return native.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        return native.swiglu_bwd(gu, dy)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on a fused ``[..., 2F]`` buffer laid out gate | up."""
    if not _is_native(gate_up):
        g, u = gate_up.chunk(2, dim=-1)
        return TF.silu(g) * u
    return _SwigluFn.apply(gate_up)


# ----------------------------------------------------------------------------
# normalisation
# ----------------------------------------------------------------------------
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, eps, rms):
        y, h, stats = native.norm_fwd(x, gamma, beta, eps, rms, residual)
        ctx.rms = rms
        ctx.has_res = residual is not None
        ctx.has_beta = beta is not None
        ctx.mg = (_main_grad(gamma), _main_grad(beta))
        ctx.save_for_backward(h if h is not None else x, gamma, stats)
        return y, h

    @staticmethod
    def backward(ctx, dy, dh):
        xn, gamma, stats = ctx.saved_tensors
        dx, dg, db = native.norm_bwd(xn, dy, gamma, stats, ctx.rms, dres=dh,
                                     want_beta=ctx.has_beta)
        dg = _small_grad(dg, ctx.mg[0])
        db = _small_grad(db, ctx.mg[1]) if ctx.has_beta else None
        return dx, dg, db, (dx if ctx.has_res else None), None, None


class _NormSkipFn(torch.autograd.Function):
    """``(norm(x), x)``: the second output is ``x`` itself, handed on as the residual stream.  Taking
    the skip connection from here instead of from ``x`` directly means ``x`` has ONE consumer in the
    autograd graph, so the two gradients that meet at a pre-norm block's input (through the norm and
    through the skip) are added inside the norm-backward kernel instead of by a separate add."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, rms):
        y, _, stats = native.norm_fwd(x, gamma, beta, eps, rms, None)
        ctx.rms = rms
        ctx.has_beta = beta is not None
        ctx.mg = (_main_grad(gamma), _main_grad(beta))
        ctx.save_for_backward(x, gamma, stats)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dskip):
        x, gamma, stats = ctx.saved_tensors
        dx, dg, db = native.norm_bwd(x, dy, gamma, stats, ctx.rms, dres=dskip, want_beta=ctx.has_beta)
        dg = _small_grad(dg, ctx.mg[0])
        db = _small_grad(db, ctx.mg[1]) if ctx.has_beta else None
        return dx, dg, db, None, None


def norm_skip(x, weight, bias=None, eps: float = 1e-5, rms: bool = False):
    """``(norm(x), skip)`` for pre-norm blocks: use ``skip`` (same values as ``x``) as the residual of
    the branch that consumes the norm output.  LayerNorm, or RMSNorm with ``rms=True``."""
    if not _is_native(x):
        if rms:
            return rms_norm(x, weight, eps), x
        return layer_norm(x, weight, bias, eps), x
    return _NormSkipFn.apply(x, weight, None if rms else bias, eps, rms)


def layer_norm(x, weight, bias, eps: float = 1e-5, residual=None):
    """LayerNorm over the last dim (reference: tensor/ops.rs:1727).  With ``residual`` the kernel
    first forms ``h = x + residual`` and returns ``(norm(h), h)``."""
    if not _is_native(x):
        h = x + residual if residual is not None else x
        y = TF.layer_norm(h, (h.shape[-1],), weight, bias, eps)
        return (y, h) if residual is not None else y
    y, h = _NormFn.apply(x, weight, bias, residual, eps, False)
    return (y, h) if residual is not None else y


def rms_norm(x, weight, eps: float = 1e-6, residual=None):
    if not _is_native(x):
        h = x + residual if residual is not None else x
        hf = _acc(h)
        y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).to(h.dtype) * weight
        return (y, h) if residual is not None else y
    y, h = _NormFn.apply(x, weight, None, residual, eps, True)
    return (y, h) if residual is not None else y


# ----------------------------------------------------------------------------
# softmax / losses
# ----------------------------------------------------------------------------
class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = native.softmax_fwd(x)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return native.softmax_bwd(y, dy)


def softmax(x):
    """Softmax over the last dim (reference: tensor/ops.rs:1656)."""
    if not _is_native(x):
        return torch.softmax(x, dim=-1)
    return _SoftmaxFn.apply(x)


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows = logits.shape[0]
        loss, dlogits = native.cross_entropy(logits, targets, grad_scale=1.0 / rows,
                                             loss_scale=1.0 / rows, want_grad=logits.requires_grad)
        ctx.save_for_backward(dlogits)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (dlogits,) = ctx.saved_tensors
        # the gradient was produced with scale 1/rows in forward; fold the upstream scalar in
        return dlogits * dloss.to(dlogits.dtype), None


def cross_entropy_loss(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean next-token cross entropy over rows of ``logits [B, C]`` (reference:
    tensor/ops.rs:788 — gradient precomputed in the forward kernel, as here)."""
    if logits.dim() > 2:
        logits = logits.reshape(-1, logits.shape[-1])
        targets = targets.reshape(-1)
    if not _is_native(logits):
        return TF.cross_entropy(_acc(logits), targets.long())
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    return _CrossEntropyFn.apply(logits, targets)


class _LmHeadLossFn(torch.autograd.Function):
    """Vocabulary projection + mean cross entropy.  The logits buffer is overwritten in place by
    its own gradient inside the cross-entropy kernel, so the [tokens, vocab] matrix exists once."""

    @staticmethod
    def forward(ctx, x, w, targets):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        logits = native.gemm(x2, w)
        loss, dlogits = native.cross_entropy(logits, targets.reshape(-1), grad_scale=1.0 / rows,
                                             loss_scale=1.0 / rows, want_grad=True, inplace=True)
        ctx.x_shape = x.shape
        ctx.mg = _main_grad(w)
        ctx.save_for_backward(x2, w, dlogits)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x2, w, dlogits = ctx.saved_tensors
        dx = native.gemm(dlogits, w.t())
        dx.mul_(dloss.to(dx.dtype))
        if ctx.mg is None:
            dw = native.gemm(x2.t(), dlogits)
            dw.mul_(dloss.to(dw.dtype))
        else:
            # fold the upstream scalar into the (small) activation operand instead of the
            # [d, vocab] result, then accumulate straight into the arena
            dw = _wgrad(x2 * dloss.to(x2.dtype), dlogits, ctx.mg)
        return dx.view(ctx.x_shape), dw, None


def lm_head_loss(x, weight_io, targets):
    """``cross_entropy(x @ weight_io, targets)`` (mean over tokens) without keeping logits and
    their gradient as two tensors."""
    if not _is_native(x):
        logits = x.reshape(-1, x.shape[-1]) @ weight_io
        return TF.cross_entropy(_acc(logits), targets.reshape(-1).long())
    return _LmHeadLossFn.apply(x, weight_io, targets)


def mse_loss(pred, target):
    """reference: tensor/ops.rs:713"""
    return ((pred - target) ** 2).mean()


# ----------------------------------------------------------------------------
# embedding / dropout / rope
# ----------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight, pos):
        seq = idx.shape[-1] if idx.dim() > 1 else idx.numel()
        if pos is not None:
            assert pos.shape[0] >= seq
        out = native.embedding_fwd(idx, weight, pos, seq)
        ctx.save_for_backward(idx)
        ctx.vocab = weight.shape[0]
        ctx.seq = seq
        ctx.pos_rows = pos.shape[0] if pos is not None else 0
        ctx.wdtype = weight.dtype
        ctx.mg = (_main_grad(weight), _main_grad(pos))
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dW, dpos = native.embedding_bwd(idx, dout, ctx.vocab, ctx.seq, want_pos=ctx.pos_rows > 0)
        dW = dW.to(ctx.wdtype)
        if dpos is not None:
            full = torch.zeros((ctx.pos_rows, dpos.shape[1]), dtype=ctx.wdtype, device=dpos.device)
            full[: ctx.seq] = dpos.to(ctx.wdtype)
            dpos = full
        return None, _small_grad(dW, ctx.mg[0]), _small_grad(dpos, ctx.mg[1])


def embedding(idx: torch.Tensor, weight: torch.Tensor, pos: Optional[torch.Tensor] = None):
    """Row gather (reference: tensor/ops.rs:2096) with an optional fused learned
    positional-embedding add: ``out[b, s] = weight[idx[b, s]] + pos[s]``."""
    if not _is_native(weight):
        out = TF.embedding(idx.long(), weight)
        if pos is not None:
            out = out + pos[: idx.shape[-1]]
        return out
    return _EmbeddingFn.apply(idx, weight, pos)


_dropout_step = [0]


class _DropoutFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed):
        ctx.p, ctx.seed = p, seed
        return native.dropout(x, p, seed).view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        # the mask is a pure function of (seed, index): re-apply it to dy
        return native.dropout(dy, ctx.p, ctx.seed).view(dy.shape), None, None


def dropout(x, p: float, training: bool = True, seed: Optional[int] = None):
    """Inverted dropout (reference: tensor/ops.rs:1305; a global step counter seeds each call)."""
    if not training or p <= 0.0:
        return x
    if not _is_native(x):
        return TF.dropout(x, p, True)
    if seed is None:
        _dropout_step[0] += 1
        seed = (0x9E3779B9 * _dropout_step[0]) & 0xFFFFFFFF
    return _DropoutFn.apply(x, p, seed)


def _rope_torch(x, seq_len, theta, inverse=False):
    # x: [B, S, H, hd]
    B, S, H, hd = x.shape
    half = hd // 2
    inv = theta ** (-2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / hd)
    ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None] * inv[None]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    if inverse:
        sn = -sn
    a, b = _acc(x[..., :half]), _acc(x[..., half:])
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)


class _RopeQKVFn(torch.autograd.Function):
    """In-place rotary embedding of the q and k column blocks of a fused qkv buffer."""

    @staticmethod
    def forward(ctx, qkv, seq_len, heads, kv_heads, head_dim, theta):
        tokens = qkv.numel() // qkv.shape[-1]
        q2 = qkv.view(tokens, qkv.shape[-1])
        native.rope_(q2, tokens, seq_len, heads, head_dim, 0, theta, False)
        native.rope_(q2, tokens, seq_len, kv_heads, head_dim, heads * head_dim, theta, False)
        ctx.args = (seq_len, heads, kv_heads, head_dim, theta)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, d):
        seq_len, heads, kv_heads, head_dim, theta = ctx.args
        d = d.contiguous()
        tokens = d.numel() // d.shape[-1]
        d2 = d.view(tokens, d.shape[-1])
        native.rope_(d2, tokens, seq_len, heads, head_dim, 0, theta, True)
        native.rope_(d2, tokens, seq_len, kv_heads, head_dim, heads * head_dim, theta, True)
        return d, None, None, None, None, None


def rope_qkv(qkv: torch.Tensor, seq_len: int, heads: int, kv_heads: int, head_dim: int,
             theta: float = 10000.0) -> torch.Tensor:
    """Rotary position embedding on q and k of a fused ``[B, S, (H + 2*Hkv) * hd]`` projection
    (half-split pairing ``(i, i + hd/2)``)."""
    if not _is_native(qkv):
        B, S, _ = qkv.shape
        q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=-1)
        q = _rope_torch(q.view(B, S, heads, head_dim), S, theta).reshape(B, S, -1)
        k = _rope_torch(k.view(B, S, kv_heads, head_dim), S, theta).reshape(B, S, -1)
        return torch.cat([q, k, v], dim=-1)
    # work on a private buffer: autograd forbids in-place edits of a tensor other ops saved
    return _RopeQKVFn.apply(qkv.clone() if qkv.requires_grad and qkv.is_leaf else qkv, seq_len,
                            heads, kv_heads, head_dim, theta)


# ----------------------------------------------------------------------------
# attention
# ----------------------------------------------------------------------------
def sdpa_reference(q, k, v, causal: bool, scale: Optional[float] = None):
    """Plain-math attention on [B, S, H, d] tensors (softmax in fp32; fp64 inputs stay fp64)."""
    B, S, H, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    acc = torch.float64 if q.dtype == torch.float64 else torch.float32
    qf, kf, vf = (t.permute(0, 2, 1, 3).to(acc) for t in (q, k, v))
    if kf.shape[1] != H:
        rep = H // kf.shape[1]
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        Sk = kf.shape[2]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(diagonal=Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def flash_attention_packed(qkv, heads: int, kv_heads: int, causal: bool = True,
                           scale: Optional[float] = None):
    """Attention over the fused projection output ``[B, S, (heads + 2*kv_heads) * 128]`` (CUDA,
    16-bit): same result as splitting and calling ``flash_attention``, without the gradient
    concatenation."""
    from .attention import flash_attention_packed as _packed
    return _packed(qkv, heads, kv_heads, causal, scale)


def flash_attention(q, k, v, causal: bool = True, scale: Optional[float] = None):
    """Memory-efficient attention on ``[B, S, H, d]`` tensors (strided views of a fused qkv
    projection are fine).  Reference: tensor/ops.rs:2685 (forward-only there; it falls back to
    materialised SDPA when gradients are needed — here forward and backward are both fused)."""
    if _is_native(q) and q.dtype in (torch.bfloat16, torch.float16):
        from .attention import flash_attention_cuda
        return flash_attention_cuda(q, k, v, causal, scale)
    if _is_native(q):
        return _sdpa_composed(q, k, v, causal, scale)
    return sdpa_reference(q, k, v, causal, scale)


def _sdpa_composed(q, k, v, causal, scale):
    """fp32 CUDA tensors: batched matmul + softmax kernels (the reference's composition,
    rumus/src/nn/attention.rs:17-58)."""
    B, S, H, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qh = q.permute(0, 2, 1, 3).reshape(B * H, S, d)
    kh = k.permute(0, 2, 1, 3).reshape(B * H, -1, d)
    vh = v.permute(0, 2, 1, 3).reshape(B * H, -1, d)
    s = bmm(qh, kh.transpose(1, 2)) * scale
    if causal:
        Sk = kh.shape[1]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(diagonal=Sk - S)
        s = s.masked_fill(~mask, -1e9)
    p = softmax(s)
    o = bmm(p, vh)
    return o.view(B, H, S, d).permute(0, 2, 1, 3)


# ---------------------------------------------------------------------------------------------
# Reference op names that are plain tensor-layer operations here
# ---------------------------------------------------------------------------------------------
# The reference implements views, pointwise arithmetic, slicing and concatenation itself
# (rumus/src/tensor/ops.rs); here the tensor layer is PyTorch, so these are its own
# (differentiable, broadcasting, strided) operations under the reference's names, kept so that code
# written against the reference's op list finds every entry.

def transpose(x, dim0: int = -2, dim1: int = -1):
    """rumus/src/tensor/ops.rs:36 / :1612 (tracked): a strided view, no copy."""
    return x.transpose(dim0, dim1)


def batched_transpose(x):
    """rumus/src/tensor/ops.rs:1644: swap the last two dims of a ``[B, M, N]`` tensor."""
    return x.transpose(-2, -1)


def reshape(x, *shape):
    """rumus/src/tensor/ops.rs:44 / :1242 (tracked)."""
    return x.reshape(*shape)


def flatten(x, start_dim: int = 1):
    """rumus/src/tensor/ops.rs:2366: ``[B, ...] -> [B, prod(...)]``."""
    return x.flatten(start_dim)


def contiguous(x):
    """rumus/src/tensor/ops.rs:61 / :1573 (tracked)."""
    return x.contiguous()


def add(a, b):
    """rumus/src/tensor/ops.rs:404 (same shape) and :2154 (broadcast)."""
    return a + b


def sub(a, b):
    """rumus/src/tensor/ops.rs:448 and :2174."""
    return a - b


def mul(a, b):
    """rumus/src/tensor/ops.rs:469 and :2194."""
    return a * b


broadcast_add, broadcast_sub, broadcast_mul = add, sub, mul


def tanh_act(x):
    """rumus/src/tensor/ops.rs:1422."""
    return tanh(x)


def to_dtype(x, dtype: torch.dtype):
    """rumus/src/tensor/ops.rs:2205 (F32 <-> F16 there; any floating dtype here, differentiable)."""
    return x.to(dtype)


def slice_batch(x, start: int, end: int):
    """rumus/src/tensor/ops.rs:944: rows ``[start, end)`` of the leading dim."""
    return x[start:end]


def slice_range(x, dim: int, start: int, end: int):
    """rumus/src/tensor/ops.rs:2423."""
    return x.narrow(dim, start, end - start)


def cat(tensors, dim: int = 0):
    """rumus/src/tensor/ops.rs:2498."""
    return torch.cat(list(tensors), dim=dim)


def stack(tensors, dim: int = 0):
    """rumus/src/tensor/ops.rs:2599."""
    return torch.stack(list(tensors), dim=dim)


def add_channel_bias(x, bias):
    """rumus/src/tensor/ops.rs:1084: ``x [.., C, H, W] + bias [C]``."""
    return x + bias.view(-1, 1, 1)


def im2col(x, kernel_size: int, stride: int = 1, padding: int = 0):
    """rumus/src/tensor/ops.rs:1010: ``[C, H, W]`` (or ``[B, C, H, W]``) -> ``[C*k*k, L]`` columns
    (``[B, C*k*k, L]``).  Convolutions do not go through this op here (they use the channels-last
    kernels of ``ops/vision.py``); it exists for code that builds its own unfold-based layers."""
    squeeze = x.dim() == 3
    cols = torch.nn.functional.unfold(x[None] if squeeze else x, kernel_size, padding=padding,
                                      stride=stride)
    return cols[0] if squeeze else cols


def batch_norm_2d(x, weight, bias, running_mean, running_var, training: bool,
                  momentum: float = 0.1, eps: float = 1e-5):
    """rumus/src/tensor/ops.rs:1840."""
    from .vision import batch_norm2d
    return batch_norm2d(x, weight, bias, running_mean, running_var, training, momentum, eps)


def max_pool2d(x, kernel_size: int, stride: Optional[int] = None, padding: int = 0):
    """rumus/src/tensor/ops.rs:1163."""
    from .vision import max_pool2d as _mp
    return _mp(x, kernel_size, stride, padding)


def adaptive_avg_pool2d(x, output_size):
    """rumus/src/tensor/ops.rs:2019."""
    from .vision import adaptive_avg_pool2d as _ap
    return _ap(x, output_size)


def quantize(weight, block_size: int = 32):
    """rumus/src/tensor/ops.rs:2290: per-block INT8 of a ``[K, N]`` weight (reference byte layout)."""
    from ..nn.quant import quantize_q8
    return quantize_q8(weight, block_size)


def dequantize(q, dtype: torch.dtype = torch.float32):
    """rumus/src/tensor/ops.rs:2332."""
    from ..nn.quant import dequantize_q8
    return dequantize_q8(q, dtype)
