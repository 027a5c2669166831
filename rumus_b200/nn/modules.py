"""Module library.

Every layer is a ``torch.nn.Module`` whose ``state_dict`` keys and tensor layouts
match the reference framework's checkpoints (rumus/src/nn/*.rs): ``Linear.weight``
is ``[in, out]``, ``Conv2d.weight`` is 2-D ``[C_out, C_in*K*K]``, BatchNorm carries
``running_mean`` / ``running_var`` only, attention exposes separate
``q_proj / k_proj / v_proj / out_proj`` entries even though the projections run
as one fused GEMM.  Forward passes call ``rumus_b200.ops.functional`` (sm_100a
kernels on CUDA tensors, PyTorch math on CPU tensors).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F


class Module(nn.Module):
    """Base class: adds the reference's ``Module`` conveniences (rumus/src/nn/module.rs:19-58)."""

    def parameters_list(self):
        return list(self.parameters())

    def to_gpu(self, device: Optional[int] = None):
        """reference: ModuleToGpu (rumus/src/nn/module.rs:66-79)"""
        return self.to(torch.device("cuda", device if device is not None else torch.cuda.current_device()))


class _Lcg:
    """64-bit LCG used by the reference initialisers (rumus/src/nn/linear.rs:15-31)."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def uniform(self, n: int, bound: float) -> torch.Tensor:
        out = torch.empty(n, dtype=torch.float32)
        s = self.s
        vals = []
        for _ in range(n):
            s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
            u = (s >> 33) / float(1 << 31)
            vals.append((2.0 * u - 1.0) * bound)
        self.s = s
        out.copy_(torch.tensor(vals, dtype=torch.float32))
        return out


_linear_rng = _Lcg(42)
_conv_rng = _Lcg(123456789)
_embed_rng = _Lcg(987654321)
_REFERENCE_INIT = {"enabled": False}


def use_reference_init(flag: bool = True) -> None:
    """Switch initialisers to the reference's LCG streams (slow, pure Python; for parity tests)."""
    _REFERENCE_INIT["enabled"] = flag
    if flag:
        _linear_rng.s, _conv_rng.s, _embed_rng.s = 42, 123456789, 987654321


def _uniform(shape, bound, rng: _Lcg, device=None, dtype=None):
    n = int(math.prod(shape))
    if _REFERENCE_INIT["enabled"]:
        t = rng.uniform(n, bound).view(*shape)
    else:
        t = (torch.rand(shape) * 2 - 1) * bound
    return t.to(device=device, dtype=dtype or torch.float32)


class Linear(Module):
    """``y = x @ weight + bias`` with ``weight [in, out]`` (rumus/src/nn/linear.rs:44-100).

    The ``[in, out]`` storage is what the reference checkpoints hold; it reaches the tcgen05 GEMM
    as an N-major B operand, and its transpose views serve dgrad / wgrad without copies.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 dtype=None, act: Optional[str] = None):
        super().__init__()
        self.in_features, self.out_features, self.act = in_features, out_features, act
        bound = math.sqrt(1.0 / in_features)
        self.weight = nn.Parameter(_uniform((in_features, out_features), bound, _linear_rng, device, dtype))
        self.bias = nn.Parameter(_uniform((out_features,), bound, _linear_rng, device, dtype)) if bias else None

    def forward(self, x, residual=None):
        return F.linear(x, self.weight, self.bias, act=self.act, residual=residual)


class LayerNorm(Module):
    """rumus/src/nn (LayerNorm: weight/bias [D], eps 1e-5); kernel: csrc/kernels/norm.cu"""

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(dim, device=device, dtype=dtype))

    def forward(self, x, residual=None):
        return F.layer_norm(x, self.weight, self.bias, self.eps, residual=residual)


class RMSNorm(Module):
    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x, residual=None):
        return F.rms_norm(x, self.weight, self.eps, residual=residual)


class Embedding(Module):
    """``weight [vocab, dim]``, U(-1, 1) init (rumus/src/nn/embedding.rs)."""

    def __init__(self, num_embeddings: int, dim: int, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(_uniform((num_embeddings, dim), 1.0, _embed_rng, device, dtype))

    def forward(self, idx, pos: Optional[torch.Tensor] = None):
        return F.embedding(idx, self.weight, pos)


class Dropout(Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return F.dropout(x, self.p, self.training)


class Flatten(Module):
    def forward(self, x):
        return x.reshape(x.shape[0], -1)


def scaled_dot_product_attention(q, k, v, mask=None):
    """Materialised attention on ``[B*, S, d]`` tensors with an additive mask
    (rumus/src/nn/attention.rs:17-58).  Kept for API parity; models use ``flash_attention``."""
    d = q.shape[-1]
    s = F.bmm(q, k.transpose(1, 2)) * (1.0 / math.sqrt(d))
    if mask is not None:
        s = s + mask
    return F.bmm(F.softmax(s), v)


class _ProjView(nn.Module):
    """Placeholder child so that ``q_proj`` etc. show up as attributes holding views."""

    def __init__(self, weight, bias):
        super().__init__()
        object.__setattr__(self, "weight", weight)
        object.__setattr__(self, "bias", bias)


class MultiheadAttention(Module):
    """Self-attention (rumus/src/nn/attention.rs:60-140).

    Checkpoint keys are ``q_proj/k_proj/v_proj/out_proj .weight/.bias`` (``[in,out]``) as in
    the reference; internally q/k/v live in ONE ``[d, (H + 2*Hkv)*hd]`` parameter so the
    projection is a single GEMM whose output feeds FlashAttention through strided views.
    """

    def __init__(self, d_model: int, num_heads: int, bias: bool = True, causal: bool = True,
                 num_kv_heads: Optional[int] = None, rope_theta: Optional[float] = None,
                 device=None, dtype=None):
        super().__init__()
        assert d_model % num_heads == 0
        self.d_model, self.num_heads = d_model, num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.head_dim = d_model // num_heads
        self.causal = causal
        self.rope_theta = rope_theta
        bound = math.sqrt(1.0 / d_model)
        kv_dim = self.num_kv_heads * self.head_dim
        wq = _uniform((d_model, d_model), bound, _linear_rng, device, dtype)
        bq = _uniform((d_model,), bound, _linear_rng, device, dtype) if bias else None
        wk = _uniform((d_model, kv_dim), bound, _linear_rng, device, dtype)
        bk = _uniform((kv_dim,), bound, _linear_rng, device, dtype) if bias else None
        wv = _uniform((d_model, kv_dim), bound, _linear_rng, device, dtype)
        bv = _uniform((kv_dim,), bound, _linear_rng, device, dtype) if bias else None
        self.qkv_weight = nn.Parameter(torch.cat([wq, wk, wv], dim=1).contiguous())
        self.qkv_bias = nn.Parameter(torch.cat([bq, bk, bv]).contiguous()) if bias else None
        self.out_proj = Linear(d_model, d_model, bias, device, dtype)
        self._register_state_dict_hook(_mha_state_dict_hook)
        self._register_load_state_dict_pre_hook(_mha_load_hook, with_module=True)

    def _splits(self):
        kv = self.num_kv_heads * self.head_dim
        return [self.d_model, kv, kv]

    def forward(self, x, mask=None, residual=None):
        B, S, _ = x.shape
        qkv = F.linear(x, self.qkv_weight, self.qkv_bias)
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if self.rope_theta is not None:
            qkv = F.rope_qkv(qkv, S, H, Hkv, hd, self.rope_theta)
        if (mask is None and hd == 128 and qkv.is_cuda
                and qkv.dtype in (torch.bfloat16, torch.float16) and qkv.data_ptr() % 16 == 0):
            # packed path: the backward kernels write d_q / d_k / d_v into one d_qkv buffer
            o = F.flash_attention_packed(qkv, H, Hkv, self.causal)
            return self.out_proj(o.reshape(B, S, self.d_model), residual=residual)
        q, k, v = qkv.split(self._splits(), dim=-1)
        q = q.view(B, S, H, hd)
        k = k.view(B, S, Hkv, hd)
        v = v.view(B, S, Hkv, hd)
        if mask is not None:
            # additive-mask path of the reference API (materialised scores)
            qh = q.permute(0, 2, 1, 3).reshape(B * H, S, hd)
            kh = k.permute(0, 2, 1, 3).reshape(B * H, S, hd)
            vh = v.permute(0, 2, 1, 3).reshape(B * H, S, hd)
            o = scaled_dot_product_attention(qh, kh, vh, mask)
            o = o.view(B, H, S, hd).permute(0, 2, 1, 3)
        else:
            o = F.flash_attention(q, k, v, self.causal)
        return self.out_proj(o.reshape(B, S, self.d_model), residual=residual)


def _mha_state_dict_hook(module, state, prefix, local_metadata):
    w = state.pop(prefix + "qkv_weight")
    ws = w.split(module._splits(), dim=1)
    b = state.pop(prefix + "qkv_bias", None)
    bs = b.split(module._splits()) if b is not None else (None, None, None)
    out = OrderedDict()
    for name, wi, bi in zip(("q_proj", "k_proj", "v_proj"), ws, bs):
        out[prefix + name + ".weight"] = wi.contiguous()
        if bi is not None:
            out[prefix + name + ".bias"] = bi.contiguous()
    # keep a stable order: q,k,v then the rest (out_proj.*)
    rest = [(k, state.pop(k)) for k in list(state.keys()) if k.startswith(prefix)]
    for k, v in out.items():
        state[k] = v
    for k, v in rest:
        state[k] = v
    return state


def _mha_load_hook(module, state, prefix, local_metadata, strict, missing, unexpected, errors):
    names = ("q_proj", "k_proj", "v_proj")
    if all(prefix + n + ".weight" in state for n in names):
        state[prefix + "qkv_weight"] = torch.cat([state.pop(prefix + n + ".weight") for n in names], dim=1)
        if all(prefix + n + ".bias" in state for n in names):
            state[prefix + "qkv_bias"] = torch.cat([state.pop(prefix + n + ".bias") for n in names])


class TransformerBlock(Module):
    """Pre-norm block ``h = x + Attn(LN(x)); h = h + MLP(LN(h))``
    (rumus/src/nn/transformer.rs:19-59; fields ``ln1, attn, ln2, mlp_fc1, mlp_fc2``).

    ``activation`` generalises the reference's hard-coded GELU.  On CUDA the residual adds are
    fused: attention's add rides in the ``out_proj`` GEMM epilogue, the MLP's in the ``mlp_fc2``
    epilogue, and the activation (and its derivative in backward) in GEMM epilogues.
    """

    def __init__(self, d_model: int, num_heads: int, mlp_dim: Optional[int] = None,
                 activation: str = "gelu", causal: bool = True, device=None, dtype=None):
        super().__init__()
        mlp_dim = mlp_dim or 4 * d_model
        self.d_model = d_model
        self.activation = activation
        self.ln1 = LayerNorm(d_model, 1e-5, device, dtype)
        self.attn = MultiheadAttention(d_model, num_heads, True, causal, device=device, dtype=dtype)
        self.ln2 = LayerNorm(d_model, 1e-5, device, dtype)
        self.mlp_fc1 = Linear(d_model, mlp_dim, True, device, dtype)
        self.mlp_fc2 = Linear(mlp_dim, d_model, True, device, dtype)

    def forward(self, x, mask=None):
        # the skip stream is taken from the norm op (see F.norm_skip): the gradient that comes back
        # along it is added inside the norm's backward kernel
        y, skip = F.norm_skip(x, self.ln1.weight, self.ln1.bias, self.ln1.eps)
        h = self.attn(y, mask, residual=skip)
        y2, skip2 = F.norm_skip(h, self.ln2.weight, self.ln2.bias, self.ln2.eps)
        return F.mlp(y2, self.mlp_fc1.weight, self.mlp_fc1.bias, self.mlp_fc2.weight,
                     self.mlp_fc2.bias, act=self.activation, residual=skip2)


# activation / loss free functions (rumus/src/nn/mod.rs exports)
relu = F.relu
gelu = F.gelu
sigmoid = F.sigmoid
tanh = F.tanh
leaky_relu = F.leaky_relu
silu = F.silu
softmax = F.softmax
mse_loss = F.mse_loss
cross_entropy_loss = F.cross_entropy_loss
