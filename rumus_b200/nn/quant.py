"""Weight-only quantisation: INT4 group-wise asymmetric (AWQ/GPTQ-style storage) and INT8
block quantisation, in the reference's storage formats.

INT4 (rumus-vision/src/quant.rs:42-126): weight ``[K, N]``, K padded to the group size,
per-(group, column) ``scale = (max-min)/15``, ``zp = -min/scale``,
``q = clamp(round(v/scale + zp), 0, 15)``; eight nibbles per 32-bit word along K:
word ``(row // 8) * N + col``, nibble ``row % 8``.  Scales / zero-points are ``[groups, N]``
(fp32 in the reference; fp16 here when ``scale_dtype=torch.float16``, as the serving config asks).

INT8 (rumus/src/tensor/ops.rs:2290, shaders/quantize.wgsl:30): the matrix is transposed so each
column's K run is contiguous, then cut into blocks of ``block_size`` values; a block is a 4-byte
header (f16 scale in the low 16 bits) followed by ``block_size`` int8 values;
``scale = absmax/127`` (1.0 for an all-zero block), ``q = clamp(round(v*127/absmax), -128, 127)``.

The GEMV / dequantise kernels live in ``csrc/kernels/quant.cu``; CPU tensors use the PyTorch
restatement below, which is also the test oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .modules import Linear, Module


@dataclass
class QuantizedTensor:
    """INT4 group-quantised ``[K, N]`` weight."""
    k: int
    n: int
    padded_k: int
    group_size: int
    packed: torch.Tensor       # int32 [padded_k // 8, N]
    scales: torch.Tensor       # [groups, N]
    zero_points: torch.Tensor  # [groups, N]

    @property
    def num_groups(self) -> int:
        return self.padded_k // self.group_size

    @staticmethod
    def from_f32(weight: torch.Tensor, group_size: int = 128,
                 scale_dtype: torch.dtype = torch.float32) -> "QuantizedTensor":
        assert group_size % 8 == 0 and weight.dim() == 2
        k, n = weight.shape
        # the packer is plain tensor math and runs where the weight lives (a 7B model quantised on
        # the GPU at load time takes seconds; the same code on CPU tensors is the test oracle)
        w = weight.detach().float()
        dev0 = w.device
        padded_k = ((k + group_size - 1) // group_size) * group_size
        groups = padded_k // group_size
        wp = torch.zeros(padded_k, n, device=dev0)
        wp[:k] = w
        g = wp.view(groups, group_size, n)
        mn, mx = g.min(dim=1).values, g.max(dim=1).values
        rng = mx - mn
        ok = rng > 1e-10
        scale = torch.where(ok, rng / 15.0, torch.ones_like(rng))
        zp = torch.where(ok, -mn / scale, torch.zeros_like(rng))
        if scale_dtype != torch.float32:
            # quantise with the values the kernel will actually read back
            scale = scale.to(scale_dtype).float()
            zp = zp.to(scale_dtype).float()
        q = torch.clamp(torch.round(g / scale[:, None, :] + zp[:, None, :]), 0, 15).to(torch.int64)
        q = q.view(padded_k // 8, 8, n)
        shifts = (torch.arange(8, dtype=torch.int64, device=dev0) * 4).view(1, 8, 1)
        words = (q << shifts).sum(dim=1)                      # [padded_k/8, N] as int64 in [0, 2^32)
        words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
        dev = weight.device
        return QuantizedTensor(k, n, padded_k, group_size, words.to(dev),
                               scale.to(scale_dtype).to(dev), zp.to(scale_dtype).to(dev))

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        words = self.packed.to(torch.int64) & 0xFFFFFFFF
        shifts = (torch.arange(8, dtype=torch.int64, device=words.device) * 4).view(1, 8, 1)
        q = ((words[:, None, :] >> shifts) & 0xF).reshape(self.padded_k, self.n).float()
        s = self.scales.float().repeat_interleave(self.group_size, dim=0)
        z = self.zero_points.float().repeat_interleave(self.group_size, dim=0)
        return ((q - z) * s)[: self.k].to(dtype)

    def to(self, device) -> "QuantizedTensor":
        return QuantizedTensor(self.k, self.n, self.padded_k, self.group_size, self.packed.to(device),
                               self.scales.to(device), self.zero_points.to(device))


def qmatmul_int4(x: torch.Tensor, qw: QuantizedTensor) -> torch.Tensor:
    """``x [M, K] @ dequant(qw) [K, N]`` (rumus-vision/src/shaders/qmatmul_int4.wgsl:41)."""
    if x.is_cuda:
        from ..ops.quant_cuda import QMatmulInt4Fn
        return QMatmulInt4Fn.apply(x, qw)
    return x @ qw.dequantize(x.dtype)


class QLinear(Module):
    """Frozen INT4 linear layer (rumus-vision/src/quant.rs:165-222)."""

    def __init__(self, qweight: QuantizedTensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.qweight = qweight
        self.register_buffer("packed", qweight.packed)
        self.register_buffer("scales", qweight.scales)
        self.register_buffer("zero_points", qweight.zero_points)
        self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False) if bias is not None else None

    @staticmethod
    def from_linear(linear: Linear, group_size: int = 128,
                    scale_dtype: torch.dtype = torch.float32) -> "QLinear":
        return QLinear(QuantizedTensor.from_f32(linear.weight.data, group_size, scale_dtype),
                       linear.bias.data if linear.bias is not None else None)

    def _q(self) -> QuantizedTensor:
        q = self.qweight
        return QuantizedTensor(q.k, q.n, q.padded_k, q.group_size, self.packed, self.scales,
                               self.zero_points)

    def forward(self, x):
        shp = x.shape
        y = qmatmul_int4(x.reshape(-1, shp[-1]), self._q())
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.view(*shp[:-1], self.qweight.n)


# ----------------------------------------------------------------------------- INT8
def _f16_bits(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).view(torch.int16).to(torch.int32) & 0xFFFF


@dataclass
class Q8Tensor:
    """INT8 block-quantised ``[K, N]`` weight in the reference's fused byte layout."""
    k: int
    n: int
    block_size: int
    data: torch.Tensor  # uint8 [num_blocks * (4 + block_size)]

    @property
    def num_blocks(self) -> int:
        return (self.k * self.n + self.block_size - 1) // self.block_size


def quantize_q8(weight: torch.Tensor, block_size: int = 32) -> Q8Tensor:
    assert block_size > 0 and block_size % 4 == 0 and weight.dim() == 2
    if weight.is_cuda:
        from ..ops.quant_cuda import quantize_q8_cuda
        return quantize_q8_cuda(weight, block_size)
    k, n = weight.shape
    flat = weight.detach().float().t().contiguous().view(-1)   # column-major: each column's K run
    numel = flat.numel()
    nb = (numel + block_size - 1) // block_size
    pad = nb * block_size - numel
    if pad:
        flat = torch.cat([flat, torch.zeros(pad)])
    blocks = flat.view(nb, block_size)
    absmax = blocks.abs().max(dim=1).values
    scale = torch.where(absmax == 0, torch.ones_like(absmax), absmax / 127.0)
    inv = torch.where(absmax == 0, torch.zeros_like(absmax), 127.0 / absmax)
    q = torch.clamp(torch.round(blocks * inv[:, None]), -128, 127).to(torch.int8)
    out = torch.zeros(nb, 4 + block_size, dtype=torch.uint8)
    bits = _f16_bits(scale)
    out[:, 0] = (bits & 0xFF).to(torch.uint8)
    out[:, 1] = ((bits >> 8) & 0xFF).to(torch.uint8)
    out[:, 4:] = q.view(torch.uint8)
    return Q8Tensor(k, n, block_size, out.view(-1))


def dequantize_q8(q: Q8Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if q.data.is_cuda:
        from ..ops.quant_cuda import dequantize_q8_cuda
        return dequantize_q8_cuda(q, dtype)
    blocks = q.data.view(q.num_blocks, 4 + q.block_size)
    bits = blocks[:, 0].to(torch.int32) | (blocks[:, 1].to(torch.int32) << 8)
    scale = bits.to(torch.int16).view(torch.float16).float()
    vals = blocks[:, 4:].contiguous().view(torch.int8).float() * scale[:, None]
    flat = vals.view(-1)[: q.k * q.n]
    return flat.view(q.n, q.k).t().contiguous().to(dtype)


def matmul_q8(x: torch.Tensor, q: Q8Tensor) -> torch.Tensor:
    """``x [M, K] @ dequant(q) [K, N]`` (rumus/src/backend/gpu/shaders/matmul_q8.wgsl:38)."""
    if x.is_cuda:
        from ..ops.quant_cuda import matmul_q8_cuda
        return matmul_q8_cuda(x, q)
    return x @ dequantize_q8(q, x.dtype)


class Q8Linear(Module):
    def __init__(self, q: Q8Tensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.q = q
        self.register_buffer("data", q.data)
        self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False) if bias is not None else None

    @staticmethod
    def from_linear(linear: Linear, block_size: int = 32) -> "Q8Linear":
        return Q8Linear(quantize_q8(linear.weight.data, block_size),
                        linear.bias.data if linear.bias is not None else None)

    def forward(self, x):
        shp = x.shape
        y = matmul_q8(x.reshape(-1, shp[-1]), Q8Tensor(self.q.k, self.q.n, self.q.block_size, self.data))
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.view(*shp[:-1], self.q.n)
