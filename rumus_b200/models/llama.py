"""Llama-style decoder: RMSNorm, rotary embeddings, SwiGLU MLP, no biases, untied head.

Used by the 7B tensor x pipeline parallel training configuration and by the INT4 serving
configuration (32 layers, d4096, 32 heads, FFN 11008, vocab 32000).  None of RMSNorm / RoPE /
SwiGLU exists in the reference; module names follow its conventions (``attn.q_proj`` ...,
``[in, out]`` weights) so checkpoints keep the same flavour.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..nn import Embedding, Linear, Module, MultiheadAttention, RMSNorm
from ..ops import functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    seq_len: int = 4096
    d_model: int = 4096
    num_heads: int = 32
    num_kv_heads: int = 32
    num_layers: int = 32
    ffn_dim: int = 11008
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5

    @staticmethod
    def llama_7b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(vocab_size=256, seq_len=64, d_model=128, num_heads=2, num_kv_heads=2,
                           num_layers=2, ffn_dim=256)

    def num_params(self) -> int:
        d, f, v, l = self.d_model, self.ffn_dim, self.vocab_size, self.num_layers
        kv = self.num_kv_heads * (d // self.num_heads)
        return 2 * v * d + l * (2 * d * d + 2 * d * kv + 3 * d * f + 2 * d) + d

    def flops_per_token(self) -> float:
        d, f, v, s, l = self.d_model, self.ffn_dim, self.vocab_size, self.seq_len, self.num_layers
        kv = self.num_kv_heads * (d // self.num_heads)
        dense = 2 * (l * (2 * d * d + 2 * d * kv + 3 * d * f) + d * v)
        attn = l * 2 * 2 * s * d / 2
        return 3.0 * (dense + attn)


class LlamaMLP(Module):
    """``down( silu(gate(x)) * up(x) )`` with gate and up fused in one ``[d, 2F]`` GEMM.
    Checkpoint keys: ``gate_proj.weight, up_proj.weight, down_proj.weight`` (``[in, out]``)."""

    def __init__(self, d_model: int, ffn_dim: int, device=None, dtype=None):
        super().__init__()
        self.ffn_dim = ffn_dim
        g = Linear(d_model, ffn_dim, False, device, dtype)
        u = Linear(d_model, ffn_dim, False, device, dtype)
        self.gate_up_weight = nn.Parameter(torch.cat([g.weight.data, u.weight.data], dim=1).contiguous())
        self.down_proj = Linear(ffn_dim, d_model, False, device, dtype)
        self._register_state_dict_hook(_mlp_state_dict_hook)
        self._register_load_state_dict_pre_hook(_mlp_load_hook, with_module=True)

    def forward(self, x, residual=None):
        gu = F.linear(x, self.gate_up_weight)
        return self.down_proj(F.swiglu(gu), residual=residual)


def _mlp_state_dict_hook(module, state, prefix, local_metadata):
    w = state.pop(prefix + "gate_up_weight")
    g, u = w.split(module.ffn_dim, dim=1)
    state[prefix + "gate_proj.weight"] = g.contiguous()
    state[prefix + "up_proj.weight"] = u.contiguous()
    return state


def _mlp_load_hook(module, state, prefix, local_metadata, strict, missing, unexpected, errors):
    if prefix + "gate_proj.weight" in state and prefix + "up_proj.weight" in state:
        state[prefix + "gate_up_weight"] = torch.cat(
            [state.pop(prefix + "gate_proj.weight"), state.pop(prefix + "up_proj.weight")], dim=1)


class LlamaBlock(Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None):
        super().__init__()
        self.ln1 = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
        self.attn = MultiheadAttention(cfg.d_model, cfg.num_heads, bias=False, causal=True,
                                       num_kv_heads=cfg.num_kv_heads, rope_theta=cfg.rope_theta,
                                       device=device, dtype=dtype)
        self.ln2 = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
        self.mlp = LlamaMLP(cfg.d_model, cfg.ffn_dim, device, dtype)

    def forward(self, x):
        y, skip = F.norm_skip(x, self.ln1.weight, None, self.ln1.eps, rms=True)
        h = self.attn(y, residual=skip)
        y2, skip2 = F.norm_skip(h, self.ln2.weight, None, self.ln2.eps, rms=True)
        return self.mlp(y2, residual=skip2)


class Llama(Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.token_emb = Embedding(cfg.vocab_size, cfg.d_model, device, dtype)
        self.blocks = nn.ModuleList([LlamaBlock(cfg, device, dtype) for _ in range(cfg.num_layers)])
        self.ln_final = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
        self.head = Linear(cfg.d_model, cfg.vocab_size, False, device, dtype)

    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))

    def hidden(self, idx):
        x = self.token_emb(idx)
        for blk in self.blocks:
            x = blk(x)
        return self.ln_final(x)

    def forward(self, idx, targets: Optional[torch.Tensor] = None):
        x = self.hidden(idx)
        if targets is None:
            return self.head(x)
        return F.lm_head_loss(x, self.head.weight, targets)
