"""GPT-style decoder (learned positional embedding, pre-LN blocks, GELU or ReLU MLP).

Covers two benchmark configurations: the CPU fp32 2-layer decoder (d128, 4 heads, FFN 512 ReLU,
vocab 1024, seq 64) and the 1.3B model (24 layers, d2048, 16 heads, FFN 8192 GELU, vocab 50304,
seq 2048).  Structure and checkpoint names follow the reference's TinyGPT test model
(rumus/tests/transformer_test.rs:21-73): ``token_emb, pos_emb, blocks.N.{ln1,attn,ln2,mlp_fc1,
mlp_fc2}, ln_final, head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..nn import Embedding, LayerNorm, Linear, Module, TransformerBlock
from ..ops import functional as F


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    seq_len: int = 2048
    d_model: int = 2048
    num_heads: int = 16
    num_layers: int = 24
    ffn_dim: int = 8192
    activation: str = "gelu"

    @staticmethod
    def tiny_cpu() -> "GPTConfig":
        return GPTConfig(vocab_size=1024, seq_len=64, d_model=128, num_heads=4, num_layers=2,
                         ffn_dim=512, activation="relu")

    @staticmethod
    def gpt_1p3b() -> "GPTConfig":
        return GPTConfig()

    def num_params(self) -> int:
        d, f, v, s, l = self.d_model, self.ffn_dim, self.vocab_size, self.seq_len, self.num_layers
        per_block = 4 * d * d + 4 * d + 2 * d * f + f + d + 4 * d
        return v * d + s * d + l * per_block + 2 * d + d * v

    def flops_per_token(self) -> float:
        """Training FLOPs per token (fwd + bwd = 3x forward): dense GEMMs plus causal attention."""
        d, f, v, s, l = self.d_model, self.ffn_dim, self.vocab_size, self.seq_len, self.num_layers
        dense = 2 * (l * (4 * d * d + 2 * d * f) + d * v)
        attn = l * 2 * 2 * s * d / 2  # QK^T and PV, causal half
        return 3.0 * (dense + attn)


class GPT(Module):
    def __init__(self, cfg: GPTConfig, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        self.token_emb = Embedding(cfg.vocab_size, cfg.d_model, device, dtype)
        self.pos_emb = Embedding(cfg.seq_len, cfg.d_model, device, dtype)
        self.blocks = nn.ModuleList([
            TransformerBlock(cfg.d_model, cfg.num_heads, cfg.ffn_dim, cfg.activation, True, device, dtype)
            for _ in range(cfg.num_layers)])
        self.ln_final = LayerNorm(cfg.d_model, 1e-5, device, dtype)
        self.head = Linear(cfg.d_model, cfg.vocab_size, False, device, dtype)

    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        """GPT-2 style normal init (random-init weights for benchmarks)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
                elif name.endswith("bias"):
                    p.zero_()

    def hidden(self, idx: torch.Tensor) -> torch.Tensor:
        x = self.token_emb(idx, self.pos_emb.weight)
        for blk in self.blocks:
            x = blk(x)
        return self.ln_final(x)

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None):
        """Returns logits ``[B, S, V]``, or the mean next-token loss when ``targets`` is given."""
        x = self.hidden(idx)
        if targets is None:
            return self.head(x)
        return F.lm_head_loss(x, self.head.weight, targets)
