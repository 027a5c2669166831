"""Llama-style decoder for tensor x pipeline parallel training (TP with sequence-parallel
activations inside a stage, 1F1B between stages).

A stage owns a contiguous range of blocks; the first stage also owns the token embedding, the
last stage the final norm, the vocabulary-parallel head and the loss.  Between blocks the
residual stream is token-sharded ``[M/T, d]`` (M = micro-batch tokens): norms and residual adds
touch 1/T of the tokens, column-parallel layers all-gather it, row-parallel layers reduce-scatter
back (``parallel/tp.py``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..nn import Embedding, Module, RMSNorm
from ..ops import functional as F
from ..parallel.tp import (ColumnParallelLinear, RowParallelLinear, TPContext, gather_rows,
                           mark_tp_replicated, scatter_rows)
from .llama import LlamaConfig


class ParallelLlamaBlock(Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, device=None, dtype=None):
        super().__init__()
        self.cfg, self.tp = cfg, tp
        T = tp.world
        self.hd = cfg.d_model // cfg.num_heads
        self.h_local = cfg.num_heads // T
        self.hkv_local = cfg.num_kv_heads // T
        qkv_out = (cfg.num_heads + 2 * cfg.num_kv_heads) * self.hd
        self.ln1 = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
        # per-rank column layout: [q heads of this rank | k heads | v heads]
        self.qkv = ColumnParallelLinear(cfg.d_model, qkv_out, tp, bias=False, device=device, dtype=dtype)
        self.out_proj = RowParallelLinear(cfg.num_heads * self.hd, cfg.d_model, tp, bias=False,
                                          device=device, dtype=dtype)
        self.ln2 = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
        self.gate_up = ColumnParallelLinear(cfg.d_model, 2 * cfg.ffn_dim, tp, bias=False, device=device,
                                            dtype=dtype)
        self.down = RowParallelLinear(cfg.ffn_dim, cfg.d_model, tp, bias=False, device=device, dtype=dtype)
        # the norms run on this rank's token slab only: their weight gradients are partial sums
        mark_tp_replicated(self.ln1.weight)
        mark_tp_replicated(self.ln2.weight)

    def forward(self, x_local, batch: int, seq: int):
        H, Hkv, hd = self.h_local, self.hkv_local, self.hd
        # the skip stream comes out of the norm op and goes into the row-parallel layer's reduction:
        # no stand-alone residual add in forward, none for the two gradients in backward
        y1, skip = F.norm_skip(x_local, self.ln1.weight, None, self.ln1.eps, rms=True)
        qkv = self.qkv(y1)                                      # [M, (H + 2Hkv) * hd] local heads
        qkv = F.rope_qkv(qkv.view(batch, seq, -1), seq, H, Hkv, hd, self.cfg.rope_theta)
        q, k, v = qkv.split([H * hd, Hkv * hd, Hkv * hd], dim=-1)
        o = F.flash_attention(q.view(batch, seq, H, hd), k.view(batch, seq, Hkv, hd),
                              v.view(batch, seq, Hkv, hd), True)
        h = self.out_proj(o.reshape(batch * seq, H * hd), residual=skip)
        y2, skip2 = F.norm_skip(h, self.ln2.weight, None, self.ln2.eps, rms=True)
        return self.down(F.swiglu(self.gate_up(y2)), residual=skip2)


class _VocabParallelCE(torch.autograd.Function):
    """Cross entropy over a vocabulary split across the TP group: three small all-reduces
    (row max, sum of exponentials, target logit) instead of gathering the logits."""

    @staticmethod
    def forward(ctx, logits_local, targets, tp: TPContext, vocab_start: int):
        lf = logits_local if logits_local.dtype == torch.float64 else logits_local.float()
        m = lf.max(dim=-1).values
        tp.all_reduce(m, op=dist.ReduceOp.MAX)
        e = torch.exp(lf - m[:, None])
        s = e.sum(dim=-1)
        tp.all_reduce(s)
        vloc = logits_local.shape[1]
        tl = targets - vocab_start
        mine = (tl >= 0) & (tl < vloc)
        tgt_logit = torch.where(mine, lf.gather(1, tl.clamp(0, vloc - 1)[:, None]).squeeze(1),
                                torch.zeros_like(m))
        tp.all_reduce(tgt_logit)
        loss = (m + torch.log(s) - tgt_logit).mean()
        p = e / s[:, None]
        p[mine, tl[mine]] -= 1.0
        ctx.save_for_backward((p / logits_local.shape[0]).to(logits_local.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None, None, None


class ParallelLlamaStage(Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, stage: int, num_stages: int, device=None,
                 dtype=None):
        super().__init__()
        self.cfg, self.tp, self.stage, self.num_stages = cfg, tp, stage, num_stages
        per = cfg.num_layers // num_stages
        assert per * num_stages == cfg.num_layers
        self.first, self.last = stage == 0, stage == num_stages - 1
        if self.first:
            self.token_emb = Embedding(cfg.vocab_size, cfg.d_model, device, dtype)
        self.blocks = nn.ModuleList([ParallelLlamaBlock(cfg, tp, device, dtype) for _ in range(per)])
        if self.last:
            self.ln_final = RMSNorm(cfg.d_model, cfg.rms_eps, device, dtype)
            mark_tp_replicated(self.ln_final.weight)
            self.head = ColumnParallelLinear(cfg.d_model, cfg.vocab_size, tp, bias=False, device=device,
                                             dtype=dtype)
        self.batch = self.seq = None

    def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed + 1000 * self.stage + self.tp.rank)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))

    def set_microbatch_shape(self, batch: int, seq: int) -> None:
        """Stages that do not see the tokens need the micro-batch geometry for attention."""
        self.batch, self.seq = batch, seq

    def load_dense(self, dense_state: dict) -> None:
        """Load this stage's / rank's shard from a dense ``Llama`` state dict (reference-layout
        names: ``blocks.N.attn.q_proj.weight`` ... ``[in, out]``)."""
        T, r = self.tp.world, self.tp.rank
        cfg = self.cfg
        per = cfg.num_layers // self.num_stages
        hd = cfg.d_model // cfg.num_heads

        def cols(w, n_heads):
            n = n_heads // T * hd
            return w[:, r * n:(r + 1) * n]

        with torch.no_grad():
            if self.first:
                self.token_emb.weight.copy_(dense_state["token_emb.weight"])
            for i, blk in enumerate(self.blocks):
                p = f"blocks.{self.stage * per + i}."
                wq, wk, wv = (dense_state[p + f"attn.{n}_proj.weight"] for n in "qkv")
                blk.qkv.weight.copy_(torch.cat([cols(wq, cfg.num_heads), cols(wk, cfg.num_kv_heads),
                                                cols(wv, cfg.num_kv_heads)], dim=1))
                wo = dense_state[p + "attn.out_proj.weight"]
                k = wo.shape[0] // T
                blk.out_proj.weight.copy_(wo[r * k:(r + 1) * k])
                f = cfg.ffn_dim // T
                wg, wu = dense_state[p + "mlp.gate_proj.weight"], dense_state[p + "mlp.up_proj.weight"]
                blk.gate_up.weight.copy_(torch.cat([wg[:, r * f:(r + 1) * f], wu[:, r * f:(r + 1) * f]], dim=1))
                wd = dense_state[p + "mlp.down_proj.weight"]
                blk.down.weight.copy_(wd[r * f:(r + 1) * f])
                blk.ln1.weight.copy_(dense_state[p + "ln1.weight"])
                blk.ln2.weight.copy_(dense_state[p + "ln2.weight"])
            if self.last:
                self.ln_final.weight.copy_(dense_state["ln_final.weight"])
                v = cfg.vocab_size // T
                self.head.weight.copy_(dense_state["head.weight"][:, r * v:(r + 1) * v])

    def export_dense(self, gather_stages: bool = True) -> Optional[dict]:
        """Inverse of ``load_dense``: the reference-layout dense state dict assembled from the
        shards.  Tensor-parallel shards are all-gathered inside the TP group and concatenated along
        the dimension they were cut on (columns for q/k/v/gate/up/head, rows for out/down); with
        ``gather_stages`` the pipeline stages are then merged on global rank 0 (returns the full
        dict there, ``None`` on the other ranks).  Saving it with ``save_safetensors`` gives a
        checkpoint any other TP x PP layout — or the dense model — can load."""
        T, cfg = self.tp.world, self.cfg
        per = cfg.num_layers // self.num_stages
        hd = cfg.d_model // cfg.num_heads

        def gather(t: torch.Tensor):
            t = t.detach().contiguous()
            if T == 1:
                return [t]
            parts = [torch.empty_like(t) for _ in range(T)]
            dist.all_gather(parts, t, group=self.tp.group)
            return parts

        out = {}
        if self.first:
            out["token_emb.weight"] = self.token_emb.weight.detach().clone()
        nq, nkv = cfg.num_heads // T * hd, cfg.num_kv_heads // T * hd
        f = cfg.ffn_dim // T
        for i, blk in enumerate(self.blocks):
            p = f"blocks.{self.stage * per + i}."
            qkv = gather(blk.qkv.weight)
            out[p + "attn.q_proj.weight"] = torch.cat([w[:, :nq] for w in qkv], dim=1)
            out[p + "attn.k_proj.weight"] = torch.cat([w[:, nq:nq + nkv] for w in qkv], dim=1)
            out[p + "attn.v_proj.weight"] = torch.cat([w[:, nq + nkv:] for w in qkv], dim=1)
            out[p + "attn.out_proj.weight"] = torch.cat(gather(blk.out_proj.weight), dim=0)
            gu = gather(blk.gate_up.weight)
            out[p + "mlp.gate_proj.weight"] = torch.cat([w[:, :f] for w in gu], dim=1)
            out[p + "mlp.up_proj.weight"] = torch.cat([w[:, f:] for w in gu], dim=1)
            out[p + "mlp.down_proj.weight"] = torch.cat(gather(blk.down.weight), dim=0)
            out[p + "ln1.weight"] = blk.ln1.weight.detach().clone()
            out[p + "ln2.weight"] = blk.ln2.weight.detach().clone()
        if self.last:
            out["ln_final.weight"] = self.ln_final.weight.detach().clone()
            out["head.weight"] = torch.cat(gather(self.head.weight), dim=1)
        if not gather_stages or not dist.is_initialized():
            return out
        world = dist.get_world_size()
        mine = {k: v.cpu() for k, v in out.items()} if self.tp.rank == 0 else None
        every = [None] * world
        dist.all_gather_object(every, mine)
        if dist.get_rank() != 0:
            return None
        full = {}
        for d in every:
            if d:
                full.update(d)
        return full

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] -> token-sharded residual stream [B*S/T, d]."""
        self.batch, self.seq = tokens.shape
        x = self.token_emb(tokens).reshape(-1, self.cfg.d_model)
        return scatter_rows(x, self.tp)

    def forward(self, x):
        """First stage: ``x`` = tokens [B, S].  Other stages: the token-sharded activation.
        Last stage: ``x`` = (activation or tokens, targets [B, S]) and the result is the loss."""
        targets = None
        if self.last:
            x, targets = x
        if self.first:
            x = self.embed(x)
        for blk in self.blocks:
            x = blk(x, self.batch, self.seq)
        if not self.last:
            return x
        h = self.ln_final(x)
        logits_local = self.head(h)                           # [M, V/T] (all-gather fused in)
        vloc = logits_local.shape[1]
        return _VocabParallelCE.apply(logits_local, targets.reshape(-1), self.tp, self.tp.rank * vloc)
