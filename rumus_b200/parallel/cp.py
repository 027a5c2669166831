"""Context (sequence) parallel attention for long sequences: every rank holds ``S / P`` tokens.

Two schemes over a process group of ``P`` ranks, both differentiable:

* ``ulysses_attention`` — two all-to-alls around an ordinary attention call: the first turns the
  sequence sharding ``[B, S/P, H, D]`` into a head sharding ``[B, S, H/P, D]``, FlashAttention runs
  on whole sequences for ``H/P`` heads, the second all-to-all restores the sequence sharding.
  Needs ``H % P == 0`` (and ``Hkv % P == 0``).
* ``ring_attention`` — K/V blocks travel around the ring (``P - 1`` exchanges), every rank
  attends its local queries to each visiting block and merges the partial results with their
  log-sum-exp, exactly as a FlashAttention kernel merges K/V tiles.  Causal masking is by block:
  blocks from later ranks are skipped, the own block is causal, earlier blocks are full.  The
  backward pass re-runs the ring: dK/dV contributions travel with their block and arrive at the
  owner after ``P`` steps.

The reference has no context parallelism (attention is single-device: rumus/src/nn/attention.rs:17-58,
rumus/src/tensor/ops.rs:2685-2743); these are the long-context extensions of the tensor-parallel
sequence-sharded layout used by ``parallel/tp.py``.

Transport is ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks): attention inputs of this
size are bandwidth-, not latency-bound, and the exchanges overlap with the attention kernels of the
previous block through the asynchronous p2p requests.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F


# --------------------------------------------------------------------------------------------
# Ulysses: all-to-all (sequence -> heads), attention, all-to-all (heads -> sequence)
# --------------------------------------------------------------------------------------------
def _all_to_all_4d(x: torch.Tensor, scatter_dim: int, gather_dim: int, group) -> torch.Tensor:
    """Split ``x`` along ``scatter_dim`` into P parts, exchange, concatenate along ``gather_dim``."""
    world = dist.get_world_size(group)
    parts = [t.contiguous() for t in x.chunk(world, dim=scatter_dim)]
    recv = [torch.empty_like(parts[0]) for _ in range(world)]
    if x.is_cuda:
        dist.all_to_all(recv, parts, group=group)
    else:
        # gloo has no all_to_all: P rounds of pairwise exchanges
        rank = dist.get_rank(group)
        recv[rank].copy_(parts[rank])
        for shift in range(1, world):
            dst, src = (rank + shift) % world, (rank - shift) % world
            ops = [dist.P2POp(dist.isend, parts[dst], dist.get_global_rank(group, dst) if group else dst, group),
                   dist.P2POp(dist.irecv, recv[src], dist.get_global_rank(group, src) if group else src, group)]
            for r in dist.batch_isend_irecv(ops):
                r.wait()
    return torch.cat(recv, dim=gather_dim)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group):
        ctx.scatter_dim, ctx.gather_dim, ctx.group = scatter_dim, gather_dim, group
        return _all_to_all_4d(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all_4d(g, ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None, None


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                      group: Optional[dist.ProcessGroup] = None,
                      scale: Optional[float] = None) -> torch.Tensor:
    """``q [B, S/P, H, D]``, ``k/v [B, S/P, Hkv, D]`` (this rank's tokens, ranks in sequence order)
    -> ``[B, S/P, H, D]``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return F.flash_attention(q, k, v, causal, scale)
    H, Hkv = q.shape[2], k.shape[2]
    assert H % world == 0 and Hkv % world == 0, "heads must divide over the context-parallel group"
    qh = _AllToAll.apply(q, 2, 1, group)     # [B, S, H/P, D]
    kh = _AllToAll.apply(k, 2, 1, group)
    vh = _AllToAll.apply(v, 2, 1, group)
    o = F.flash_attention(qh, kh, vh, causal, scale)
    return _AllToAll.apply(o, 1, 2, group)   # [B, S/P, H, D]


# --------------------------------------------------------------------------------------------
# Ring attention
# --------------------------------------------------------------------------------------------
def _use_kernels(q: torch.Tensor) -> bool:
    return q.is_cuda and q.shape[-1] == 128 and q.dtype in (torch.bfloat16, torch.float16)


def _attend_block(q, k, v, mode: str, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of local queries to one K/V block: returns (out [B,Sq,H,D] fp32, lse [B,H,Sq]).
    ``mode``: "full" or "causal" (block diagonal of the global causal mask).  On CUDA with
    head_dim 128 this is the tcgen05 FlashAttention forward (which returns the log-sum-exp);
    otherwise plain fp32 math."""
    if _use_kernels(q):
        from ..ops.attention import fa_forward
        o, lse, _ = fa_forward(q, k, v, mode == "causal", scale)
        return o.float(), lse
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    qf = q.permute(0, 2, 1, 3).float()
    kf = k.permute(0, 2, 1, 3).float()
    vf = v.permute(0, 2, 1, 3).float()
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, dim=1)
        vf = vf.repeat_interleave(H // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if mode == "causal":
        Sk = kf.shape[2]
        mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                       # [B,H,Sq]
    p = torch.exp(s - lse.unsqueeze(-1))
    o = (p @ vf).permute(0, 2, 1, 3)                       # [B,Sq,H,D]
    return o, lse


def _ring_exchange(tensors, group):
    """Send ``tensors`` to the next rank, receive the previous rank's; returns the received ones."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    if group is not None:
        nxt, prv = dist.get_global_rank(group, nxt), dist.get_global_rank(group, prv)
    recv = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, prv, group))
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("-inf"), dtype=torch.float32,
                         device=q.device)
        kb, vb = k, v
        for step in range(world):
            src = (rank - step) % world            # owner of the block now held
            if not causal or src <= rank:
                mode = "causal" if (causal and src == rank) else "full"
                o_b, lse_b = _attend_block(q, kb, vb, mode, scale)
                new = torch.logaddexp(lse, lse_b)
                w_old = torch.exp(lse - new).permute(0, 2, 1).unsqueeze(-1)
                w_new = torch.exp(lse_b - new).permute(0, 2, 1).unsqueeze(-1)
                out = out * w_old + o_b * w_new
                lse = new
            if step + 1 < world:
                kb, vb = _ring_exchange([kb, vb], group)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.group = causal, scale, group
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, causal, scale = ctx.group, ctx.causal, ctx.scale
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        B, Sq, H, D = q.shape
        Hkv = k.shape[2]
        rep = H // Hkv
        do = dout.float()
        delta = (do * out).sum(-1).permute(0, 2, 1)        # [B,H,Sq]
        qf = q.permute(0, 2, 1, 3).float()
        dof = do.permute(0, 2, 1, 3)
        dq = torch.zeros_like(qf)
        kb, vb = k, v
        dkb = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dvb = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
        kern = _use_kernels(q)
        if kern:
            from ..ops.attention import fa_backward
            out_t = out.to(q.dtype)
            dout_t = dout.contiguous()
        for step in range(world):
            src = (rank - step) % world
            if kern and (not causal or src <= rank):
                # block backward with the GLOBAL output and log-sum-exp: P = exp(S - lse) are then
                # the true attention weights of this block and delta = rowsum(dO * O) is global
                dq_c, dk_c, dv_c = fa_backward(q, kb.contiguous(), vb.contiguous(), out_t, lse, dout_t,
                                               causal and src == rank, scale)
                dq += dq_c.permute(0, 2, 1, 3).float()
                dkb += dk_c.float()
                dvb += dv_c.float()
            elif not causal or src <= rank:
                kf = kb.permute(0, 2, 1, 3).float()
                vf = vb.permute(0, 2, 1, 3).float()
                if rep != 1:
                    kf = kf.repeat_interleave(rep, dim=1)
                    vf = vf.repeat_interleave(rep, dim=1)
                s = (qf @ kf.transpose(-1, -2)) * scale
                if causal and src == rank:
                    mask = torch.ones(Sq, kf.shape[2], dtype=torch.bool, device=q.device).tril()
                    s = s.masked_fill(~mask, float("-inf"))
                p = torch.exp(s - lse.unsqueeze(-1))                     # [B,H,Sq,Sk]
                dv_c = p.transpose(-1, -2) @ dof                          # [B,H,Sk,D]
                dp = dof @ vf.transpose(-1, -2)
                ds = p * (dp - delta.unsqueeze(-1)) * scale
                dq += ds @ kf
                dk_c = ds.transpose(-1, -2) @ qf
                if rep != 1:
                    dk_c = dk_c.view(B, Hkv, rep, -1, D).sum(2)
                    dv_c = dv_c.view(B, Hkv, rep, -1, D).sum(2)
                dkb += dk_c.permute(0, 2, 1, 3)
                dvb += dv_c.permute(0, 2, 1, 3)
            # the block and its gradient accumulators move on together; after `world` moves the
            # accumulators are back at the block's owner
            if step + 1 < world:
                kb, vb, dkb, dvb = _ring_exchange([kb, vb, dkb, dvb], group)
            else:
                dkb, dvb = _ring_exchange([dkb, dvb], group)
        return (dq.permute(0, 2, 1, 3).to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                   group: Optional[dist.ProcessGroup] = None,
                   scale: Optional[float] = None) -> torch.Tensor:
    """Same contract as ``ulysses_attention`` without the head-count restriction."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if world == 1:
        return F.flash_attention(q, k, v, causal, scale)
    return _RingAttention.apply(q, k, v, causal, scale, group)
