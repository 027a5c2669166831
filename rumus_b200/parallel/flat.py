"""Flat parameter / gradient arenas.

A ``FlatUnit`` owns the parameters of one sharding unit (an embedding table, one transformer
block, the final norm + head) as views into ONE contiguous low-precision buffer, and their
gradients as views into ONE contiguous gradient buffer (``param.main_grad``; the weight-gradient
GEMMs write there directly, see ``ops.functional._wgrad``).  The optimizer state (fp32 master
weights and Adam moments) is kept for this rank's *shard* of the flat vector only.

The same structure serves a single GPU (world size 1: the shard is the whole vector and one fused
Adam launch updates the unit) and FSDP (``parallel/fsdp.py``: parameters are all-gathered from
the shards, gradients are reduce-scattered into them).

The reference shards every state_dict tensor on dim 0 per linear layer
(rumus/src/nn/fsdp.rs:63-115); a flat per-block vector is the layout that lets one kernel move or
update a whole block.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn

ALIGN = 128  # elements; keeps every parameter view 256-byte aligned for TMA and vector access


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatUnit:
    def __init__(self, name: str, params: List[nn.Parameter], world_size: int = 1, rank: int = 0,
                 alloc: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None,
                 param_alloc: Optional[Callable[[int, torch.dtype, torch.device], torch.Tensor]] = None):
        assert params, name
        self.name, self.params = name, params
        self.world_size, self.rank = world_size, rank
        self.dtype, self.device = params[0].dtype, params[0].device
        offs, off = [], 0
        for p in params:
            assert p.dtype == self.dtype and p.device == self.device
            offs.append(off)
            off += _round_up(p.numel(), ALIGN)
        self.offsets = offs
        self.numel = off
        self.padded = _round_up(off, world_size * ALIGN * 4)
        self.shard_numel = self.padded // world_size
        alloc = alloc or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.persist: Optional[torch.Tensor] = None   # set by reshard(): the shard's own buffer
        # ``param_alloc``: a different home for the full parameter vector than for the gradients
        # (a unit that is about to be resharded must not take peer-visible memory for it)
        self.flat_param = (param_alloc or alloc)(self.padded, self.dtype, self.device)
        self.flat_grad = alloc(self.padded, self.dtype, self.device)
        for p, o in zip(params, offs):
            view = self.flat_param[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.flat_grad[o:o + p.numel()].view(p.shape)
            p.grad_accumulate = False
            p.flat_unit = self
        lo = rank * self.shard_numel
        self.shard_range = (lo, lo + self.shard_numel)
        # optimizer state for this rank's shard
        self.master = self.flat_param[lo:lo + self.shard_numel].float()
        self.exp_avg = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)

    # views of this rank's shard inside the full buffers
    def param_shard(self) -> torch.Tensor:
        if self.persist is not None:
            return self.persist
        lo, hi = self.shard_range
        return self.flat_param[lo:hi]

    def bind_storage(self, buf: torch.Tensor) -> None:
        """Points the full flat vector, and every parameter view, at ``buf`` (at least ``padded``
        elements).  The contents are whatever ``buf`` holds."""
        self.flat_param = buf[: self.padded]
        for p, o in zip(self.params, self.offsets):
            p.data = self.flat_param[o:o + p.numel()].view(p.shape)

    def reshard(self, slot: torch.Tensor, shard_alloc=None) -> None:
        """Gives up the unit's own full parameter buffer: this rank's shard moves to a buffer of
        its own (``persist``; from ``shard_alloc`` when the shard has to be peer-visible), and the
        full vector lives in ``slot``, a buffer shared with other units that only holds this
        unit's parameters while an engine has gathered them there."""
        lo, hi = self.shard_range
        if shard_alloc is None:
            self.persist = self.flat_param[lo:hi].clone()
        else:
            self.persist = shard_alloc(self.shard_numel, self.dtype, self.device)
            self.persist.copy_(self.flat_param[lo:hi])
        self.bind_storage(slot)

    def grad_shard(self) -> torch.Tensor:
        lo, hi = self.shard_range
        return self.flat_grad[lo:hi]

    def begin_step(self) -> None:
        """Next backward overwrites (rather than accumulates into) the gradient arena."""
        for p in self.params:
            p.grad_accumulate = False

    def collect_stray_grads(self) -> None:
        """Parameters whose gradient came through plain autograd (``p.grad``) are copied into the
        arena so that the arena is the single source of truth."""
        for p in self.params:
            if p.grad is not None:
                if p.grad_accumulate:
                    p.main_grad.add_(p.grad)
                else:
                    p.main_grad.copy_(p.grad)
                p.grad_accumulate = True
                p.grad = None

    def named_views(self, module_names: Dict[nn.Parameter, str]):
        return [(module_names[p], p) for p in self.params]


def build_units(model: nn.Module, unit_roots: List[tuple], world_size: int = 1, rank: int = 0,
                alloc=None, param_alloc_for: Optional[Callable[[str], Optional[Callable]]] = None) -> List[FlatUnit]:
    """``unit_roots`` is a list of ``(name, [modules or parameters])``; every model parameter
    must be covered exactly once."""
    seen = set()
    units = []
    for name, members in unit_roots:
        ps = []
        for m in members:
            it = [m] if isinstance(m, nn.Parameter) else list(m.parameters())
            for p in it:
                if id(p) not in seen:
                    seen.add(id(p))
                    ps.append(p)
        units.append(FlatUnit(name, ps, world_size, rank, alloc,
                              param_alloc_for(name) if param_alloc_for is not None else None))
    missing = [n for n, p in model.named_parameters() if id(p) not in seen]
    if missing:
        raise ValueError(f"parameters not assigned to a flat unit: {missing[:5]}")
    return units


def default_units(model: nn.Module) -> List[tuple]:
    """Embeddings | one unit per entry of ``model.blocks`` | everything else (final norm, head)."""
    roots = []
    blocks = getattr(model, "blocks", None)
    block_params = set()
    if blocks is not None:
        for b in blocks:
            for p in b.parameters():
                block_params.add(id(p))
    emb = [p for n, p in model.named_parameters()
           if id(p) not in block_params and ("emb" in n.split(".")[0])]
    if emb:
        roots.append(("embeddings", emb))
    if blocks is not None:
        for i, b in enumerate(blocks):
            roots.append((f"blocks.{i}", [b]))
    emb_ids = {id(p) for p in emb}
    rest = [p for n, p in model.named_parameters()
            if id(p) not in block_params and id(p) not in emb_ids]
    if rest:
        roots.append(("tail", rest))
    return roots
