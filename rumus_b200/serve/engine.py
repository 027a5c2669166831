"""Continuous-batching inference engine for Llama-style models with INT4 (AWQ-layout) weights,
a paged KV cache and tensor parallelism.

The reference server (rumus-serve/src/{scheduler,gpu_worker,model}.rs) batches statically under a
deadline around a mock model.  Here:

* requests join and leave between steps (C++ scheduler + block allocator,
  ``csrc/serve/kv_scheduler.cpp``): each step decodes one token for every running sequence and
  spends the rest of the token budget on prompt chunks of waiting sequences;
* weights are INT4 group-128 with fp16 scales, sharded Megatron-style across the TP group
  (qkv / gate-up by output columns, out-proj / down by input rows on group boundaries);
  decode uses the streaming GEMV kernel, prefill the dequant + tcgen05 GEMM path;
* attention reads and writes a block-paged KV cache (``csrc/kernels/paged_attention.cu``); whole
  prompts run through the FlashAttention forward kernel;
* the two partial-sum reductions per layer are all-reduces over the TP group (fused arena kernel
  or NCCL).
"""
from __future__ import annotations

import ctypes
import math
import os
import time
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig
from ..utils.metrics import trace_range
from ..nn.quant import QuantizedTensor, qmatmul_int4
from ..ops import _lib, functional as F, native
from ..ops._lib import check, count_launch, ptr, stream_ptr

P, LL, I, Fl = c_void_p, c_longlong, c_int, c_float
native.register_signature("rb_paged_decode_splits", [I])
native.register_signature("rb_paged_decode_attn", [I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, Fl, P])
native.register_signature("rb_kv_append", [I, P, P, LL, P, P, P, I, I, P])
native.register_signature("rb_paged_decode_attn_hm", [I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, Fl, P])
native.register_signature("rb_kv_append_hm", [I, P, P, LL, P, P, P, I, I, I, I, P])
native.register_signature("rb_argmax", [I, P, LL, I, I, P, P, P])


# --------------------------------------------------------------------------- host scheduler
class Scheduler:
    """ctypes face of the C++ continuous-batching scheduler / block allocator."""

    def __init__(self, num_blocks: int, block_size: int, max_batch: int, token_budget: int):
        L = _lib.host_lib()
        L.rbs_create.restype = c_void_p
        L.rbs_create.argtypes = [c_int] * 4
        L.rbs_destroy.argtypes = [c_void_p]
        L.rbs_add_request.argtypes = [c_void_p, c_longlong, c_int, c_int]
        L.rbs_schedule.argtypes = [c_void_p] + [c_void_p] * 6 + [c_int]
        L.rbs_commit.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                 c_void_p, c_int]
        L.rbs_block_table.argtypes = [c_void_p, c_longlong, c_void_p, c_int]
        L.rbs_block_tables.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]
        L.rbs_context_len.argtypes = [c_void_p, c_longlong]
        L.rbs_abort.argtypes = [c_void_p, c_longlong]
        for n in ("rbs_num_free_blocks", "rbs_num_waiting", "rbs_num_running"):
            getattr(L, n).argtypes = [c_void_p]
        L.rbs_num_preemptions.restype = c_longlong
        L.rbs_num_preemptions.argtypes = [c_void_p]
        self.L = L
        self.h = c_void_p(L.rbs_create(num_blocks, block_size, max_batch, token_budget))
        self.cap = max(max_batch, 64) * 4
        self.block_size = block_size

    def __del__(self):
        try:
            self.L.rbs_destroy(self.h)
        except Exception:
            pass

    def add(self, rid: int, prompt_len: int, max_new: int) -> int:
        return self.L.rbs_add_request(self.h, rid, prompt_len, max_new)

    def schedule(self):
        cap = self.cap
        dec = (c_longlong * cap)(); pre = (c_longlong * cap)()
        ps = (c_int * cap)(); pl = (c_int * cap)()
        nd, npf = c_int(0), c_int(0)
        self.L.rbs_schedule(self.h, dec, ctypes.byref(nd), pre, ps, pl, ctypes.byref(npf), cap)
        return ([dec[i] for i in range(nd.value)],
                [(pre[i], ps[i], pl[i]) for i in range(npf.value)])

    def commit(self, decode_ids, prefills, eos_ids=()):
        cap = self.cap
        dec = (c_longlong * max(1, len(decode_ids)))(*decode_ids)
        pre = (c_longlong * max(1, len(prefills)))(*[p[0] for p in prefills])
        pl = (c_int * max(1, len(prefills)))(*[p[2] for p in prefills])
        eos = (c_longlong * max(1, len(eos_ids)))(*eos_ids)
        fin = (c_longlong * cap)()
        n = self.L.rbs_commit(self.h, dec, len(decode_ids), pre, pl, len(prefills), eos, len(eos_ids),
                              fin, cap)
        return [fin[i] for i in range(n)]

    def block_table(self, rid: int, max_blocks: int) -> List[int]:
        out = (c_int * max_blocks)()
        n = self.L.rbs_block_table(self.h, rid, out, max_blocks)
        return [out[i] for i in range(max(0, min(n, max_blocks)))]

    def block_tables(self, rids: List[int], max_blocks: int, pin: bool = False) -> torch.Tensor:
        """Block tables of several sequences as one int32 ``[len(rids), max_blocks]`` tensor (unused
        entries zero), filled by a single native call."""
        n = len(rids)
        out = torch.empty((n, max_blocks), dtype=torch.int32, pin_memory=pin)
        counts = (c_int * n)()
        ids = (c_longlong * n)(*rids)
        missing = self.L.rbs_block_tables(self.h, ids, n, c_void_p(out.data_ptr()), max_blocks, counts)
        if missing:
            raise KeyError(f"{missing} unknown sequence id(s) in {rids}")
        return out

    def context_len(self, rid: int) -> int:
        return self.L.rbs_context_len(self.h, rid)

    def free_blocks(self) -> int:
        return self.L.rbs_num_free_blocks(self.h)

    def num_waiting(self) -> int:
        return self.L.rbs_num_waiting(self.h)

    def num_running(self) -> int:
        return self.L.rbs_num_running(self.h)

    def preemptions(self) -> int:
        return int(self.L.rbs_num_preemptions(self.h))


# --------------------------------------------------------------------------- model
@dataclass
class ServeConfig:
    model: LlamaConfig
    group_size: int = 128
    block_size: int = 64
    num_blocks: int = 4096
    max_batch: int = 64
    token_budget: int = 4096
    dtype: torch.dtype = torch.bfloat16
    scale_dtype: torch.dtype = torch.float16
    comm_mode: str = "nccl"
    # KV cache layout: False = [blocks, block_size, Hkv, D] (a token's heads together), True =
    # [blocks, Hkv, block_size, D] (a head's tokens together: long contiguous reads in decode
    # attention).  Opt-in until measured on hardware.
    kv_head_major: bool = field(default_factory=lambda: os.environ.get("RB_KV_HEAD_MAJOR", "0") == "1")
    # Decode batches run as captured CUDA graphs (one per padded batch size and context bucket): a decode
    # step is ~450 small launches whose host cost exceeds their device time.  RB_SERVE_GRAPHS=0 disables.
    cuda_graphs: bool = field(default_factory=lambda: os.environ.get("RB_SERVE_GRAPHS", "1") == "1")


class _Layer:
    pass


class Int4LlamaShard:
    """This rank's shard of an INT4-quantised Llama: random-init weights generated per layer and
    quantised on the fly (``seed`` makes every rank draw the same full matrices before slicing)."""

    def __init__(self, cfg: ServeConfig, device, rank: int = 0, world: int = 1, seed: int = 0):
        m = cfg.model
        self.cfg, self.device, self.rank, self.world = cfg, device, rank, world
        assert m.num_heads % world == 0 and m.num_kv_heads % world == 0
        hd = m.d_model // m.num_heads
        self.hd = hd
        self.h_local, self.hkv_local = m.num_heads // world, m.num_kv_heads // world
        # row-parallel K splits must fall on quantisation-group boundaries: the FFN width is padded with
        # zero columns (gate, up) / zero rows (down) to a multiple of world x group size, which leaves the
        # function unchanged (silu(0) * 0 = 0 meets zero rows).  Llama-7B: 11008 -> 11264 at 4 and 8 ranks.
        step = world * cfg.group_size
        ffn_pad = (m.ffn_dim + step - 1) // step * step if world > 1 else m.ffn_dim
        ffn_local = ffn_pad // world
        self.ffn_padded = ffn_pad
        assert (self.h_local * hd) % cfg.group_size == 0 or world == 1
        # full matrices are drawn (same seed on every rank, so the slices fit together) and
        # quantised on the device the shard lives on
        gdev = device if torch.device(device).type == "cuda" else "cpu"
        g = torch.Generator(device=gdev).manual_seed(seed)
        std = 0.02

        def rnd(*shape):
            return torch.randn(*shape, generator=g, device=gdev) * std

        def q(w):
            return QuantizedTensor.from_f32(w.contiguous(), cfg.group_size, cfg.scale_dtype).to(device)

        self.emb = rnd(m.vocab_size, m.d_model).to(cfg.dtype).to(device)
        self.layers: List[_Layer] = []
        r, W = rank, world
        for _ in range(m.num_layers):
            L = _Layer()
            wq, wk, wv = rnd(m.d_model, m.num_heads * hd), rnd(m.d_model, m.num_kv_heads * hd), \
                rnd(m.d_model, m.num_kv_heads * hd)
            ql, kl = self.h_local * hd, self.hkv_local * hd
            L.qkv = q(torch.cat([wq[:, r * ql:(r + 1) * ql], wk[:, r * kl:(r + 1) * kl],
                                 wv[:, r * kl:(r + 1) * kl]], dim=1))
            wo = rnd(m.num_heads * hd, m.d_model)
            L.out = q(wo[r * ql:(r + 1) * ql])
            wg, wu = rnd(m.d_model, m.ffn_dim), rnd(m.d_model, m.ffn_dim)
            if ffn_pad != m.ffn_dim:
                wg = torch.nn.functional.pad(wg, (0, ffn_pad - m.ffn_dim))
                wu = torch.nn.functional.pad(wu, (0, ffn_pad - m.ffn_dim))
            L.gate_up = q(torch.cat([wg[:, r * ffn_local:(r + 1) * ffn_local],
                                     wu[:, r * ffn_local:(r + 1) * ffn_local]], dim=1))
            wd = rnd(m.ffn_dim, m.d_model)
            if ffn_pad != m.ffn_dim:
                wd = torch.nn.functional.pad(wd, (0, 0, 0, ffn_pad - m.ffn_dim))
            L.down = q(wd[r * ffn_local:(r + 1) * ffn_local])
            L.ln1 = torch.ones(m.d_model, dtype=cfg.dtype, device=device)
            L.ln2 = torch.ones(m.d_model, dtype=cfg.dtype, device=device)
            self.layers.append(L)
        self.ln_f = torch.ones(m.d_model, dtype=cfg.dtype, device=device)
        vloc = m.vocab_size // world
        self.vocab_local = vloc
        self.head = rnd(m.d_model, m.vocab_size)[:, r * vloc:(r + 1) * vloc].contiguous().to(cfg.dtype).to(device)


class PagedKVCache:
    def __init__(self, cfg: ServeConfig, hkv_local: int, hd: int, device):
        n, bs = cfg.num_blocks, cfg.block_size
        self.block_size = bs
        self.head_major = bool(cfg.kv_head_major)
        self.hkv, self.hd = hkv_local, hd
        shape = (n, hkv_local, bs, hd) if self.head_major else (n, bs, hkv_local, hd)
        self.k = [torch.zeros(shape, dtype=cfg.dtype, device=device) for _ in range(cfg.model.num_layers)]
        self.v = [torch.zeros(shape, dtype=cfg.dtype, device=device) for _ in range(cfg.model.num_layers)]

    def append(self, layer: int, k_src, v_src, slots):
        """k_src/v_src: [T, Hkv*D] row views (possibly strided); slots: int64 [T]."""
        kc, vc = self.k[layer], self.v[layer]
        row = self.hkv * self.hd
        if k_src.is_cuda:
            if self.head_major:
                check(native.lib().rb_kv_append_hm(native.dtype_code(kc.dtype), ptr(k_src), ptr(v_src),
                                                   k_src.stride(0), ptr(slots), ptr(kc), ptr(vc),
                                                   k_src.shape[0], self.hkv, self.hd, self.block_size,
                                                   stream_ptr()), "rb_kv_append_hm")
            else:
                check(native.lib().rb_kv_append(native.dtype_code(kc.dtype), ptr(k_src), ptr(v_src),
                                                k_src.stride(0), ptr(slots), ptr(kc), ptr(vc),
                                                k_src.shape[0], row, stream_ptr()), "rb_kv_append")
            count_launch()
        elif self.head_major:
            blk, off = slots // self.block_size, slots % self.block_size
            T = k_src.shape[0]
            kc[blk, :, off] = k_src.reshape(T, self.hkv, self.hd)
            vc[blk, :, off] = v_src.reshape(T, self.hkv, self.hd)
        else:
            kc.view(-1, row)[slots] = k_src
            vc.view(-1, row)[slots] = v_src

    def gather(self, layer: int, table: torch.Tensor, positions: torch.Tensor):
        """K and V ``[len(positions), Hkv, D]`` of logical token ``positions`` of the sequence whose
        block table is ``table``."""
        blk, off = table[positions // self.block_size], positions % self.block_size
        if self.head_major:
            return self.k[layer][blk, :, off], self.v[layer][blk, :, off]
        return self.k[layer][blk, off], self.v[layer][blk, off]


def paged_decode_attention(q, k_cache, v_cache, block_tables, ctx_lens, scale: float, max_ctx: int,
                           head_major: bool = False):
    """q [B, H, D]; returns [B, H, D].  ``head_major``: cache is [blocks, Hkv, block_size, D]."""
    B, H, D = q.shape
    Hkv = k_cache.shape[1] if head_major else k_cache.shape[2]
    bs = k_cache.shape[2] if head_major else k_cache.shape[1]
    if q.is_cuda:
        L = native.lib()
        splits = L.rb_paged_decode_splits(int(max_ctx))
        so = torch.empty((B, H, splits, D), dtype=torch.float32, device=q.device)
        sml = torch.empty((B, H, splits, 2), dtype=torch.float32, device=q.device)
        out = torch.empty_like(q)
        fn = L.rb_paged_decode_attn_hm if head_major else L.rb_paged_decode_attn
        check(fn(native.dtype_code(q.dtype), ptr(q), ptr(k_cache), ptr(v_cache),
                 ptr(block_tables), ptr(ctx_lens), ptr(out), ptr(so), ptr(sml), B, H,
                 Hkv, D, bs, block_tables.shape[1], splits,
                 float(scale), stream_ptr()), "rb_paged_decode_attn")
        count_launch(2)
        return out
    outs = []
    for b in range(B):
        n = int(ctx_lens[b])
        idx = torch.arange(n)
        blk = block_tables[b, idx // bs].long()
        if head_major:
            kk, vv = k_cache[blk, :, idx % bs].float(), v_cache[blk, :, idx % bs].float()
        else:
            kk, vv = k_cache[blk, idx % bs].float(), v_cache[blk, idx % bs].float()   # [n, Hkv, D]
        rep = H // Hkv
        kk, vv = kk.repeat_interleave(rep, 1), vv.repeat_interleave(rep, 1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), kk) * scale
        outs.append(torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv).to(q.dtype))
    return torch.stack(outs)


def greedy_sample(logits: torch.Tensor):
    """Row argmax -> (ids int64 [B], max values fp32 [B])."""
    if logits.is_cuda:
        B, V = logits.shape
        ids = torch.empty(B, dtype=torch.int64, device=logits.device)
        vals = torch.empty(B, dtype=torch.float32, device=logits.device)
        check(native.lib().rb_argmax(native.dtype_code(logits.dtype), ptr(logits), logits.stride(0), B, V,
                                     ptr(ids), ptr(vals), stream_ptr()), "rb_argmax")
        count_launch()
        return ids, vals
    vals, ids = logits.float().max(dim=-1)
    return ids, vals


def _rope(x, positions, heads, hd, theta):
    """x [T, heads*hd] rotated in place by absolute positions [T]."""
    T = x.shape[0]
    if x.is_cuda:
        native.rope_(x, T, 1, heads, hd, 0, theta, False, pos_ids=positions)
        return x
    xr = x.view(T, heads, hd).float()
    half = hd // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32) / hd)
    ang = positions.float()[:, None] * inv[None]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = xr[..., :half], xr[..., half:]
    x.copy_(torch.cat([a * cs - b * sn, b * cs + a * sn], -1).reshape(T, heads * hd).to(x.dtype))
    return x


@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new: int
    arrival: float = 0.0
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    output: List[int] = field(default_factory=list)


class Engine:
    # partial sums up to this size take the one-shot all-reduce (every rank reads all partials:
    # one flag round, latency bound); larger ones (long prompt chunks) are bandwidth bound and go
    # through NCCL's reduce-scatter / all-gather schedule
    ONESHOT_MAX_BYTES = 2 << 20
    # decode batches are padded to one of these sizes before they are captured / replayed
    GRAPH_BATCHES = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)

    def __init__(self, cfg: ServeConfig, device=None, group: Optional[dist.ProcessGroup] = None, seed: int = 0):
        self.cfg = cfg
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device or torch.device("cpu")
        self.model = Int4LlamaShard(cfg, self.device, self.rank, self.world, seed)
        self.cache = PagedKVCache(cfg, self.model.hkv_local, self.model.hd, self.device)
        self.sched = Scheduler(cfg.num_blocks, cfg.block_size, cfg.max_batch, cfg.token_budget)
        self.requests: Dict[int, Request] = {}
        self.max_blocks = (cfg.model.seq_len + 512 + cfg.block_size - 1) // cfg.block_size
        self.steps = 0
        self.tokens_out = 0
        self._ar = None
        self._graphs: Dict[tuple, object] = {}
        self._graph_pool = None
        self._capturing = False
        self._cap_k = 0
        self.graph_replays = 0
        if self.world > 1 and cfg.comm_mode == "fused" and self.device.type == "cuda":
            from ..parallel.symm import SymmArena
            n = cfg.token_budget * cfg.model.d_model
            esz = torch.empty((), dtype=cfg.dtype).element_size()
            self.arena = SymmArena(2 * n * esz + (1 << 20), group)
            # two partial-sum buffers used in turn (see csrc/comm/oneshot_allreduce.cu)
            self._ar_bufs = [self.arena.alloc(n, cfg.dtype)[0] for _ in range(2)]
            self._ar_flags = self.arena.alloc_flags(self.world)
            self._ar_epoch = 0
            # added on the device to the epochs of captured all-reduce launches (see _decode_graph)
            self._ar_gen = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.arena.barrier()
            self._ar = True

    # ------------------------------------------------------------------ requests
    def add_request(self, rid: int, prompt: List[int], max_new: int, arrival: Optional[float] = None) -> bool:
        if self.sched.add(rid, len(prompt), max_new) != 0:
            return False
        self.requests[rid] = Request(rid, list(prompt), max_new, arrival if arrival is not None else time.time())
        return True

    def has_work(self) -> bool:
        return self.sched.num_waiting() + self.sched.num_running() > 0

    # ------------------------------------------------------------------ row-parallel layer + all-reduce
    def _row_parallel(self, h: torch.Tensor, qw, residual: torch.Tensor) -> torch.Tensor:
        """``residual + sum over ranks of (h @ dequant(qw))``.  Fused mode: the matmul writes its
        partial result straight into a peer-visible buffer and ONE kernel does the flag round, the
        reduction over all ranks' partials and the residual add; NCCL mode: matmul, all-reduce, add."""
        if self.world == 1:
            return residual + qmatmul_int4(h, qw)
        if self._ar and h.shape[0] * qw.n * h.element_size() <= self.ONESHOT_MAX_BYTES:
            from ..ops.quant_cuda import int4_matmul
            from ..parallel import fused_ops
            T = h.shape[0]
            if self._capturing:
                # a captured launch keeps its arguments: its epoch is (device word) + k, k = its position in
                # the graph; the word is even at every replay, so buffer k & 1 matches the eager convention
                self._cap_k += 1
                epoch, base = self._cap_k, self._ar_gen
            else:
                self._ar_epoch += 1
                epoch, base = self._ar_epoch, None
            part = self._ar_bufs[epoch & 1][: T * qw.n].view(T, qw.n)
            int4_matmul(h, qw, out=part)
            out = torch.empty_like(residual)
            with trace_range("serve.oneshot_allreduce"):
                fused_ops.oneshot_allreduce(self.arena, part, out, flags_off=self._ar_flags,
                                            epoch=epoch, residual=residual.contiguous(), epoch_base=base)
            return out
        part = qmatmul_int4(h, qw)
        dist.all_reduce(part, group=self.group)
        return residual + part

    # ------------------------------------------------------------------ forward
    def _forward(self, tokens: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, attend):
        """tokens/positions/slots: [T].  ``attend(layer, q [T,H,D], k [T,Hkv,D], v) -> [T,H,D]``
        runs after this step's K/V were appended to the cache.  Returns hidden [T, d]."""
        m, md = self.cfg.model, self.model
        hd, H, Hkv = md.hd, md.h_local, md.hkv_local
        x = F.embedding(tokens, md.emb)
        T = x.shape[0]
        for li, L in enumerate(md.layers):
            h = F.rms_norm(x, L.ln1, m.rms_eps)
            qkv = qmatmul_int4(h, L.qkv)
            q = qkv[:, : H * hd]
            k = qkv[:, H * hd: (H + Hkv) * hd]
            v = qkv[:, (H + Hkv) * hd:]
            _rope(q, positions, H, hd, m.rope_theta)
            _rope(k, positions, Hkv, hd, m.rope_theta)
            self.cache.append(li, k, v, slots)
            o = attend(li, q.reshape(T, H, hd), k.reshape(T, Hkv, hd), v.reshape(T, Hkv, hd))
            x = self._row_parallel(o.reshape(T, H * hd).contiguous(), L.out, x)
            h2 = F.rms_norm(x, L.ln2, m.rms_eps)
            gu = qmatmul_int4(h2, L.gate_up)
            x = self._row_parallel(F.swiglu(gu), L.down, x)
        return F.rms_norm(x, md.ln_f, m.rms_eps)

    def _logits_argmax(self, hidden: torch.Tensor) -> torch.Tensor:
        md = self.model
        logits = native.gemm(hidden.contiguous(), md.head) if hidden.is_cuda else hidden @ md.head
        ids, vals = greedy_sample(logits)
        if self.world == 1:
            return ids
        ids = ids + self.rank * md.vocab_local
        allv = [torch.empty_like(vals) for _ in range(self.world)]
        alli = [torch.empty_like(ids) for _ in range(self.world)]
        dist.all_gather(allv, vals, group=self.group)
        dist.all_gather(alli, ids, group=self.group)
        best = torch.stack(allv).argmax(dim=0)
        return torch.stack(alli).gather(0, best[None]).squeeze(0)

    def _slots(self, rid: int, start: int, n: int) -> torch.Tensor:
        bs = self.cfg.block_size
        table = self.sched.block_table(rid, self.max_blocks)
        pos = torch.arange(start, start + n)
        blk = torch.tensor(table, dtype=torch.int64)[pos // bs]
        return (blk * bs + pos % bs).to(self.device)

    # ------------------------------------------------------------------ decode step as a CUDA graph
    def _capture_decode(self, Bp: int, ctx_bucket: int, scale: float):
        """Captures the decoder stack for a padded batch of ``Bp`` sequences whose contexts fit
        ``ctx_bucket`` tokens.  Inputs live in static device tensors; padded rows carry cache slot -1
        (the append kernel skips them), context length 1 and block table 0, and their outputs are ignored."""
        from types import SimpleNamespace
        dev = self.device
        st = SimpleNamespace(
            toks=torch.zeros(Bp, dtype=torch.int64, device=dev), pos=torch.zeros(Bp, dtype=torch.int64, device=dev),
            slots=torch.full((Bp,), -1, dtype=torch.int64, device=dev),
            tables=torch.zeros((Bp, self.max_blocks), dtype=torch.int32, device=dev),
            ctx=torch.ones(Bp, dtype=torch.int32, device=dev))

        def attend(li, q, k, v):
            return paged_decode_attention(q.contiguous(), self.cache.k[li], self.cache.v[li], st.tables, st.ctx,
                                          scale, ctx_bucket, head_major=self.cache.head_major)

        # one eager pass first, on a side stream: whatever the kernels set up lazily (function attributes,
        # workspaces, communicator channels) exists before the capture begins
        cur = torch.cuda.current_stream(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            self._forward(st.toks, st.pos, st.slots, attend)
        cur.wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        self._capturing, self._cap_k = True, 0
        try:
            with torch.cuda.graph(g, pool=self._graph_pool, capture_error_mode="thread_local"):
                st.hidden = self._forward(st.toks, st.pos, st.slots, attend)
        finally:
            self._capturing = False
        if self._graph_pool is None:
            self._graph_pool = g.pool()
        st.graph, st.n_allreduce = g, self._cap_k
        return st

    def warmup_graphs(self, max_ctx: Optional[int] = None) -> int:
        """Captures the decode graphs a run can meet (every padded batch size up to ``max_batch``, every
        context bucket up to ``max_ctx``) before traffic arrives, so that no request waits for a capture.
        Every tensor-parallel rank has to call it (the captures run collectives).  Returns how many."""
        if not (self.cfg.cuda_graphs and self.device.type == "cuda"):
            return 0
        scale = 1.0 / math.sqrt(self.model.hd)
        top = max_ctx or (self.cfg.model.seq_len + 512)
        n, cb = 0, 256
        while True:
            for Bp in self.GRAPH_BATCHES:
                if (Bp, cb) not in self._graphs:
                    self._graphs[(Bp, cb)] = self._capture_decode(Bp, cb, scale)
                    n += 1
                if Bp >= self.cfg.max_batch:
                    break
            if cb >= top:
                break
            cb *= 2
        return n

    def _decode_graph(self, B: int, last, ctx, slots_h: torch.Tensor, tables_h: torch.Tensor, scale: float):
        """Runs the decoder stack for this step's decode batch by replaying a captured graph; returns the
        hidden states ``[B, d]``, or None when the batch is larger than the largest captured size."""
        Bp = next((b for b in self.GRAPH_BATCHES if b >= B), None)
        if Bp is None:
            return None
        ctx_bucket = max(256, 1 << (max(ctx) - 1).bit_length())
        st = self._graphs.get((Bp, ctx_bucket))
        if st is None:
            st = self._graphs[(Bp, ctx_bucket)] = self._capture_decode(Bp, ctx_bucket, scale)
        pad = Bp - B
        st.toks.copy_(torch.tensor(list(last) + [0] * pad, dtype=torch.int64))
        st.pos.copy_(torch.tensor([c - 1 for c in ctx] + [0] * pad, dtype=torch.int64))
        st.ctx.copy_(torch.tensor(list(ctx) + [1] * pad, dtype=torch.int32))
        st.slots.copy_(torch.cat([slots_h.to(torch.int64), torch.full((pad,), -1, dtype=torch.int64)]))
        tp = torch.zeros((Bp, self.max_blocks), dtype=torch.int32)
        tp[:B] = tables_h.to(torch.int32)
        st.tables.copy_(tp)
        if self._ar and st.n_allreduce:
            if self._ar_epoch & 1:
                self._ar_epoch += 1          # every rank skips the same epoch number; flags only ever grow
            self._ar_gen.fill_(self._ar_epoch)
            self._ar_epoch += st.n_allreduce
        st.graph.replay()
        self.graph_replays += 1
        return st.hidden[:B]

    # ------------------------------------------------------------------ one engine step
    def step(self) -> List[int]:
        """Runs one scheduling step; returns the ids of requests that finished."""
        with trace_range("serve.schedule"):
            decode_ids, prefills = self.sched.schedule()
        if not decode_ids and not prefills:
            return []
        dev, scale = self.device, 1.0 / math.sqrt(self.model.hd)
        now_tokens: Dict[int, int] = {}
        # ---- prompt chunks (one forward per sequence; whole prompts use FlashAttention directly)
        for rid, start, n in prefills:
            req = self.requests[rid]
            seq = req.prompt + req.output   # a preempted sequence re-prefills what it had generated
            toks = torch.tensor(seq[start:start + n], dtype=torch.int64, device=dev)
            pos = torch.arange(start, start + n, dtype=torch.int64, device=dev)
            slots = self._slots(rid, start, n)
            table = torch.tensor(self.sched.block_table(rid, self.max_blocks), dtype=torch.int64, device=dev)

            def attend(li, q, k, v, start=start, n=n, table=table):
                if start == 0:
                    return F.flash_attention(q[None], k[None], v[None], True, scale)[0]
                # continuation chunk: keys/values of the prefix come from the paged cache
                idx = torch.arange(0, start + n, device=dev)
                bs = self.cfg.block_size
                kk, vv = self.cache.gather(li, table, idx)
                return F.flash_attention(q[None], kk[None], vv[None], True, scale)[0]

            with trace_range("serve.prefill_chunk"):
                hidden = self._forward(toks, pos, slots, attend)
            if start + n >= len(seq):
                now_tokens[rid] = int(self._logits_argmax(hidden[-1:])[0])
        # ---- decode batch
        if decode_ids:
            B = len(decode_ids)
            last = [self.requests[r].output[-1] if self.requests[r].output else self.requests[r].prompt[-1]
                    for r in decode_ids]
            ctx = [len(self.requests[r].prompt) + len(self.requests[r].output) for r in decode_ids]
            bs = self.cfg.block_size
            pin = dev.type == "cuda"
            tables_h = self.sched.block_tables(decode_ids, self.max_blocks, pin=pin)
            last_pos = torch.tensor(ctx, dtype=torch.int64) - 1
            # cache slot of each sequence's newest token: its block's id * block size + offset
            slots_h = (tables_h.gather(1, (last_pos // bs)[:, None]).squeeze(1).to(torch.int64) * bs
                       + last_pos % bs)
            with trace_range("serve.decode_batch"):
                hidden = None
                if self.cfg.cuda_graphs and dev.type == "cuda":
                    hidden = self._decode_graph(B, last, ctx, slots_h, tables_h, scale)
                if hidden is None:
                    toks = torch.tensor(last, dtype=torch.int64, device=dev)
                    pos = torch.tensor([c - 1 for c in ctx], dtype=torch.int64, device=dev)
                    tables = tables_h.to(dev, non_blocking=pin)
                    slots_t = slots_h.to(dev)
                    ctx_t = torch.tensor(ctx, dtype=torch.int32, device=dev)
                    max_ctx = max(ctx)

                    def attend_dec(li, q, k, v):
                        return paged_decode_attention(q.contiguous(), self.cache.k[li], self.cache.v[li], tables,
                                                      ctx_t, scale, max_ctx, head_major=self.cache.head_major)

                    hidden = self._forward(toks, pos, slots_t, attend_dec)
            ids = self._logits_argmax(hidden)
            for r, t in zip(decode_ids, ids.tolist()):
                now_tokens[r] = int(t)
        t_now = time.time()
        for rid, tok in now_tokens.items():
            req = self.requests[rid]
            if req.first_token_time is None:
                req.first_token_time = t_now
            req.output.append(tok)
            self.tokens_out += 1
        finished = self.sched.commit(decode_ids, prefills)
        for rid in finished:
            self.requests[rid].finish_time = t_now
        self.steps += 1
        return finished
