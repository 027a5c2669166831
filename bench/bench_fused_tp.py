"""Times the fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter) against
NCCL collectives + the plain GEMM on Llama-7B layer shapes, and the FSDP form of the first (a whole
flat parameter unit gathered by the kernel that multiplies by the unit's first weight) on a
GPT-1.3B block (run under torchrun):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/bench_fused_tp.py

CUDA-event timing, max over ranks, 3 warm-ups, L2 flushed between iterations.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rumus_b200.ops import native  # noqa: E402
from rumus_b200.parallel import fused_ops  # noqa: E402
from rumus_b200.parallel.symm import SymmArena  # noqa: E402


def timed(fn, iters=8, warm=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    # started directly (no launcher) this is a group of one rank: the kernels then run their full
    # code path against this GPU's own buffers, which is the case to capture under a profiler
    os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29517")
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    M = int(os.environ.get("TOKENS", "8192")); d = 4096; ffn = 11008 // world // 128 * 128
    Ml = M // world
    arena = SymmArena(1 << 30)
    res = []
    # ---- column-parallel: x [M/W, d] gathered, w [d, ffn]
    x_local = (torch.randn(Ml, d, device=dev) * 0.5).bfloat16()
    w1 = (torch.randn(d, ffn, device=dev) * 0.02).bfloat16()
    stage, stage_off = arena.alloc_bytes(M * d * 2)
    sv = stage.view(torch.bfloat16).view(M, d)
    chunk_flags = arena.alloc_local_ints(256)
    aflags = arena.alloc_flags(world)
    x_full = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
    out1 = torch.empty(M, ffn, device=dev, dtype=torch.bfloat16)
    arena.barrier()
    epoch = [0]
    flops1 = 2.0 * M * d * ffn
    for chunk_kb, ncopy in [(1024, 16), (256, 16), (256, 32), (512, 8)]:
        def fused():
            epoch[0] += 1
            sv[rank * Ml:(rank + 1) * Ml].copy_(x_local)
            fused_ops.signal_peers(arena, aflags, epoch[0])
            fused_ops.ag_gemm(arena, buf_off=stage_off, shard_bytes=Ml * d * 2, chunk_flags=chunk_flags,
                              chunk_bytes=chunk_kb * 1024, epoch=epoch[0], gather_a=True, operand_off=0,
                              other=w1, M=M, N=ffn, K=d, out=out1, src_flags_off=aflags,
                              n_copy_ctas=ncopy)
        res.append((f"ag_gemm fused chunk={chunk_kb}K copy_ctas={ncopy}", timed(fused), flops1))

    def nccl1():
        dist.all_gather_into_tensor(x_full, x_local)
        native.gemm(x_full, w1, out=out1)
    res.append(("all_gather + gemm (nccl)", timed(nccl1), flops1))
    res.append(("gemm alone", timed(lambda: native.gemm(x_full, w1, out=out1)), flops1))
    # ---- row-parallel: a [M, ffn] . w2 [ffn, d] -> reduce-scatter rows
    a2 = (torch.randn(M, ffn, device=dev) * 0.5).bfloat16()
    w2 = (torch.randn(ffn, d, device=dev) * 0.02).bfloat16()
    part, part_off = arena.alloc_bytes(M * d * 2)
    ntiles = (M // 128) * ((d + 255) // 256)
    tflags = arena.alloc_flags(ntiles * world)
    tcount = arena.alloc_local_ints(ntiles)
    out2 = torch.empty(Ml, d, device=dev, dtype=torch.bfloat16)
    full2 = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
    arena.barrier()
    ep2 = [0]
    flops2 = 2.0 * M * d * ffn
    for nred in (0, 32):
        def fused2():
            ep2[0] += 1
            fused_ops.gemm_rs(arena, a2, w2, partial_off=part_off, tile_flags_off=tflags,
                              tile_counters=tcount, epoch=ep2[0], out=out2, n_reduce_ctas=nred)
        res.append((f"gemm_rs fused reduce_ctas={nred}", timed(fused2), flops2))

    # push form: the epilogue stores every tile into the owner's slot for this rank, a local pass sums the slots
    slot_sets = [part_off, arena.alloc_bytes(M * d * 2)[1]]
    pflags = arena.alloc_flags(world)
    pcount = arena.alloc_local_ints(world)
    torch.cuda.synchronize()
    arena.barrier()
    ep4 = [0]

    def fused_push():
        ep4[0] += 1
        fused_ops.gemm_rs_push(arena, a2, w2, slots_off=slot_sets[ep4[0] & 1], done_flags_off=pflags,
                               owner_counters=pcount, epoch=ep4[0], out=out2)
    res.append(("gemm_rs fused, pushed from the epilogue", timed(fused_push), flops2))

    def nccl2():
        native.gemm(a2, w2, out=full2)
        dist.reduce_scatter_tensor(out2, full2)
    res.append(("gemm + reduce_scatter (nccl)", timed(nccl2), flops2))
    res.append(("gemm alone", timed(lambda: native.gemm(a2, w2, out=full2)), flops2))
    # ---- FSDP unit: the flat parameter vector of one GPT-1.3B block (d 2048: 12 d^2 + 13 d values), sharded
    # evenly; the kernel gathers all of it and multiplies 8 x 2048 tokens by the qkv weight that sits in it
    dg, tok = 2048, 16384
    pad = 2 * dg                                                   # ln1 weight and bias come first
    unit = 12 * dg * dg + 13 * dg
    flat_n = (unit + world * 1024 - 1) // (world * 1024) * world * 1024
    Sb = flat_n // world
    flat, flat_off = arena.alloc(flat_n, torch.bfloat16)
    shard = (torch.randn(Sb, device=dev) * 0.02).bfloat16()
    flat_full = torch.empty(flat_n, device=dev, dtype=torch.bfloat16)
    xa = (torch.randn(tok, dg, device=dev) * 0.5).bfloat16()
    outq = torch.empty(tok, 3 * dg, device=dev, dtype=torch.bfloat16)
    bflags = arena.alloc_flags(world)
    arena.barrier()
    ep3 = [0]
    flops3 = 2.0 * tok * dg * 3 * dg
    for chunk_kb, ncopy in [(1024, 16), (1024, 32), (2048, 24)]:
        def fused3():
            ep3[0] += 1
            flat[rank * Sb:(rank + 1) * Sb].copy_(shard)
            fused_ops.signal_peers(arena, bflags, ep3[0])
            fused_ops.ag_gemm(arena, buf_off=flat_off, shard_bytes=Sb * 2, chunk_flags=chunk_flags,
                              chunk_bytes=chunk_kb * 1024, epoch=ep3[0], gather_a=False, operand_off=pad * 2,
                              other=xa, M=tok, N=3 * dg, K=dg, out=outq, src_flags_off=bflags,
                              n_copy_ctas=ncopy)
        res.append((f"fsdp unit gather+qkv fused chunk={chunk_kb}K copy_ctas={ncopy}", timed(fused3), flops3))

    def nccl3():
        dist.all_gather_into_tensor(flat_full, shard)
        native.gemm(xa, flat_full[pad:pad + dg * 3 * dg].view(dg, 3 * dg), out=outq)
    res.append((f"fsdp unit all_gather ({flat_n * 2 >> 20} MB) + qkv gemm (nccl)", timed(nccl3), flops3))
    res.append(("qkv gemm alone", timed(lambda: native.gemm(xa, flat_full[pad:pad + dg * 3 * dg].view(dg, 3 * dg),
                                                            out=outq)), flops3))
    if rank == 0:
        print(f"tokens {M}, d {d}, ffn/rank {ffn}, world {world}, status {native.read_status()}")
        for k, t, fl in res:
            print(f"  {k:60s} {t * 1e3:9.1f} us  {fl / t / 1e9:7.0f} TFLOP/s")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
