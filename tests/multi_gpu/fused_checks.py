"""Multi-GPU numerics of the fused collective kernels (run under torchrun, one rank per GPU).

Every fused path is compared with the same computation done with NCCL collectives + plain
PyTorch math on identical inputs.  Exits non-zero on any mismatch or device-side timeout.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rumus_b200.ops import native  # noqa: E402
from rumus_b200.parallel import fused_ops  # noqa: E402
from rumus_b200.parallel.symm import SymmArena  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def check(name, err, tol):
    ok = err < tol
    st = native.read_status()
    print(f"[rank {dist.get_rank()}] {name}: err={err:.3e} tol={tol:.1e} status={st} {'OK' if ok and st == 0 else 'FAIL'}",
          flush=True)
    if not ok or st != 0:
        raise SystemExit(f"{name} failed")


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    arena = SymmArena(1 << 30)
    torch.manual_seed(100 + rank)

    # ---------------- all-reduce + unscale + inf flag
    n = 8 * world * 4096 * 3
    buf, off = arena.alloc(n, torch.float16)
    src = (torch.randn(n, device=dev) * 4).half()
    buf.copy_(src)
    ref = src.float().clone()
    dist.all_reduce(ref)
    ref = ref * (1.0 / 128.0) / world
    ef, xf, nf = arena.alloc_flags(world), arena.alloc_flags(world), arena.alloc_flags(world)
    cnt = arena.alloc_local_ints(1)
    found = torch.zeros(1, dtype=torch.int32, device=dev)
    inv = torch.full((), 1.0 / 128.0, device=dev)
    arena.barrier()
    fused_ops.allreduce_unscale(arena, buf, enter_flags_off=ef, exit_flags_off=xf, inf_flags_off=nf,
                                epoch=1, inv_scale=inv, extra_scale=1.0 / world, found_inf=found,
                                done_counter=cnt)
    torch.cuda.synchronize()
    check("allreduce_unscale", rel(buf, ref), 2e-3)
    assert found.item() == 0
    # second round: rank 1 injects an inf -> every rank must see the flag
    buf.copy_(src)
    if rank == world - 1:
        buf[5] = float("inf")
    arena.barrier()
    fused_ops.allreduce_unscale(arena, buf, enter_flags_off=ef, exit_flags_off=xf, inf_flags_off=nf,
                                epoch=2, inv_scale=inv, extra_scale=1.0 / world, found_inf=found,
                                done_counter=cnt)
    torch.cuda.synchronize()
    assert found.item() == 1, "non-finite flag must reach every rank"
    print(f"[rank {rank}] allreduce inf flag OK", flush=True)

    # ---------------- rs_adam + all_gather vs NCCL reduce-scatter + reference Adam
    P = world * 8 * 1024 * 5
    S = P // world
    gbuf = arena.alloc_flat(P, torch.bfloat16); pbuf = arena.alloc_flat(P, torch.bfloat16)
    torch.manual_seed(7)
    full_init = torch.randn(P, device=dev)
    pbuf.copy_(full_init.bfloat16())
    master = pbuf[rank * S:(rank + 1) * S].float()
    m = torch.zeros(S, device=dev); v = torch.zeros(S, device=dev)
    rmaster, rm, rv = master.clone(), m.clone(), v.clone()
    gflags, pflags = arena.alloc_flags(world), arena.alloc_flags(world)
    cnt2 = arena.alloc_local_ints(1)
    arena.barrier()
    lr, b1, b2, eps = 1e-2, 0.9, 0.95, 1e-8
    for step in range(1, 4):
        torch.manual_seed(1000 * step + rank)
        g = torch.randn(P, device=dev).bfloat16()
        gbuf.copy_(g)
        gref = g.float().clone()
        dist.all_reduce(gref)
        gref = gref[rank * S:(rank + 1) * S] / world
        fused_ops.rs_adam(arena, torch.bfloat16, gbuf.arena_offset, pbuf.arena_offset, rank * S, S,
                          master, m, v, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=0.0,
                          step=step, adamw=False, grad_flags_off=gflags, param_flags_off=pflags,
                          epoch=step, done_counter=cnt2)
        fused_ops.all_gather(arena, pbuf.arena_offset, S * 2, src_flags_off=pflags, epoch=step)
        rm.mul_(b1).add_(gref, alpha=1 - b1); rv.mul_(b2).addcmul_(gref, gref, value=1 - b2)
        rmaster.sub_(lr * (rm / (1 - b1 ** step)) / ((rv / (1 - b2 ** step)).sqrt() + eps))
        torch.cuda.synchronize()
        full_ref = torch.empty(P, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full_ref, rmaster.bfloat16())
        check(f"rs_adam step {step} master", rel(master, rmaster), 1e-4)
        check(f"all_gather step {step}", rel(pbuf, full_ref), 1e-3)
        dist.barrier()

    # ---------------- ag_gemm (gather A rows) vs all_gather + matmul
    Ml, K, N = 256, 512, 768
    M = Ml * world
    stage, stage_off = arena.alloc_bytes(M * K * 2)
    chunk_flags = arena.alloc_local_ints(256)
    aflags = arena.alloc_flags(world)
    torch.manual_seed(50 + rank)
    x_local = (torch.randn(Ml, K, device=dev) * 0.5).bfloat16()
    torch.manual_seed(99)
    w = (torch.randn(K, N, device=dev) * 0.1).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    x_full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(x_full, x_local)
    ref_y = x_full.float() @ w.float() + bias.float()
    arena.barrier()
    for epoch, wmat in ((1, w), (2, w.t().contiguous().t())):
        sv = stage.view(torch.bfloat16).view(M, K)
        sv.zero_()
        sv[rank * Ml:(rank + 1) * Ml].copy_(x_local)
        fused_ops.signal_peers(arena, aflags, epoch)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fused_ops.ag_gemm(arena, buf_off=stage_off, shard_bytes=Ml * K * 2, chunk_flags=chunk_flags,
                          chunk_bytes=64 * 1024, epoch=epoch, gather_a=True, operand_off=0, other=wmat,
                          M=M, N=N, K=K, out=out, src_flags_off=aflags, bias=bias)
        torch.cuda.synchronize()
        check(f"ag_gemm gather_a (b layout {epoch})", rel(out, ref_y), 1e-2)
        check(f"ag_gemm staging {epoch}", rel(sv, x_full), 1e-6)
        arena.barrier()

    # ---------------- ag_gemm (gather B rows: FSDP weight slab inside a flat vector)
    Kb, Nb, Mb = 1024, 512, 640
    pad = 4096  # the weight does not start at the beginning of the flat vector
    flat_n = ((pad + Kb * Nb + world * 1024 - 1) // (world * 1024)) * world * 1024
    flat, flat_off = arena.alloc(flat_n, torch.bfloat16)
    torch.manual_seed(3)
    flat_ref = (torch.randn(flat_n, device=dev) * 0.1).bfloat16()
    Sb = flat_n // world
    flat.zero_()
    flat[rank * Sb:(rank + 1) * Sb].copy_(flat_ref[rank * Sb:(rank + 1) * Sb])
    bflags = arena.alloc_flags(world)
    torch.manual_seed(60 + rank)
    xa = (torch.randn(Mb, Kb, device=dev) * 0.5).bfloat16()
    wref = flat_ref[pad:pad + Kb * Nb].view(Kb, Nb)
    arena.barrier()
    fused_ops.signal_peers(arena, bflags, 3)
    outb = torch.empty(Mb, Nb, device=dev, dtype=torch.bfloat16)
    fused_ops.ag_gemm(arena, buf_off=flat_off, shard_bytes=Sb * 2, chunk_flags=chunk_flags,
                      chunk_bytes=32 * 1024, epoch=3, gather_a=False, operand_off=pad * 2, other=xa,
                      M=Mb, N=Nb, K=Kb, out=outb, src_flags_off=bflags)
    torch.cuda.synchronize()
    check("ag_gemm gather_b", rel(outb, xa.float() @ wref.float()), 1e-2)
    check("ag_gemm gather_b flat", rel(flat, flat_ref), 1e-6)
    arena.barrier()

    # ---------------- gemm_rs vs matmul + reduce_scatter
    Mr, Kr, Nr = 128 * world * 2, 384, 512
    part, part_off = arena.alloc_bytes(Mr * Nr * 2)
    ntiles = (Mr // 128) * ((Nr + 255) // 256)
    tflags = arena.alloc_flags(ntiles * world)
    tcount = arena.alloc_local_ints(ntiles)
    torch.manual_seed(70 + rank)
    ar = (torch.randn(Mr, Kr, device=dev) * 0.5).bfloat16()
    br = (torch.randn(Kr, Nr, device=dev) * 0.1).bfloat16()
    biasr = torch.randn(Nr, device=dev).bfloat16()
    full = ar.float() @ br.float()
    dist.all_reduce(full)
    ref_local = full[rank * (Mr // world):(rank + 1) * (Mr // world)] + biasr.float()
    arena.barrier()
    for epoch in (1, 2):
        outr = torch.empty(Mr // world, Nr, device=dev, dtype=torch.bfloat16)
        fused_ops.gemm_rs(arena, ar, br, partial_off=part_off, tile_flags_off=tflags,
                          tile_counters=tcount, epoch=epoch, out=outr, bias=biasr)
        torch.cuda.synchronize()
        check(f"gemm_rs epoch {epoch}", rel(outr, ref_local), 1.5e-2)
        arena.barrier()

    # residual added by the reducing owner
    resr = torch.randn(Mr // world, Nr, device=dev).bfloat16()
    outr = torch.empty(Mr // world, Nr, device=dev, dtype=torch.bfloat16)
    fused_ops.gemm_rs(arena, ar, br, partial_off=part_off, tile_flags_off=tflags,
                      tile_counters=tcount, epoch=3, out=outr, bias=biasr, residual=resr)
    torch.cuda.synchronize()
    check("gemm_rs + residual", rel(outr, ref_local + resr.float()), 1.5e-2)
    arena.barrier()

    # ---------------- gemm_rs, push form: four calls in a row over the two alternating slot sets, no barrier
    # between them (no rank may run ahead into slots a peer is still reading)
    slot_sets = [arena.alloc_bytes(Mr * Nr * 2)[1] for _ in range(2)]
    pflags = arena.alloc_flags(world)
    pcount = arena.alloc_local_ints(world)
    torch.cuda.synchronize()
    arena.barrier()
    outs_p = []
    for epoch in range(1, 5):
        outp = torch.empty(Mr // world, Nr, device=dev, dtype=torch.bfloat16)
        fused_ops.gemm_rs_push(arena, ar, br, slots_off=slot_sets[epoch & 1], done_flags_off=pflags,
                               owner_counters=pcount, epoch=epoch, out=outp, bias=biasr,
                               residual=resr if epoch % 2 == 0 else None)
        outs_p.append(outp)
    torch.cuda.synchronize()
    for epoch, outp in enumerate(outs_p, start=1):
        want_p = ref_local + (resr.float() if epoch % 2 == 0 else 0)
        check(f"gemm_rs_push call {epoch}", rel(outp, want_p), 1.5e-2)
    arena.barrier()

    # ---------------- one-shot all-reduce of decode-sized partial sums (+ residual), two buffers in turn
    T, d = 48, 4096
    bufs = [arena.alloc(128 * d, torch.bfloat16)[0] for _ in range(2)]
    oflags = arena.alloc_flags(world)
    arena.barrier()
    for epoch in range(1, 6):
        rows = T if epoch % 2 else 7
        torch.manual_seed(500 * epoch + rank)
        mine = (torch.randn(rows, d, device=dev) * 0.5).bfloat16()
        torch.manual_seed(77 + epoch)
        res = torch.randn(rows, d, device=dev).bfloat16()
        part_buf = bufs[epoch & 1][: rows * d].view(rows, d)
        part_buf.copy_(mine)
        want = mine.float().clone()
        dist.all_reduce(want)
        want = want + res.float()
        got = torch.empty_like(mine)
        fused_ops.oneshot_allreduce(arena, part_buf, got, flags_off=oflags, epoch=epoch, residual=res)
        torch.cuda.synchronize()
        check(f"oneshot_allreduce epoch {epoch}", rel(got, want), 1e-2)

    dist.barrier()
    if rank == 0:
        print("ALL FUSED CHECKS PASSED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
