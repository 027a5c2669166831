"""Times the fused FSDP communication kernels against NCCL + the flat Adam kernel on one sharding
unit (run under torchrun, one rank per GPU):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/bench_fused_comm.py

CUDA-event timing on the launching stream, max over ranks, 3 warm-ups; the unit (default 100M bf16
parameters, i.e. 200 MB of gradients) is larger than the 126 MB L2.
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
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
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
    P = int(os.environ.get("UNIT_NUMEL", str(100 * 1024 * 1024))) // (8 * world) * (8 * world)
    S = P // world
    arena = SymmArena(4 * P + (128 << 20))
    g = arena.alloc_flat(P, torch.bfloat16); w = arena.alloc_flat(P, torch.bfloat16)
    g.normal_(); w.normal_()
    master = w[rank * S:(rank + 1) * S].float(); m = torch.zeros_like(master); v = torch.zeros_like(master)
    gf, pf = arena.alloc_flags(world), arena.alloc_flags(world)
    cnt = arena.alloc_local_ints(1)
    arena.barrier()
    epoch = [0]
    res = {}
    for threads_ctas in [(64, 16), (148, 32), (296, 148)]:
        rs_ctas, ag_ctas = threads_ctas

        def rs():
            epoch[0] += 1
            fused_ops.rs_adam(arena, torch.bfloat16, g.arena_offset, w.arena_offset, rank * S, S, master, m, v,
                              lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1,
                              adamw=False, grad_flags_off=gf, param_flags_off=pf, epoch=epoch[0],
                              done_counter=cnt, ctas=rs_ctas)

        def ag():
            # the flags of the last rs() epoch are already set: this times the copy alone
            fused_ops.all_gather(arena, w.arena_offset, S * 2, src_flags_off=pf, epoch=epoch[0], ctas=ag_ctas)

        res[f"fused rs_adam ctas={rs_ctas}"] = timed(rs)
        res[f"fused all_gather ctas={ag_ctas}"] = timed(ag)
    # ---- all-reduce + unscale + non-finite flag (one data-parallel gradient bucket of 25 MB)
    nb = (25 << 20) // 2 // (8 * world) * (8 * world)
    bucket, _ = arena.alloc(nb, torch.float16)
    bucket.normal_()
    ef, xf, nf = arena.alloc_flags(world), arena.alloc_flags(world), arena.alloc_flags(world)
    cnt_ar = arena.alloc_local_ints(1)
    found = torch.zeros(1, dtype=torch.int32, device=dev)
    inv = torch.full((), 1.0 / 1024.0, device=dev)
    ar_epoch = [0]
    arena.barrier()

    def fused_ar():
        ar_epoch[0] += 1
        fused_ops.allreduce_unscale(arena, bucket, enter_flags_off=ef, exit_flags_off=xf, inf_flags_off=nf,
                                    epoch=ar_epoch[0], inv_scale=inv, extra_scale=1.0 / world, found_inf=found,
                                    done_counter=cnt_ar, ctas=32)

    def nccl_ar():
        dist.all_reduce(bucket)
        bucket.mul_(inv / world)
        torch.isfinite(bucket).all()

    res["fused allreduce+unscale 25MB"] = timed(fused_ar)
    res["nccl all_reduce + unscale + isfinite 25MB"] = timed(nccl_ar)
    # ---- decode-sized all-reduce (one-shot kernel, partial sums already in the arena) against NCCL
    os_bufs = [arena.alloc(64 * 4096, torch.bfloat16)[0] for _ in range(2)]
    os_flags = arena.alloc_flags(world)
    os_epoch = [0]
    arena.barrier()
    small = {}
    for kb in (8, 16, 32, 64, 256, 512):
        n = kb * 1024 // 2
        outp = torch.empty(n, dtype=torch.bfloat16, device=dev)
        resd = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        tmp = torch.zeros(n, dtype=torch.bfloat16, device=dev)

        def oneshot():
            os_epoch[0] += 1
            fused_ops.oneshot_allreduce(arena, os_bufs[os_epoch[0] & 1][:n], outp, flags_off=os_flags,
                                        epoch=os_epoch[0], residual=resd)

        def nccl_small():
            dist.all_reduce(tmp)
            torch.add(resd, tmp, out=outp)

        small[kb] = (timed(oneshot, iters=20), timed(nccl_small, iters=20))
    shard = torch.empty(S, dtype=torch.bfloat16, device=dev)
    res["nccl reduce_scatter"] = timed(lambda: dist.reduce_scatter_tensor(shard, g, op=dist.ReduceOp.AVG))
    res["adam_flat (shard)"] = timed(lambda: native.adam_flat(shard, master, m, v, w[rank * S:(rank + 1) * S],
                                                              lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                                              weight_decay=0.0, step=1, adamw=False))
    res["nccl all_gather"] = timed(lambda: dist.all_gather_into_tensor(w, w[rank * S:(rank + 1) * S]))
    if rank == 0:
        print(f"unit {P / 1e6:.0f}M bf16 params, world {world}, status {native.read_status()}")
        peer_bytes = (world - 1) * S * 2
        for k, t in res.items():
            print(f"  {k:44s} {t * 1e3:9.1f} us   ({peer_bytes / t / 1e6:7.1f} GB/s of peer traffic per GPU)")
        print("  decode all-reduce + residual add, latency in us (one-shot kernel | NCCL all_reduce + add):")
        for kb, (a_us, b_us) in small.items():
            print(f"    {kb:4d} KB   {a_us * 1e3:7.1f} | {b_us * 1e3:7.1f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
