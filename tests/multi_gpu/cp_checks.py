"""Context-parallel attention on GPUs (run under torchrun, one rank per GPU): Ulysses all-to-all and
ring attention with the tcgen05 FlashAttention kernels per block, against full-sequence attention."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rumus_b200.ops import functional as F, native  # noqa: E402
from rumus_b200.parallel.cp import ring_attention, ulysses_attention  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    B, S, H, Hkv, D = 2, 256 * world, 2 * world, world, 128
    torch.manual_seed(3)
    q, k, v = [(torch.randn(B, S, h, D, device=dev) * 0.6).bfloat16() for h in (H, Hkv, Hkv)]
    w = torch.randn(B, S, H, D, device=dev).bfloat16()
    sl = slice(rank * S // world, (rank + 1) * S // world)
    for causal in (True, False):
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        o_ref = F.flash_attention(qr, kr, vr, causal)
        (o_ref.float() * w.float()).sum().backward()
        for name, fn in (("ulysses", ulysses_attention), ("ring", ring_attention)):
            ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
            o = fn(ql, kl, vl, causal)
            (o.float() * w[:, sl].float()).sum().backward()
            torch.cuda.synchronize()
            errs = [rel(o, o_ref[:, sl]), rel(ql.grad, qr.grad[:, sl]), rel(kl.grad, kr.grad[:, sl]),
                    rel(vl.grad, vr.grad[:, sl])]
            ok = all(e < 2e-2 for e in errs) and native.read_status() == 0
            print(f"[rank {rank}] {name} causal={causal}: " + " ".join(f"{e:.2e}" for e in errs) +
                  (" OK" if ok else " FAIL"), flush=True)
            if not ok:
                raise SystemExit(f"{name} failed")
    dist.barrier()
    if rank == 0:
        print("ALL CP CHECKS PASSED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
