"""FSDP with parameters resharded between uses, on GPUs (run under torchrun, one rank per GPU):
the resident flow and the resharded flow must give the same losses and weights, in the fused mode
(shards pulled by ``shard_gather_kernel``) and in the NCCL mode."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from rumus_b200.models import GPT, GPTConfig  # noqa: E402
from rumus_b200.ops import native  # noqa: E402
from rumus_b200.parallel import FSDP  # noqa: E402


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    native.lib().rb_init_device()
    cfg = GPTConfig(vocab_size=1024, seq_len=128, d_model=256, num_heads=2, num_layers=5, ffn_dim=512)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, cfg.vocab_size, (4, world * 2, cfg.seq_len + 1), generator=g)

    def run(mode, reshard):
        model = GPT(cfg, device=dev, dtype=torch.bfloat16)
        model.init_weights(0.02, seed=0)
        eng = FSDP(model, lr=1e-3, mode=mode, reshard_after_forward=reshard)
        losses = []
        for step in range(4):
            tok = data[step, rank * 2:(rank + 1) * 2].to(dev)
            eng.zero_grad()
            loss = model(tok[:, :-1], tok[:, 1:])
            loss.backward()
            eng.step()
            losses.append(loss.item())
        torch.cuda.synchronize()
        with eng.summon_full_params():
            sd = {k: v.detach().float().clone() for k, v in model.state_dict().items()}
        return losses, sd, eng.param_bytes()

    ok = True
    for mode in ("nccl", "fused"):
        l0, sd0, b0 = run(mode, False)
        l1, sd1, b1 = run(mode, True)
        worst = max((sd0[k] - sd1[k]).abs().max().item() for k in sd0)
        same = l0 == l1 and worst == 0.0 and b1 < b0
        if rank == 0:
            print(f"{mode}: losses {l0} vs {l1}; max weight diff {worst}; parameter bytes {b0} -> {b1}")
        ok = ok and same
    assert native.read_status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    if rank == 0 and flag.item() == 1:
        print("ALL RESHARD CHECKS PASSED")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
