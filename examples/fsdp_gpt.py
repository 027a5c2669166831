"""Fully sharded data-parallel training of a small GPT, one process per rank:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/fsdp_gpt.py

On GPUs the reduce-scatter + Adam and the all-gather are the fused peer-memory kernels
(``--mode nccl`` switches to NCCL collectives); without GPUs the same schedule runs on gloo ranks.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from rumus_b200.models import GPT, GPTConfig
from rumus_b200.parallel import FSDP


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo")
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    cfg = GPTConfig(vocab_size=512, seq_len=64, d_model=128, num_heads=1 if cuda else 4, num_layers=2, ffn_dim=512)
    model = GPT(cfg, device=dev, dtype=torch.bfloat16 if cuda else torch.float32)
    model.init_weights(0.02, seed=0)
    mode = "nccl" if "--mode=nccl" in sys.argv else None
    engine = FSDP(model, lr=3e-3, mode=mode)
    g = torch.Generator().manual_seed(100 + rank)
    for step in range(30):
        # a learnable stream: every sequence counts upwards from a random start
        start = torch.randint(0, cfg.vocab_size, (4, 1), generator=g)
        tok = ((start + torch.arange(cfg.seq_len + 1)[None]) % cfg.vocab_size).to(dev)
        engine.zero_grad()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        engine.step()
        if rank == 0 and step % 5 == 0:
            print(f"step {step}: loss {loss.item():.3f} ({engine.mode} mode, world {world})")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
