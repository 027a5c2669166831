"""A two-layer GPT on a toy next-token task: Embedding / TransformerBlock / LayerNorm / AdamW /
cross-entropy and the Trainer helper (the reference's rumus/tests/transformer_test.rs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from rumus_b200.models import GPT, GPTConfig
from rumus_b200.optim import AdamW, CosineAnnealingLR
from rumus_b200.train import Trainer


def main():
    dev = "cuda" if "--cuda" in sys.argv and torch.cuda.is_available() else "cpu"
    cfg = GPTConfig(vocab_size=16, seq_len=12, d_model=32, num_heads=2, num_layers=2, ffn_dim=64)
    torch.manual_seed(0)
    model = GPT(cfg, device=dev)
    seq = (torch.arange(13, device=dev)[None] + torch.arange(8, device=dev)[:, None]) % 16   # counting task
    opt = AdamW(model.parameters(), lr=3e-3, weight_decay=0.01)
    sched = CosineAnnealingLR(3e-3, t_max=300, eta_min=3e-4)   # schedulers compute the LR, the caller applies it
    trainer = Trainer(opt)
    for step in range(300):
        loss = float(trainer.train_step(lambda: model(seq[:, :-1], seq[:, 1:])))
        sched.step()
        opt.set_lr(sched.get_lr())
    print(f"final cross-entropy {loss:.4f} (chance is {torch.log(torch.tensor(16.0)).item():.2f})")
    assert loss < 0.5


if __name__ == "__main__":
    main()
