"""XOR MLP: Module / Linear / Adam / mse_loss, then a safetensors save-load round trip
(the reference's rumus/tests/mlp_test.rs).  Runs on CPU or, with --cuda, on the GPU kernels."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tempfile

import torch

import rumus_b200.nn as nn
from rumus_b200.io import load_into, save_safetensors
from rumus_b200.ops import functional as F
from rumus_b200.optim import Adam


class XorMlp(nn.Module):
    def __init__(self):
        super().__init__()
        self.hidden = nn.Linear(2, 8)      # weight is [in, out], as in the reference
        self.output = nn.Linear(8, 1)

    def forward(self, x):
        return self.output(F.relu(self.hidden(x)))


def main():
    dev = "cuda" if "--cuda" in sys.argv and torch.cuda.is_available() else "cpu"
    torch.manual_seed(0)
    x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]], device=dev)
    y = torch.tensor([[0.], [1.], [1.], [0.]], device=dev)
    model = XorMlp().to(dev)
    opt = Adam(model.parameters(), lr=0.01)
    for step in range(1000):
        opt.zero_grad()
        loss = F.mse_loss(model(x), y)
        loss.backward()
        opt.step()
        if loss.item() < 0.01:
            break
    print(f"step {step}: mse {loss.item():.4f}; predictions {model(x).flatten().tolist()}")
    with tempfile.NamedTemporaryFile(suffix=".safetensors") as f:
        save_safetensors(model.state_dict(), f.name)
        clone = XorMlp().to(dev)
        load_into(clone, f.name)
    assert torch.equal(model(x), clone(x))
    print("checkpoint round trip: exact")


if __name__ == "__main__":
    main()
