"""Weight-only INT4 quantisation of a Linear layer (group 128, the reference's packing) and ONNX
export of a small model (rumus-vision/src/quant.rs, rumus/src/onnx/)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tempfile

import torch
import torch.nn as tnn

import rumus_b200.nn as nn
from rumus_b200.io.onnx_export import export_onnx


def main():
    torch.manual_seed(0)
    lin = nn.Linear(256, 64)
    q = nn.QLinear.from_linear(lin, group_size=128)
    x = torch.randn(4, 256)
    err = (q(x) - lin(x)).abs().max().item()
    packed = q.qweight.packed.numel() * 4 + q.qweight.scales.numel() * q.qweight.scales.element_size() * 2
    print(f"INT4 max abs error {err:.4f}; {lin.weight.numel() * 4} B fp32 -> {packed} B packed")
    model = tnn.Sequential(nn.Linear(8, 16), tnn.ReLU(), nn.Linear(16, 4))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mlp.onnx")
        export_onnx(model, [torch.randn(2, 8)], path)
        print(f"wrote {os.path.getsize(path)} bytes of ONNX (IR 9, opset 17)")


if __name__ == "__main__":
    main()
