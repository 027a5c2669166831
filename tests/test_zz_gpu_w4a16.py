"""Fused W4A16 tcgen05 GEMM (``csrc/kernels/w4a16_gemm.cu``) against the dequantised fp32 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("scale_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("M,K,N", [(9, 256, 128),        # one tile, one K slice of 4 blocks
                                   (16, 4096, 512),      # K split across CTAs, fp32 workspace
                                   (33, 1160, 520),      # K padded to the group, N not a multiple of 128
                                   (128, 1024, 256)])    # the largest batch (UMMA N = 128)
@pytest.mark.parametrize("two_pass", [False, True])
def test_w4a16_matches_dequantised_product(dtype, scale_dtype, M, K, N, two_pass, monkeypatch):
    # two_pass: workspace cleared before and converted after the launch by separate kernels; default:
    # the CTA that adds a tile's last K slice converts it and restores the zeroed workspace
    monkeypatch.setenv("RB_W4A16_TWO_PASS", "1" if two_pass else "0")
    from rumus_b200.nn.quant import QuantizedTensor
    from rumus_b200.ops import native
    from rumus_b200.ops import quant_cuda as Q
    torch.manual_seed(M + K + N)
    w = torch.randn(K, N) * 0.05
    q = QuantizedTensor.from_f32(w, 128, scale_dtype).to("cuda")
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dtype)
    bias = torch.randn(N, device="cuda").to(dtype)
    y = Q.int4_matmul_fused(x, q, bias)
    assert y is not None
    ref = x.float() @ q.dequantize(torch.float32) + bias.float()
    assert native.read_status() == 0
    assert _rel(y, ref) < 1.5e-2, _rel(y, ref)
    # the shared workspace is zero again after a launch: the same call gives the same answer
    y_again = Q.int4_matmul_fused(x, q, bias)
    assert _rel(y_again, y) < 1e-3
    # rows are independent: a one-row change only moves that row
    x2 = x.clone()
    x2[M // 2] += 1.0
    y2 = Q.int4_matmul_fused(x2, q, bias)
    same = torch.ones(M, dtype=torch.bool, device="cuda")
    same[M // 2] = False
    assert torch.equal(y2[same], y[same]) or _rel(y2[same], y[same]) < 1e-3   # split-K atomics reorder sums
