"""Fused W8A16 tcgen05 GEMM (``csrc/kernels/w8a16_gemm.cu``) against the dequantised fp32 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bs", [32, 64, 128])
@pytest.mark.parametrize("M,K,N", [(1, 256, 128),         # one row, one tile, one K slice
                                   (16, 4096, 512),       # K split across CTAs
                                   (33, 1160, 520),       # K not a multiple of 64, N not a multiple of 128
                                   (128, 1024, 256),      # the largest batch of one launch
                                   (300, 512, 384)])      # several launches over row chunks
def test_w8a16_matches_dequantised_product(dtype, bs, M, K, N):
    from rumus_b200.nn.quant import dequantize_q8, quantize_q8
    from rumus_b200.ops import native
    from rumus_b200.ops import quant_cuda as Q
    torch.manual_seed(M + K + N + bs)
    w = torch.randn(K, N) * 0.05
    qc = quantize_q8(w, bs)
    from rumus_b200.nn.quant import Q8Tensor
    qg = Q8Tensor(qc.k, qc.n, qc.block_size, qc.data.cuda())
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dtype)
    bias = torch.randn(N, device="cuda").to(dtype)
    y = Q.q8_matmul_fused(x, qg, bias)
    assert y is not None
    ref = x.float() @ dequantize_q8(qc).cuda() + bias.float()
    assert native.read_status() == 0
    assert _rel(y, ref) < 8e-3, _rel(y, ref)
    # the shared workspace is zero again after a launch: the same call gives the same answer
    y_again = Q.q8_matmul_fused(x, qg, bias)
    assert _rel(y_again, y) < 1e-3


def test_q8_matmul_routes_fp32_and_large_batches_to_the_dense_path():
    from rumus_b200.nn.quant import Q8Tensor, dequantize_q8, matmul_q8, quantize_q8
    torch.manual_seed(3)
    w = torch.randn(256, 128) * 0.05
    qc = quantize_q8(w, 32)
    qg = Q8Tensor(qc.k, qc.n, qc.block_size, qc.data.cuda())
    x32 = torch.randn(5, 256, device="cuda")
    assert _rel(matmul_q8(x32, qg), x32 @ dequantize_q8(qc).cuda()) < 2e-3
    xb = torch.randn(1000, 256, device="cuda").bfloat16()
    assert _rel(matmul_q8(xb, qg), xb.float() @ dequantize_q8(qc).cuda()) < 1e-2
