"""Two-CTA tcgen05 GEMM (``csrc/kernels/gemm_2cta.cu``) against fp32 PyTorch products.

Opt-in (``RB_GEMM_2CTA=1``, the switch that also routes large GEMMs to this kernel): the kernel has
to be seen passing here before it becomes a default path."""
import os

import pytest
import torch
import torch.nn.functional as TF

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("RB_GEMM_2CTA", "0") != "1", reason="two-CTA GEMM is opt-in")]


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 64),        # one tile, one K block
                                   (512, 768, 384),       # several tiles per cluster
                                   (1000, 520, 136),      # ragged M / N / K (rows of the peer CTA partly or fully out of range)
                                   (2048, 1536, 1024)])
def test_two_cta_gemm_majors(dtype, a_t, b_t, shape):
    from rumus_b200.ops import native
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a_store = torch.randn((K, M) if a_t else (M, K), device="cuda", generator=g).to(dtype)
    b_store = torch.randn((N, K) if b_t else (K, N), device="cuda", generator=g).to(dtype)
    a = a_store.t() if a_t else a_store
    b = b_store.t() if b_t else b_store
    out = native.gemm(a, b, path=3)
    assert native.gemm.last_path == 3
    assert native.read_status() == 0
    assert _rel(out, a.float() @ b.float()) < 2e-2


def test_two_cta_gemm_epilogues():
    from rumus_b200.ops import native
    torch.manual_seed(0)
    M, N, K = 768, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    y, pre = native.gemm(a, b, bias=bias, act="gelu", residual=res, aux_out=True, path=3)
    ref_pre = a.float() @ b.float() + bias.float()
    assert _rel(pre, ref_pre) < 1e-2
    assert _rel(y, TF.gelu(ref_pre, approximate="tanh") + res.float()) < 1e-2
    y32 = native.gemm(a, b, out_dtype=torch.float32, path=3)
    assert y32.dtype == torch.float32 and _rel(y32, a.float() @ b.float()) < 5e-3
    assert native.read_status() == 0
