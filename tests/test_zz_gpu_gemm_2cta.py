"""Two-CTA tcgen05 GEMM (``csrc/kernels/gemm_pair.cuh``, ``gemm_2cta.cu``) against fp32 PyTorch
products: both tile shapes (256 x 256 and 512 x 256 per CTA pair), all operand majors, ragged
edges, the fused epilogue through the TMA-store path and through per-row stores."""
import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("mt", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 64),        # one tile, one K block
                                   (512, 768, 384),       # several tiles per cluster
                                   (1000, 520, 136),      # ragged M / N / K (row blocks partly or fully out of range)
                                   (2048, 1536, 1024)])
def test_two_cta_gemm_majors(dtype, a_t, b_t, shape, mt):
    from rumus_b200.ops import native
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a_store = torch.randn((K, M) if a_t else (M, K), device="cuda", generator=g).to(dtype)
    b_store = torch.randn((N, K) if b_t else (K, N), device="cuda", generator=g).to(dtype)
    a = a_store.t() if a_t else a_store
    b = b_store.t() if b_t else b_store
    out = native.gemm(a, b, path=3, mt=mt)
    assert native.gemm.last_path == 3
    assert native.read_status() == 0
    assert _rel(out, a.float() @ b.float()) < 2e-2


@pytest.mark.parametrize("mt", [1, 2])
@pytest.mark.parametrize("tma_store", ["1", "0"])
def test_two_cta_gemm_epilogues(mt, tma_store, monkeypatch):
    monkeypatch.setenv("RB_G2_TMA_STORE", tma_store)
    from rumus_b200.ops import native
    torch.manual_seed(0)
    M, N, K = 768, 520, 256
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    y, pre = native.gemm(a, b, bias=bias, act="gelu", residual=res, aux_out=True, path=3, mt=mt)
    ref_pre = a.float() @ b.float() + bias.float()
    assert _rel(pre, ref_pre) < 1e-2
    assert _rel(y, TF.gelu(ref_pre, approximate="tanh") + res.float()) < 1e-2
    # derivative epilogue: dact'(aux_in) * acc
    d = native.gemm(a, b, aux_in=pre, dact="gelu", path=3, mt=mt)
    x = pre.float().requires_grad_(True)
    TF.gelu(x, approximate="tanh").sum().backward()
    assert _rel(d, (a.float() @ b.float()) * x.grad) < 1.5e-2
    y32 = native.gemm(a, b, out_dtype=torch.float32, path=3, mt=mt)
    assert y32.dtype == torch.float32 and _rel(y32, a.float() @ b.float()) < 5e-3
    # accumulate into an existing fp32 buffer (residual aliases the output)
    acc = torch.randn(M, N, device="cuda")
    ref = acc.clone() + a.float() @ b.float()
    native.gemm(a, b, out_dtype=torch.float32, residual=acc, out=acc, path=3, mt=mt)
    assert _rel(acc, ref) < 5e-3
    assert native.read_status() == 0


def test_two_cta_gemm_output_row_pitch_not_tma_legal():
    """An output whose row pitch is not a multiple of 16 bytes takes the per-row store path."""
    from rumus_b200.ops import native
    torch.manual_seed(1)
    M, N, K = 512, 264, 128
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    buf = torch.zeros(M, N + 3, device="cuda", dtype=torch.bfloat16)
    out = buf[:, :N]
    native.gemm(a, b, out=out, path=3)
    assert _rel(out, a.float() @ b.float()) < 2e-2
    assert float(buf[:, N:].abs().max()) == 0.0
    assert native.read_status() == 0
