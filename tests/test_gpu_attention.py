"""FlashAttention forward/backward (tcgen05 kernels) against an fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        from rumus_b200.ops import native
        assert native.read_status() == 0, "a device-side bounded wait timed out"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,D,causal", [
    (2, 256, 4, 128, True), (1, 384, 2, 128, False), (2, 200, 3, 128, True),
    (1, 128, 2, 64, True), (1, 1024, 2, 128, True), (1, 77, 1, 128, False),
])
def test_flash_attention_forward(dtype, B, S, H, D, causal):
    from rumus_b200.ops import functional as F
    torch.manual_seed(S + H)
    qkv = (torch.randn(B, S, 3 * H * D, device="cuda") * 0.7).to(dtype)
    q, k, v = (t.view(B, S, H, D) for t in qkv.split(H * D, dim=-1))  # strided views of fused qkv
    o = F.flash_attention(q, k, v, causal)
    ref = F.sdpa_reference(q.float(), k.float(), v.float(), causal)
    assert _rel(o, ref) < 2e-2, _rel(o, ref)


@pytest.mark.parametrize("B,S,H,Hkv,causal", [
    (2, 256, 4, 4, True), (1, 320, 2, 2, False), (1, 200, 4, 2, True), (1, 1024, 2, 2, True),
])
def test_flash_attention_backward(B, S, H, Hkv, causal):
    from rumus_b200.ops import functional as F
    D = 128
    torch.manual_seed(S * 3 + H)
    q = (torch.randn(B, S, H, D, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    k = (torch.randn(B, S, Hkv, D, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    v = (torch.randn(B, S, Hkv, D, device="cuda") * 0.7).bfloat16().requires_grad_(True)
    w = torch.randn(B, S, H, D, device="cuda").bfloat16()
    o = F.flash_attention(q, k, v, causal)
    (o.float() * w.float()).sum().backward()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = F.sdpa_reference(qr, kr, vr, causal)
    (orf * w.float()).sum().backward()
    assert _rel(o, orf) < 2e-2
    assert _rel(q.grad, qr.grad) < 3e-2, _rel(q.grad, qr.grad)
    assert _rel(k.grad, kr.grad) < 3e-2, _rel(k.grad, kr.grad)
    assert _rel(v.grad, vr.grad) < 3e-2, _rel(v.grad, vr.grad)


@pytest.mark.parametrize("B,S,H,Hkv,causal", [(2, 256, 4, 4, True), (1, 200, 4, 2, True), (1, 130, 2, 2, False)])
def test_flash_attention_packed_matches_split(B, S, H, Hkv, causal):
    """Packed-qkv attention (gradients written into one d_qkv buffer) against the split form."""
    from rumus_b200.ops import functional as F
    torch.manual_seed(3)
    D = 128
    W = (H + 2 * Hkv) * D
    base = (torch.randn(B, S, W, device="cuda") * 0.6).bfloat16()
    a = base.clone().requires_grad_(True)
    b = base.clone().requires_grad_(True)
    o1 = F.flash_attention_packed(a, H, Hkv, causal)
    q, k, v = b.split([H * D, Hkv * D, Hkv * D], dim=-1)
    o2 = F.flash_attention(q.view(B, S, H, D), k.view(B, S, Hkv, D), v.view(B, S, Hkv, D), causal)
    assert torch.equal(o1, o2)
    g = torch.randn_like(o1)
    o1.backward(g)
    o2.backward(g)
    assert _rel(a.grad, b.grad) < 1e-3, _rel(a.grad, b.grad)
    ref = base.float().requires_grad_(True)
    qf, kf, vf = ref.split([H * D, Hkv * D, Hkv * D], dim=-1)
    kf4, vf4 = kf.view(B, S, Hkv, D), vf.view(B, S, Hkv, D)
    if Hkv != H:
        kf4 = kf4.repeat_interleave(H // Hkv, dim=2)
        vf4 = vf4.repeat_interleave(H // Hkv, dim=2)
    F.sdpa_reference(qf.view(B, S, H, D), kf4, vf4, causal).backward(g.float())
    assert _rel(a.grad, ref.grad) < 3e-2, _rel(a.grad, ref.grad)
