"""Bounds-guard mode on the GPU: representative kernels run on ragged shapes with every output
and scratch buffer between canary bands (``rumus_b200/utils/canary.py``); nothing may be written
outside a buffer.  Runs last: it exercises the same kernels as the numerics suites."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_guard_sees_a_write_past_the_end_on_the_device():
    """The overrun is produced with a strided view of the guarded buffer itself, so every byte
    written lies inside one allocation: the device never sees an invalid address."""
    from rumus_b200.utils.canary import CanaryError, canary_guard
    with pytest.raises(CanaryError, match="after the tensor"):
        with canary_guard():
            a = torch.empty((3, 5), dtype=torch.float32, device="cuda")
            torch.as_strided(a, (16,), (1,)).fill_(1.0)
    with canary_guard() as g:
        a = torch.zeros((3, 5), dtype=torch.bfloat16, device="cuda")
        assert a.data_ptr() % 512 == 0 and a.is_contiguous() and float(a.sum()) == 0.0
        a.fill_(2.0)
        assert g.check() == 1


def test_kernels_stay_inside_their_outputs_on_ragged_shapes():
    from rumus_b200.ops import functional as F
    from rumus_b200.ops import native
    from rumus_b200.utils.canary import canary_guard
    torch.manual_seed(0)
    dev = "cuda"
    with canary_guard() as g:
        # tcgen05 GEMMs with epilogues and their backward (M not a multiple of the 128-row tile)
        x = (torch.randn(3, 100, 136, device=dev) * 0.5).bfloat16().requires_grad_(True)
        w1 = (torch.randn(136, 264, device=dev) * 0.05).bfloat16().requires_grad_(True)
        b1 = (torch.randn(264, device=dev) * 0.1).bfloat16().requires_grad_(True)
        w2 = (torch.randn(264, 136, device=dev) * 0.05).bfloat16().requires_grad_(True)
        b2 = (torch.randn(136, device=dev) * 0.1).bfloat16().requires_grad_(True)
        F.mlp(x, w1, b1, w2, b2, act="gelu", residual=x).float().pow(2).mean().backward()
        F.linear(x, w1, b1, act="relu").float().sum().backward()
        # SIMT fallback (shapes TMA cannot address)
        a = torch.randn(130, 257, device=dev)
        b = torch.randn(257, 70, device=dev)
        native.gemm(a, b, bias=torch.randn(70, device=dev), act="relu")
        native.bmm(torch.randn(6, 33, 17, device=dev), torch.randn(6, 17, 29, device=dev))
        # norms, forward and backward, row length not a multiple of the vector width of a warp
        for D, rms in ((100, False), (100, True), (4096 + 8, False)):
            xn = torch.randn(77, D, device=dev).bfloat16().requires_grad_(True)
            res = torch.randn(77, D, device=dev).bfloat16().requires_grad_(True)
            gam = torch.ones(D, device=dev).bfloat16().requires_grad_(True)
            bet = torch.zeros(D, device=dev).bfloat16().requires_grad_(True)
            y, h = F.rms_norm(xn, gam, 1e-6, residual=res) if rms else F.layer_norm(xn, gam, bet, 1e-5, residual=res)
            (y.float().sum() + h.float().pow(2).sum()).backward()
        # softmax and cross entropy over ragged row lengths
        for n in (7, 50304 // 8 + 3):
            xs = (torch.randn(19, n, device=dev) * 3).bfloat16().requires_grad_(True)
            F.softmax(xs).float().sum().backward()
            xl = (torch.randn(19, n, device=dev) * 3).bfloat16().requires_grad_(True)
            F.cross_entropy_loss(xl, torch.randint(0, n, (19,), device=dev)).backward()
        # FlashAttention forward and backward, sequence length not a multiple of the tile
        q, k, v = ((torch.randn(2, 200, 4, 128, device=dev) * 0.5).bfloat16().requires_grad_(True) for _ in range(3))
        F.flash_attention(q, k, v, True).float().pow(2).sum().backward()
        n_checked = g.check()
    assert n_checked >= 15
    assert native.read_status() == 0
