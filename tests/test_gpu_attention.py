"""Slice-causal attention kernels against an fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _reference(qkv, b, h, D):
    """Full causal attention in fp32 on qkv [L, b, h, 3, D]; returns out [L, b, h*D]."""
    L = qkv.shape[0]
    x = qkv.float().view(L, b, h, 3, D)
    q, k, v = (x[:, :, :, i].permute(1, 2, 0, 3) for i in range(3))  # [b, h, L, D]
    s = (q @ k.transpose(-1, -2)) * D ** -0.5
    mask = torch.ones(L, L, device=qkv.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, -1) @ v
    return o.permute(2, 0, 1, 3).reshape(L, b, h * D)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D,b,h,slices", [
    (128, 2, 2, [128, 128]),
    (64, 2, 4, [64, 32, 16, 16]),
    (128, 1, 3, [200, 56, 128, 64, 8]),
    (64, 3, 2, [136, 120]),
])
def test_attention_slices_match_full_causal(dtype, D, b, h, slices):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(0)
    L = sum(slices)
    qkv = torch.randn(L, b, h * 3 * D, device="cuda", dtype=dtype)
    o = torch.zeros(L * b, h * D, device="cuda", dtype=dtype)
    lse2 = torch.zeros(b * h, L, device="cuda")
    c = 0
    for t in slices:
        F.attn_fwd(qkv, b, h, D, t, c, o[c * b:(c + t) * b], lse2)
        c += t
    F.check_device_status()
    qkv_ref = qkv.float().requires_grad_()
    ref = _reference(qkv_ref, b, h, D)
    tol = 4e-3 if dtype == torch.float16 else 2e-2
    assert _rel(o.view(L, b, h * D), ref) < tol

    g = torch.randn(L * b, h * D, device="cuda", dtype=dtype)
    ref.backward(g.float().view(L, b, h * D))
    dqkv = torch.zeros(L * b, h * 3 * D, device="cuda", dtype=dtype)
    delta = torch.full((b * h, L), float("nan"), device="cuda")
    do_full = torch.full((L * b, h * D), float("nan"), device="cuda", dtype=dtype)
    c = L
    for t in reversed(slices):
        c -= t
        do_full[c * b:(c + t) * b] = g[c * b:(c + t) * b]     # what the out-proj dgrad would write
        F.attn_bwd(qkv, b, h, D, t, c, L, o[c * b:(c + t) * b], do_full, lse2, delta,
                   dqkv[c * b:(c + t) * b])
    F.check_device_status()
    got = dqkv.view(L, b, h, 3, D).float()
    want = qkv_ref.grad.view(L, b, h, 3, D)
    for w, name in enumerate("qkv"):
        assert _rel(got[:, :, :, w], want[:, :, :, w]) < 3 * tol, name
