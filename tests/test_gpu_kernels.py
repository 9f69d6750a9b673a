"""sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1024, 768, 256), (1000, 1024, 512), (128, 256, 64),
                                   (72, 2048, 2048), (1024, 6144, 2048)])
@pytest.mark.parametrize("bn", [0, 64, 128, 256, 512, 1128, 1256])
def test_gemm_forward_layout(dtype, M, N, K, bn):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    w = torch.randn(N, K, device="cuda", dtype=dtype) * 0.05
    bias = torch.randn(N, device="cuda", dtype=dtype)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)  # a skipped store must show
    F.gemm(a, w, out, bias=bias, force_bn=bn)
    ref = a.float() @ w.float().t() + bias.float()
    F.check_device_status()
    assert _rel(out, ref) < (2e-3 if dtype == torch.float16 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_dgrad_layout(dtype):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(1)
    M, Nout, Kin = 520, 768, 512
    dy = torch.randn(M, Nout, device="cuda", dtype=dtype)
    w = torch.randn(Nout, Kin, device="cuda", dtype=dtype) * 0.05
    dx = torch.empty(M, Kin, device="cuda", dtype=dtype)
    for bn in (64, 128, 256, 512, 1128, 1256):
        dx.fill_(float("nan"))
        F.gemm(dy, w, dx, b_mn=True, force_bn=bn)
        assert _rel(dx, dy.float() @ w.float()) < 1e-2
    F.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_wgrad_layout_accumulates(dtype):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(2)
    T, Nout, Kin = 328, 384, 512
    dy = torch.randn(T, Nout, device="cuda", dtype=dtype)
    x = torch.randn(T, Kin, device="cuda", dtype=dtype)
    for bn in (64, 128, 256, 512, 1128, 1256):
        dw = torch.ones(Nout, Kin, device="cuda", dtype=torch.float32)
        F.gemm(dy, x, dw, a_mn=True, b_mn=True, accumulate=True, force_bn=bn)
        F.gemm(dy, x, dw, a_mn=True, b_mn=True, accumulate=True, force_bn=bn)
        ref = 1.0 + 2.0 * (dy.float().t() @ x.float())
        assert _rel(dw, ref) < 2e-3
    F.check_device_status()


@pytest.mark.parametrize("act", ["relu", "gelu"])
def test_gemm_activation_epilogues(act):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(3)
    dtype = torch.float16
    M, N, K = 256, 512, 256
    x = torch.randn(M, K, device="cuda", dtype=dtype)
    w = torch.randn(N, K, device="cuda", dtype=dtype) * 0.1
    b = torch.randn(N, device="cuda", dtype=dtype)
    res = torch.randn(M, N, device="cuda", dtype=dtype)
    out = torch.empty(M, N, device="cuda", dtype=dtype)
    pre = torch.empty(M, N, device="cuda", dtype=dtype)
    F.gemm(x, w, out, bias=b, act=act, aux_out=pre if act == "gelu" else None)
    z = x.float() @ w.float().t() + b.float()
    ref = torch.relu(z) if act == "relu" else torch.nn.functional.gelu(z)
    assert _rel(out, ref) < 3e-3
    if act == "gelu":
        assert _rel(pre, z) < 2e-3
    # residual epilogue
    F.gemm(x, w, out, bias=b, residual=res)
    assert _rel(out, z + res.float()) < 2e-3
    # derivative epilogue: d/dz act(z) * upstream, upstream = x @ w^T (re-used as a stand-in)
    aux = (ref.to(dtype) if act == "relu" else z.to(dtype))
    F.gemm(x, w, out, dact=act, aux_in=aux)
    up = x.float() @ w.float().t()
    zz = aux.float().requires_grad_()
    (torch.relu(zz) if act == "relu" else torch.nn.functional.gelu(zz)).backward(up)
    assert _rel(out, zz.grad) < 5e-3
    F.check_device_status()


# 6144: 48 KB of dynamic shared memory + static in the forward; 3000 x 2048 and 1500 x 5120: several
# passes of the persistent backward CTAs; 77 x 1024: one warp per row, fewer rows than a CTA holds
@pytest.mark.parametrize("rows,H", [(520, 256), (520, 2048), (520, 5120), (520, 6144), (520, 12288),
                                    (3000, 2048), (1500, 5120), (77, 1024), (5, 2048)])
def test_layernorm_fwd_bwd(rows, H):
    from terapipe_b200.ops import functional as F
    torch.manual_seed(4)
    dtype = torch.float16
    x = torch.randn(rows, H, device="cuda", dtype=dtype)
    g = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
    b = (0.1 * torch.randn(H, device="cuda")).to(dtype)
    y = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    F.layernorm_fwd(x, g, b, y, mean, rstd)
    xf = x.float().requires_grad_()
    gf, bf = g.float().requires_grad_(), b.float().requires_grad_()
    ref = torch.nn.functional.layer_norm(xf, (H,), gf, bf)
    assert _rel(y, ref) < 2e-3
    dy = torch.randn(rows, H, device="cuda", dtype=dtype)
    dres = torch.randn(rows, H, device="cuda", dtype=dtype)
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dgamma = torch.ones(H, device="cuda")
    dbeta = torch.ones(H, device="cuda")
    scratch = torch.empty(F.layernorm_bwd_scratch_floats(rows, H), device="cuda")
    F.layernorm_bwd(dy, x, mean, rstd, g, dx, dgamma, dbeta, scratch, dres=dres)
    assert _rel(dx, xf.grad + dres.float()) < 3e-3
    assert _rel(dgamma, 1 + gf.grad) < 2e-3
    assert _rel(dbeta, 1 + bf.grad) < 2e-3


def test_colsum_and_fused_adam():
    from terapipe_b200.ops import functional as F
    torch.manual_seed(5)
    dy = torch.randn(1000, 768, device="cuda", dtype=torch.float16)
    db = torch.ones(768, device="cuda")
    F.colsum(dy, db)
    assert _rel(db, 1 + dy.float().sum(0)) < 1e-3
    n = 4096 * 33
    p = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_()
    opt = torch.optim.Adam([ref_p], lr=1e-3)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    model = torch.empty(n, device="cuda", dtype=torch.float16)
    state = torch.zeros(3, device="cuda")
    for _ in range(3):
        g = torch.randn(n, device="cuda")
        ref_p.grad = g.clone()
        opt.step()
        grad = g * 128.0
        F.adam_tick(state)
        F.fused_adam(grad, p, m, v, model, state, lr=1e-3, grad_scale=1 / 128.0)
        assert grad.abs().max().item() == 0.0
    assert _rel(p, ref_p.detach()) < 1e-5
    assert _rel(model, p) < 1e-3
