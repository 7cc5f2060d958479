"""GPU: the standalone forward ops against a plain PyTorch fp32 reference with the same bf16 rounding points."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(x):
    return x.to(torch.bfloat16).float()


@pytest.mark.parametrize("unsqueeze_dim,rot", [(1, 64), (2, 64), (1, 32)])
def test_apply_rotary(cuda_device, unsqueeze_dim, rot):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(0)
    B, S, HQ, HK, D = 2, 37, 15, 5, 64
    shape = (lambda h: (B, h, S, D)) if unsqueeze_dim == 1 else (lambda h: (B, S, h, D))
    q = torch.randn(shape(HQ), generator=g).to(torch.bfloat16)
    k = torch.randn(shape(HK), generator=g).to(torch.bfloat16)
    ang = torch.rand(1, S, rot // 2, generator=g) * 6.0
    cos = torch.cat([ang.cos(), ang.cos()], -1).to(torch.bfloat16)
    sin = torch.cat([ang.sin(), ang.sin()], -1).to(torch.bfloat16)
    oq, ok = E.apply_rotary(q.to(cuda_device), k.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), unsqueeze_dim)

    def ref(x):
        c, s = cos.float().unsqueeze(unsqueeze_dim), sin.float().unsqueeze(unsqueeze_dim)
        xr, xp = x.float()[..., :rot], x.float()[..., rot:]
        half = rot // 2
        rotated = torch.cat([-xr[..., half:], xr[..., :half]], -1)
        y = bf(bf(xr * c) + bf(rotated * s))
        return torch.cat([y, xp], -1).to(torch.bfloat16)

    assert torch.equal(oq.cpu(), ref(q)) and torch.equal(ok.cpu(), ref(k))


@pytest.mark.parametrize("rows,H", [(1, 960), (33, 576), (257, 2048)])
def test_rmsnorm_and_residual_rmsnorm(cuda_device, rows, H):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    r = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)

    def ref_norm(v):
        rstd = torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + 1e-5)
        return bf(w.float() * bf(v.float() * rstd))

    out = E.rmsnorm(x.to(cuda_device), w.to(cuda_device), 1e-5).cpu().float()
    want = ref_norm(x)
    # the reciprocal rms differs in the last fp32 bits (rsqrt approximation, summation order): one bf16 ulp
    assert ((out - want).abs() <= want.abs() * 2 ** -7 + 1e-30).all()
    assert (out != want).float().mean() < 0.02

    out2, summed = E.residual_rmsnorm(x.to(cuda_device), r.to(cuda_device), w.to(cuda_device), 1e-5)
    want_sum = bf(x.float() + r.float())
    assert torch.equal(summed.cpu().float(), want_sum)
    want2 = ref_norm(want_sum)
    assert ((out2.cpu().float() - want2).abs() <= want2.abs() * 2 ** -7 + 1e-30).all()


def test_swiglu_including_strided_views(cuda_device):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(2)
    gu = torch.randn(19, 2 * 2560, generator=g).to(torch.bfloat16).to(cuda_device)
    gate, up = gu[:, :2560], gu[:, 2560:]                 # strided views of one fused projection output
    out = E.swiglu(gate, up).cpu().float()
    gf, uf = gate.cpu().float(), up.cpu().float()
    want = bf(bf(gf / (1 + torch.exp(-gf))) * uf)
    # exp differs by an ulp between the CPU and the GPU libraries; after bf16 rounding almost nothing moves
    assert ((out - want).abs() <= want.abs() * 2 ** -7 + 1e-30).all()
    assert (out != want).float().mean() < 0.01


def test_fakes_and_errors(cuda_device):
    from prime_kernels_b200 import elementwise as E

    x = torch.empty(4, 960, dtype=torch.bfloat16, device="meta")
    assert E.swiglu(x, x).shape == (4, 960)
    with pytest.raises(RuntimeError):
        E.rmsnorm(torch.zeros(4, 960, device=cuda_device), torch.zeros(960, device=cuda_device), 1e-5)   # fp32 unsupported
