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


# ---------------------------------------------------------------- backward passes
# Oracle: PyTorch autograd on the CPU through the eager bf16 expressions the reference's Triton backward kernels
# mirror (prime_kernels/triton_rmsnorm/rmsnorm.py:1-10: "matching the fp32-upcast PyTorch reference";
# triton_swiglu/swiglu.py:78-90; triton_rope/__init__.py:105-123).  Tolerance: one bf16 ulp where a transcendental
# or a long sum is involved (exp / rsqrt differ in the last fp32 bits between libraries, sums meet in another
# order), exact for the rotary embedding.
def _ulp_close(got, want, frac_exact=0.9, terms=None):
    # 1e-6 absolute: a gradient that is the difference of two O(1) terms carries their fp32 rounding (6e-8 each).
    # `terms`: magnitude of bf16 summands of the result (a one-ulp difference in a summand survives a cancelling sum)
    got, want = got.float(), want.float()
    scale = want.abs() if terms is None else torch.maximum(want.abs(), terms.float().abs())
    ok = (got - want).abs() <= scale * 2 ** -7 + 1e-6
    assert ok.all(), f"max rel err {((got - want).abs() / (want.abs() + 1e-30)).max().item():.4f}"
    assert (got == want).float().mean() >= frac_exact


@pytest.mark.parametrize("unsqueeze_dim,rot", [(1, 64), (2, 64), (1, 32)])
def test_apply_rotary_backward(cuda_device, unsqueeze_dim, rot):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(10)
    B, S, HQ, HK, D = 2, 29, 9, 3, 64
    shape = (lambda h: (B, h, S, D)) if unsqueeze_dim == 1 else (lambda h: (B, S, h, D))
    q = torch.randn(shape(HQ), generator=g).to(torch.bfloat16)
    k = torch.randn(shape(HK), generator=g).to(torch.bfloat16)
    gq = torch.randn(shape(HQ), generator=g).to(torch.bfloat16)
    gk = torch.randn(shape(HK), generator=g).to(torch.bfloat16)
    ang = torch.rand(1, S, rot // 2, generator=g) * 6.0
    cos = torch.cat([ang.cos(), ang.cos()], -1).to(torch.bfloat16)
    sin = torch.cat([ang.sin(), ang.sin()], -1).to(torch.bfloat16)

    def hf_rope(x):        # HuggingFace apply_rotary_pos_emb in bf16, partial rotary
        c, s = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
        xr, xp = x[..., :rot], x[..., rot:]
        rotated = torch.cat([-xr[..., rot // 2:], xr[..., :rot // 2]], -1)
        return torch.cat([xr * c + rotated * s, xp], -1)

    qc, kc = q.clone().requires_grad_(), k.clone().requires_grad_()
    (hf_rope(qc) * gq).sum().backward()
    (hf_rope(kc) * gk).sum().backward()
    qd, kd = q.to(cuda_device).requires_grad_(), k.to(cuda_device).requires_grad_()
    oq, ok = E.apply_rotary(qd, kd, cos.to(cuda_device), sin.to(cuda_device), unsqueeze_dim)
    torch.autograd.backward([oq, ok], [gq.to(cuda_device), gk.to(cuda_device)])
    assert torch.equal(qd.grad.cpu(), qc.grad) and torch.equal(kd.grad.cpu(), kc.grad)


@pytest.mark.parametrize("rows,H", [(1, 960), (33, 576), (257, 2048), (1031, 960), (5000, 1024)])
def test_rmsnorm_backward(cuda_device, rows, H):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(11)
    x = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    go = torch.randn(rows, H, generator=g).to(torch.bfloat16)

    xc, wc = x.clone().requires_grad_(), w.clone().requires_grad_()
    h = xc.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
    (wc * h.to(torch.bfloat16)).backward(go)

    xd, wd = x.to(cuda_device).requires_grad_(), w.to(cuda_device).requires_grad_()
    E.rmsnorm(xd, wd, 1e-5).backward(go.to(cuda_device))
    _ulp_close(xd.grad.cpu(), xc.grad)
    # weight gradient: a sum of `rows` bf16 products accumulated in fp32 (PyTorch on the CPU sums in bf16 steps for
    # large reductions, so compare with the fp32 sum of the same rounded products)
    normed = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16).float()
    want_dw = (go.float() * normed).to(torch.bfloat16).float().sum(0)
    got_dw = wd.grad.cpu().float()
    assert ((got_dw - want_dw).abs() <= want_dw.abs() * 2 ** -7 + 2 ** -7 * want_dw.abs().mean()).all()
    # deterministic: a second run gives the same bits
    xd2, wd2 = x.to(cuda_device).requires_grad_(), w.to(cuda_device).requires_grad_()
    E.rmsnorm(xd2, wd2, 1e-5).backward(go.to(cuda_device))
    assert torch.equal(wd2.grad, wd.grad) and torch.equal(xd2.grad, xd.grad)


@pytest.mark.parametrize("use_sum_grad", [True, False])
def test_residual_rmsnorm_backward(cuda_device, use_sum_grad):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(12)
    rows, H = 130, 960
    b = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    r = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    go = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    gs = torch.randn(rows, H, generator=g).to(torch.bfloat16)

    bc, rc, wc = b.clone().requires_grad_(), r.clone().requires_grad_(), w.clone().requires_grad_()
    s = bc + rc
    h = s.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
    out = wc * h.to(torch.bfloat16)
    torch.autograd.backward([out, s] if use_sum_grad else [out], [go, gs] if use_sum_grad else [go])

    bd, rd, wd = (t.to(cuda_device).requires_grad_() for t in (b, r, w))
    out_d, sum_d = E.residual_rmsnorm(bd, rd, wd, 1e-5)
    if use_sum_grad:
        torch.autograd.backward([out_d, sum_d], [go.to(cuda_device), gs.to(cuda_device)])
    else:
        out_d.backward(go.to(cuda_device))
    _ulp_close(bd.grad.cpu(), bc.grad, frac_exact=0.85, terms=gs if use_sum_grad else None)
    assert torch.equal(bd.grad, rd.grad)
    assert wd.grad is not None and wd.grad.shape == (H,)
    # only the sum used downstream: the gradient passes straight through
    bd2, rd2, wd2 = (t.to(cuda_device).requires_grad_() for t in (b, r, w))
    _, sum_only = E.residual_rmsnorm(bd2, rd2, wd2, 1e-5)
    sum_only.backward(gs.to(cuda_device))
    assert torch.equal(bd2.grad.cpu(), gs) and torch.equal(rd2.grad.cpu(), gs)


def test_swiglu_backward_including_strided_views(cuda_device):
    from prime_kernels_b200 import elementwise as E

    g = torch.Generator().manual_seed(13)
    gu = torch.randn(23, 2 * 1536, generator=g).to(torch.bfloat16)
    go = torch.randn(23, 1536, generator=g).to(torch.bfloat16)
    guc = gu.clone().requires_grad_()
    (torch.nn.functional.silu(guc[:, :1536]) * guc[:, 1536:]).backward(go)
    gud = gu.to(cuda_device).requires_grad_()
    E.swiglu(gud[:, :1536], gud[:, 1536:]).backward(go.to(cuda_device))
    _ulp_close(gud.grad.cpu(), guc.grad, frac_exact=0.97)
