"""GPU parity tests of the batch-1 specialised decode kernel (SmolLM2-135M / 360M / 1.7B widths), called
through torch.ops -> C ABI, against the CPU restatement of the rounding points, and against the generic
kernel of the same library.  Shallow models (2-3 layers, small vocabulary) keep the CPU oracle fast; the
widths are the real ones because the kernel is compiled for them."""
import pytest
import torch

from oracle import decode_restatement as R
from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2

WIDTHS = {
    "360m": (960, 2560, 15, 5),
    "135m": (576, 1536, 9, 3),
    "1.7b": (2048, 8192, 32, 32),
}


def _geom(D, which, layers=2, vocab=2048):
    h, i, qh, kvh = WIDTHS[which]
    return D.Geometry(f"{which}-w{layers}", h, i, layers, qh, kvh, vocab)


def _set_path(warps):
    from prime_kernels_b200._cabi import library

    assert library().pk_decode_set_fast_path(warps) == 0


@pytest.fixture(autouse=True)
def _restore_default_path():
    yield
    _set_path(7)


def _step(D, geom, wd, kv, csd, cur, pos, lm_head=True, layer_outputs=None):
    dev = kv.device
    return D.decode_step(geom, input_ids=cur.to(dev), positions=pos.to(dev), seq_lens=(pos + 1).to(torch.int32).to(dev),
                         block_table=kv.block_table, slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                         final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=geom.eps,
                         layer_outputs=layer_outputs, lm_head=lm_head)


@pytest.mark.parametrize("warps", [7, 8])
@pytest.mark.parametrize("which,ctx,shuffle,block_size", [
    ("360m", 0, False, 16),        # the new token is the whole context
    ("360m", 5, False, 16),
    ("360m", 111, True, 16),       # chunk boundary of the 7-warp kernel (112 positions with the new token)
    ("360m", 600, True, 16),       # the benchmark's context range: several chunks per kv head
    ("360m", 150, True, 8),        # a 16-position run straddles cache blocks
    ("360m", 3300, True, 16),      # beyond the pre-resolved runs: block table read per run, longer chunks
    ("135m", 40, False, 16),
    ("135m", 1000, True, 16),
    ("1.7b", 0, False, 16),        # multi-head attention (one query head per kv head), down-projection rows in two parts
    ("1.7b", 200, True, 16),       # two chunks per kv head
    ("1.7b", 1100, True, 16),      # three chunks, several runs per warp
    ("1.7b", 2900, True, 8),       # block table read per run
])
def test_fast_kernel_against_restatement(cuda_device, warps, which, ctx, shuffle, block_size):
    from prime_kernels_b200 import decode as D

    _set_path(warps)
    geom = _geom(D, which)
    w = harness.make_weights(geom, 0, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    cap = max(64, ((ctx + 40) // 16 + 1) * 16)
    cs = harness.make_cos_sin_cache(geom, cap)
    csd = cs.to(cuda_device)
    gen = torch.Generator().manual_seed(7)
    cur = torch.randint(0, geom.vocab, (1,), generator=gen)
    keys = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16)] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16)] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, 1, cap, cuda_device, block_size=block_size, shuffle=shuffle)
    if ctx:
        kv.load_prefix([torch.stack(k) for k in keys], [torch.stack(v) for v in vals])
    for s in range(3):
        pos = torch.full((1,), ctx + s, dtype=torch.int64)
        lo = torch.zeros(geom.layers, 1, geom.hidden, dtype=torch.bfloat16, device=cuda_device)
        hid, logits, nxt = _step(D, geom, wd, kv, csd, cur, pos, layer_outputs=lo)
        D.check_status(geom, cuda_device)
        tol = LOGIT_TOL
        if which == "1.7b":
            # logits of magnitude 2-4 at this width: one bf16 ulp is 0.0156, so the bound is taken relative to the
            # distance between the restatement's own two softmax-rounding variants on the same inputs
            k2 = [[k[0][:, :ctx + s].clone()] for k in keys]
            v2 = [[v[0][:, :ctx + s].clone()] for v in vals]
            _, rl_b, _ = R.decode_step(geom, w, cur, pos, k2, v2, cs, probs="bf16")
        rh, rl, rlo = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        if which == "1.7b":
            tol = LOGIT_TOL + 1.25 * (rl - rl_b).abs().max().item()
        assert (lo.cpu().float() - rlo.float()).abs().max() <= 2 ** -4
        assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4
        assert (logits.cpu().float() - rl).abs().max() <= tol
        margin = rl.topk(2, -1).values
        if margin[0, 0] - margin[0, 1] > 2 * tol:
            assert int(nxt[0]) == int(rl.argmax(-1)[0])
        for layer in range(geom.layers):      # the K/V this step appended equals the oracle's (one bf16 ulp)
            got = kv.gather(layer, 0, ctx + s + 1)[:, -1, :].cpu().float()
            want = torch.cat([keys[layer][0][:, -1, :], vals[layer][0][:, -1, :]], -1).float()
            assert (got - want).abs().max() <= (2 ** -5 if layer == 0 else 2 ** -3)
        cur = rl.argmax(-1)


def test_fast_and_generic_kernels_agree(cuda_device):
    """Same inputs through the specialised and the generic kernel: same rounding points, different fp32
    summation order -- logits within the bf16 tolerance, identical greedy id, identical appended K/V at layer 0."""
    from prime_kernels_b200 import decode as D

    geom = _geom(D, "360m", layers=3)
    w = harness.make_weights(geom, 4, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    csd = harness.make_cos_sin_cache(geom, 512, cuda_device)
    gen = torch.Generator().manual_seed(3)
    outs = []
    for warps in (7, 0):
        _set_path(warps)
        kv = harness.PagedKV(geom, 1, 512, cuda_device, shuffle=True, seed=1)
        g2 = torch.Generator().manual_seed(5)
        for cache in kv.kv_caches:
            cache.copy_(torch.randn(cache.shape, generator=g2).to(torch.bfloat16))
        pos = torch.tensor([300])
        hid, logits, nxt = _step(D, geom, wd, kv, csd, torch.tensor([77]), pos)
        D.check_status(geom, cuda_device)
        outs.append((hid.clone(), logits.clone(), nxt.clone(), kv.gather(0, 0, 301)[:, -1, :].clone()))
    (h1, l1, n1, k1), (h0, l0, n0, k0) = outs
    assert (l1.float() - l0.float()).abs().max() <= LOGIT_TOL
    assert (h1.float() - h0.float()).abs().max() <= 2 ** -4
    assert torch.equal(k1, k0)
    top = l0.float().topk(2, -1).values
    if top[0, 0] - top[0, 1] > 2 * LOGIT_TOL:
        assert torch.equal(n1, n0)


@pytest.mark.parametrize("warps", [7, 0])
def test_alternating_lm_head_does_not_reuse_old_argmax(cuda_device, warps):
    """lm_head steps alternating with hidden-only steps on one workspace: the greedy id of every lm_head step is
    that step's own argmax (an argmax cell left over from two launches earlier must never win)."""
    from prime_kernels_b200 import decode as D

    _set_path(warps)
    geom = _geom(D, "360m", layers=2)
    w = harness.make_weights(geom, 9, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    cs = harness.make_cos_sin_cache(geom, 128)
    csd = cs.to(cuda_device)
    kv = harness.PagedKV(geom, 1, 128, cuda_device)
    keys = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16)] for _ in range(geom.layers)]
    vals = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16)] for _ in range(geom.layers)]
    gen = torch.Generator().manual_seed(1)
    pattern = [True, False, True, False, False, False, True, True, False, True]
    for s, lm in enumerate(pattern):
        cur = torch.randint(0, geom.vocab, (1,), generator=gen)
        pos = torch.tensor([s])
        out = _step(D, geom, wd, kv, csd, cur, pos, lm_head=lm)
        D.check_status(geom, cuda_device)
        _, rl, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        if lm:
            _, logits, nxt = out
            assert int(nxt[0]) == int(logits[0].float().argmax())         # the kernel's own logits
            top = rl.topk(2, -1).values
            if top[0, 0] - top[0, 1] > 2 * LOGIT_TOL:
                assert int(nxt[0]) == int(rl.argmax(-1)[0])


@pytest.mark.parametrize("warps", [7, 8])
def test_fast_device_driven_generation_matches_stepwise(cuda_device, warps):
    from prime_kernels_b200 import decode as D

    _set_path(warps)
    geom = _geom(D, "135m", layers=3)
    wd = harness.weights_to(harness.make_weights(geom, 5, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 128, cuda_device)
    steps = 40
    first = torch.tensor([11])

    def fresh():
        return harness.PagedKV(geom, 1, 128, cuda_device, shuffle=True, seed=3)

    kv_a = fresh()
    sess = D.DecodeSession(geom, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                           kv_caches=kv_a.kv_caches, cos_sin_cache=csd, block_table=kv_a.block_table)
    sess.start(first, torch.zeros(1, dtype=torch.int64))
    ids_a = sess.generate(steps).cpu()
    kv_b = fresh()
    cur, ids_b = first.clone(), []
    for s in range(steps):
        _, _, nxt = _step(D, geom, wd, kv_b, csd, cur, torch.tensor([s]))
        cur = nxt.cpu().clone()
        ids_b.append(cur)
    D.check_status(geom, cuda_device)
    assert torch.equal(ids_a, torch.stack(ids_b))
    for ca, cb in zip(kv_a.kv_caches, kv_b.kv_caches):
        assert torch.equal(ca, cb)


@pytest.mark.parametrize("warps", [7, 0])
def test_padded_row_and_sequence_overflow(cuda_device, warps):
    """slot -1 writes nothing into the cache; a sequence length beyond the block table's capacity is reported
    (status 9102) instead of indexing past the table, and the workspace is usable again afterwards."""
    from prime_kernels_b200 import decode as D

    _set_path(warps)
    geom = _geom(D, "360m", layers=2)
    wd = harness.weights_to(harness.make_weights(geom, 1), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 64, cuda_device)
    kv = harness.PagedKV(geom, 1, 64, cuda_device)
    for c in kv.kv_caches:
        c.fill_(0.5)
    before = [c.clone() for c in kv.kv_caches]
    pos = torch.tensor([3])
    kw = dict(input_ids=torch.tensor([1], device=cuda_device), positions=pos.to(cuda_device), block_table=kv.block_table,
              embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
              cos_sin_cache=csd, eps=geom.eps)
    D.decode_step(geom, seq_lens=torch.tensor([4], dtype=torch.int32, device=cuda_device),
                  slot_mapping=torch.tensor([-1], device=cuda_device), **kw)
    D.check_status(geom, cuda_device)
    for c, b in zip(kv.kv_caches, before):
        assert torch.equal(c, b)
    D.decode_step(geom, seq_lens=torch.tensor([65], dtype=torch.int32, device=cuda_device),
                  slot_mapping=torch.tensor([-1], device=cuda_device), **kw)
    with pytest.raises(RuntimeError, match="max_seq_len"):
        D.check_status(geom, cuda_device)
    hid = D.decode_step(geom, seq_lens=torch.tensor([4], dtype=torch.int32, device=cuda_device),
                        slot_mapping=kv.slots(pos), **kw)
    D.check_status(geom, cuda_device)
    assert torch.isfinite(hid.float()).all()
    assert not torch.equal(kv.kv_caches[0], before[0])


@pytest.mark.parametrize("which,ctx", [("360m", 0), ("360m", 77), ("360m", 1200), ("135m", 300), ("1.7b", 450)])
def test_fast_kernel_with_mxfp8_weights(cuda_device, which, ctx):
    """MXFP8 weights (E4M3 + one E8M0 per 32 along K, de-quantised in registers inside the GEMV) on the batch-1
    kernel: against the restatement on the exactly de-quantised weights, and against the generic kernel of this
    library on the same packed weights, over three teacher-forced steps with alternating lm_head."""
    from prime_kernels_b200 import decode as D

    h, i, qh, kvh = WIDTHS[which]
    geom = D.Geometry(f"{which}-mx", h, i, 2, qh, kvh, 2048, weight_format=1)
    w = harness.make_weights(geom, 5, norm_weights="random")
    wq = D.pack_weights_mxfp8(harness.weights_to(w, cuda_device))
    wo = {"embed": D.unpack_matrix_mxfp8(wq["embed"], geom.hidden).cpu(), "embed_lookup": w["embed"],
          "final_norm": w["final_norm"], "layers": []}
    for (n1, _, _, n2, _, _), (_, qkv_p, o_p, _, gu_p, down_p) in zip(w["layers"], wq["layers"]):
        wo["layers"].append((n1, D.unpack_matrix_mxfp8(qkv_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(o_p, geom.q_heads * 64).cpu(), n2,
                             D.unpack_matrix_mxfp8(gu_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(down_p, geom.intermediate).cpu()))
    cap = (ctx + 48 + 15) // 16 * 16
    cs = harness.make_cos_sin_cache(geom, cap)
    csd = cs.to(cuda_device)
    gen = torch.Generator().manual_seed(31)
    keys = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16)] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16)] for _ in range(geom.layers)]
    results = {}
    # the batch-1 kernel, then the generic kernel (which does not take packed rows longer than its ring entries: the
    # 8448-byte down-projection rows of the 1.7B widths run on the batch-1 kernel only)
    paths = (7,) if which == "1.7b" else (7, 0)
    for path in paths:
        _set_path(path)
        kv = harness.PagedKV(geom, 1, cap, cuda_device, shuffle=True, seed=2)
        if ctx:
            kv.load_prefix([k[0][None] for k in keys], [v[0][None] for v in vals])
        ks = [[k[0].clone()] for k in keys]
        vs = [[v[0].clone()] for v in vals]
        cur = torch.tensor([123])
        outs = []
        for s in range(3):
            pos = torch.tensor([ctx + s], dtype=torch.int64)
            hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                             seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                             slot_mapping=kv.slots(pos), embed=wq["embed"], embed_lookup=wq["embed_lookup"],
                                             layers=wq["layers"], final_norm=wq["final_norm"], kv_caches=kv.kv_caches,
                                             cos_sin_cache=csd, eps=geom.eps, lm_head=True)
            D.check_status(geom, cuda_device)
            tol = LOGIT_TOL
            if which == "1.7b":      # one bf16 ulp of these logits is 0.0156: bound relative to the restatement's own variants
                _, rl_b, _ = R.decode_step(geom, wo, cur, pos, [[k[0].clone()] for k in ks], [[v[0].clone()] for v in vs], cs,
                                           probs="bf16")
            rh, rl, _ = R.decode_step(geom, wo, cur, pos, ks, vs, cs)
            if which == "1.7b":
                tol = LOGIT_TOL + 1.25 * (rl - rl_b).abs().max().item()
            assert (logits.cpu().float() - rl).abs().max() <= tol, f"path {path} step {s}"
            assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4
            outs.append((hid.clone(), logits.clone()))
            cur = rl.argmax(-1)
        results[path] = outs
    for (ha, la), (hb, lb) in zip(results[7], results[paths[-1]]):
        assert (la.float() - lb.float()).abs().max() <= LOGIT_TOL
        assert (ha.float() - hb.float()).abs().max() <= 2 ** -4
