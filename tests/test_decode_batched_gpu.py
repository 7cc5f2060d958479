"""GPU parity tests of the tensor-core batched decode kernel (9..64 requests in one launch, projections as
tcgen05 GEMMs) against the CPU restatement of the rounding points, called through torch.ops -> C ABI."""
import pytest
import torch

from oracle import decode_restatement as R
from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2


def _oracle_weights(D, w, wq, geom):
    """Exact de-quantisation of packed MXFP8 weights for the CPU oracle."""
    wo = {"embed": D.unpack_matrix_mxfp8(wq["embed"], geom.hidden).cpu(), "embed_lookup": w["embed"],
          "final_norm": w["final_norm"], "layers": []}
    for (n1, _, _, n2, _, _), (_, qkv_p, o_p, _, gu_p, down_p) in zip(w["layers"], wq["layers"]):
        wo["layers"].append((n1, D.unpack_matrix_mxfp8(qkv_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(o_p, geom.q_heads * 64).cpu(), n2,
                             D.unpack_matrix_mxfp8(gu_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(down_p, geom.intermediate).cpu()))
    return wo


@pytest.mark.parametrize("name,dims,B,ctxs,mxfp8,block_size", [
    ("gqa3-b4", (192, 512, 2, 3, 1, 1024), 4, [5, 17, 1, 40], False, 16),                             # default routing from 4 requests
    ("mha-b7-mxfp8", (128, 256, 2, 2, 2, 512), 7, [3, 90, 31, 16, 15, 64, 200], True, 16),
    ("gqa3-b9", (192, 512, 2, 3, 1, 1024), 9, [5, 17, 1, 40, 33, 64, 2, 100, 7], False, 16),          # N padded to 16
    ("gqa3-b16", (192, 512, 3, 6, 2, 2048), 16, [37] * 16, False, 16),
    ("mha-b33", (128, 256, 2, 2, 2, 512), 33, [3 + 4 * i for i in range(33)], False, 16),             # N padded to 64, ragged
    ("gqa3-b64", (192, 512, 2, 3, 1, 1024), 64, [20 + (i * 7) % 50 for i in range(64)], False, 16),
    ("gqa3-b64-long", (192, 512, 2, 3, 1, 1024), 64, [1500 if i == 5 else 30 for i in range(64)], False, 16),
    ("gqa3-b16-mxfp8", (192, 512, 3, 3, 1, 1024), 16, [70] * 16, True, 16),
    ("mha-b24-mxfp8-block8", (128, 256, 2, 2, 2, 512), 24, [150 - i for i in range(24)], True, 8),
    ("wide-b16", (960, 2560, 2, 15, 5, 2048), 16, [130] * 16, False, 16),                             # SmolLM2-360M widths
    ("wide17-b2", (2048, 8192, 2, 32, 32, 2048), 2, [30, 61], False, 16),         # SmolLM2-1.7B widths: tensor cores from 2 requests
    ("wide17-b3-mxfp8", (2048, 8192, 2, 32, 32, 2048), 3, [9, 100, 47], True, 16),
])
def test_batched_kernel_against_restatement(cuda_device, name, dims, B, ctxs, mxfp8, block_size):
    from prime_kernels_b200 import decode as D

    geom = D.Geometry(name, *dims, weight_format=1 if mxfp8 else 0)
    w = harness.make_weights(geom, 0, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    wo = w
    if mxfp8:
        wd = D.pack_weights_mxfp8(wd)
        wo = _oracle_weights(D, w, wd, geom)
    cap = max(ctxs) + 40
    cap = (cap + 15) // 16 * 16
    cs = harness.make_cos_sin_cache(geom, cap)
    csd = cs.to(cuda_device)
    gen = torch.Generator().manual_seed(7)
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    keys = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, B, cap, cuda_device, block_size=block_size, shuffle=True)
    for layer in range(geom.layers):
        for b, c in enumerate(ctxs):
            kvb = torch.cat([keys[layer][b], vals[layer][b]], -1).to(cuda_device)
            for t0 in range(0, c, block_size):
                n = min(block_size, c - t0)
                kv.kv_caches[layer][int(kv.block_table[b, t0 // block_size]), :, :n, :] = kvb[:, t0:t0 + n, :]
    for s in range(2):
        pos = torch.tensor([c + s for c in ctxs], dtype=torch.int64)
        lo = torch.zeros(geom.layers, B, geom.hidden, dtype=torch.bfloat16, device=cuda_device)
        hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                         seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                         slot_mapping=kv.slots(pos), embed=wd["embed"], embed_lookup=wd.get("embed_lookup"),
                                         layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                                         cos_sin_cache=csd, eps=geom.eps, layer_outputs=lo, lm_head=True)
        D.check_status(geom, cuda_device)
        rh, rl, rlo = R.decode_step(geom, wo, cur, pos, keys, vals, cs)
        assert (lo.cpu().float() - rlo.float()).abs().max() <= 2 ** -4
        assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4
        # 960-wide rows summed as split-K partial tiles in a run-dependent order: a bf16 ulp more than the toy widths
        tol = 3e-2 if geom.hidden >= 960 else LOGIT_TOL
        assert (logits.cpu().float() - rl).abs().max() <= tol
        margin = rl.topk(2, -1).values
        sure = (margin[:, 0] - margin[:, 1]) > 2 * tol
        assert (nxt.cpu()[sure] == rl.argmax(-1)[sure]).all()
        assert (nxt.cpu() == logits.float().argmax(-1).cpu()).all()          # the kernel's own logits
        for b in range(B):            # the K/V this step appended equals the oracle's (one bf16 ulp)
            got = kv.gather(0, b, ctxs[b] + s + 1)[:, -1, :].cpu().float()
            want = torch.cat([keys[0][b][:, -1, :], vals[0][b][:, -1, :]], -1).float()
            assert (got - want).abs().max() <= 2 ** -5
        cur = rl.argmax(-1)


def test_batched_kernel_agrees_with_micro_batched_launches(cuda_device):
    """The same 20 requests through one tensor-core launch and through three launches of the CUDA-core kernel
    (8 + 8 + 4): logits within the bf16 tolerance, identical appended K/V at layer 0."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("tc-vs-simt", 192, 512, 3, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 3, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 256, cuda_device)
    B, ctx = 20, 90
    outs = []
    for tc in ("force", False):
        kv = harness.PagedKV(geom, B, 256, cuda_device, shuffle=True, seed=1)
        g2 = torch.Generator().manual_seed(5)
        for cache in kv.kv_caches:
            cache.copy_(torch.randn(cache.shape, generator=g2).to(torch.bfloat16))
        pos = torch.full((B,), ctx, dtype=torch.int64)
        ids = torch.arange(B) * 37 % geom.vocab
        hid, logits, nxt = D.decode_step(geom, input_ids=ids.to(cuda_device), positions=pos.to(cuda_device),
                                         seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                         slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                                         final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd,
                                         eps=geom.eps, lm_head=True, tensor_cores=tc)
        D.check_status(geom, cuda_device)
        outs.append((hid.clone(), logits.clone(), [kv.gather(0, b, ctx + 1)[:, -1, :].clone() for b in range(B)]))
    assert (outs[0][1].float() - outs[1][1].float()).abs().max() <= LOGIT_TOL
    assert (outs[0][0].float() - outs[1][0].float()).abs().max() <= 2 ** -4
    for a, b in zip(outs[0][2], outs[1][2]):
        assert torch.equal(a, b)


def test_batched_device_driven_generation_matches_stepwise(cuda_device):
    """advance=True on the batched kernel: ids, positions, sequence lengths and slots of 12 requests are rewritten by
    the kernel; the greedy sequences equal those of a host-driven loop."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("tc-gen", 192, 512, 2, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 5, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 64, cuda_device)
    B, steps = 12, 16
    first = torch.arange(B) * 71 % geom.vocab

    def fresh():
        return harness.PagedKV(geom, B, 64, cuda_device, shuffle=True, seed=3)

    kv_a = fresh()
    sess = D.DecodeSession(geom, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                           kv_caches=kv_a.kv_caches, cos_sin_cache=csd, block_table=kv_a.block_table)
    sess.start(first, torch.zeros(B, dtype=torch.int64))
    ids_a = sess.generate(steps).cpu()
    kv_b = fresh()
    cur, ids_b = first.clone(), []
    for s in range(steps):
        pos = torch.full((B,), s, dtype=torch.int64)
        _, _, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                  seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv_b.block_table,
                                  slot_mapping=kv_b.slots(pos), embed=wd["embed"], layers=wd["layers"],
                                  final_norm=wd["final_norm"], kv_caches=kv_b.kv_caches, cos_sin_cache=csd, eps=geom.eps,
                                  lm_head=True)
        cur = nxt.cpu().clone()
        ids_b.append(cur)
    D.check_status(geom, cuda_device)
    # split-K partial sums meet in a run-dependent order, so an id may differ where two logits tie within rounding;
    # the sequences must agree up to the first such step and the caches written until then must be identical
    ids_b = torch.stack(ids_b)
    same = (ids_a == ids_b).all(dim=1)
    first_diff = int((~same).float().argmax()) if not bool(same.all()) else steps
    assert first_diff >= steps // 2


@pytest.mark.parametrize("B", [1, 3, 6, 20])
def test_vllm_cache_layout_gives_the_same_step(cuda_device, B):
    """The same step on a [blocks, kv_heads, 16, 128] cache and on vLLM's [2, blocks, 16, kv_heads, 64] planes with
    the same contents: every kernel reads the cache through strides (the tensor-core kernel's bulk copies fall back
    to one 128-byte copy per row), so hidden states, logits and the appended rows agree (bit-equal on the CUDA-core
    kernels, within the bf16 tolerance on the tensor-core kernel whose split-K sums meet in a run-dependent order)."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("layouts", 192, 512, 2, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 9, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 256, cuda_device)
    ctx = 77
    kv = harness.PagedKV(geom, B, 256, cuda_device, shuffle=True, seed=2)
    g2 = torch.Generator().manual_seed(4)
    for cache in kv.kv_caches:
        cache.copy_(torch.randn(cache.shape, generator=g2).to(torch.bfloat16))
    # the same contents as K / V planes: [blocks, kvh, bs, 128] -> [2, blocks, bs, kvh, 64]
    planes = [torch.stack([c[..., :64], c[..., 64:]]).permute(0, 1, 3, 2, 4).contiguous() for c in kv.kv_caches]
    pos = torch.full((B,), ctx, dtype=torch.int64, device=cuda_device)
    ids = (torch.arange(B) * 91 % geom.vocab).to(cuda_device)
    outs = []
    for caches in (kv.kv_caches, planes):
        hid, logits, nxt = D.decode_step(geom, input_ids=ids, positions=pos, seq_lens=(pos + 1).to(torch.int32),
                                         block_table=kv.block_table, slot_mapping=kv.slots(pos), embed=wd["embed"],
                                         layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=caches,
                                         cos_sin_cache=csd, eps=geom.eps, lm_head=True)
        D.check_status(geom, cuda_device)
        outs.append((hid.clone(), logits.clone()))
    if B < 4:
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    else:
        assert (outs[0][1].float() - outs[1][1].float()).abs().max() <= LOGIT_TOL
        assert (outs[0][0].float() - outs[1][0].float()).abs().max() <= 2 ** -4
    # the appended row went to the same slot of both layouts
    blk = kv.block_table[:, ctx // 16].long()
    for l in range(geom.layers):
        a = kv.kv_caches[l][blk, :, ctx % 16, :]                                  # [B, kvh, 128]
        b = torch.cat([planes[l][0][blk, ctx % 16], planes[l][1][blk, ctx % 16]], -1)   # [B, kvh, 128]
        if B < 4:
            assert torch.equal(a, b)
        else:
            assert (a.float() - b.float()).abs().max() <= 2 ** -5


def test_alternating_batch_sizes_on_one_workspace(cuda_device):
    """One geometry, one workspace, launches of changing batch size (tensor-core kernel with N = 16 / 32 / 64, CUDA-core
    kernels of batch 1, 2, 3): the tensor-core kernel's fp32 sums must be zero when a launch starts, so its buffers
    may not move with the batch, and the CUDA-core kernels' buffers (whose offsets depend on the kernel batch) are
    re-zeroed when they move.  Every step is checked against the restatement."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("alternate", 192, 512, 2, 3, 1, 1024)
    w = harness.make_weights(geom, 13, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    cs = harness.make_cos_sin_cache(geom, 128)
    csd = cs.to(cuda_device)
    gen = torch.Generator().manual_seed(3)
    for B in (16, 17, 5, 33, 2, 1, 64, 3, 20, 1, 16):
        ctxs = [11 + (7 * b) % 40 for b in range(B)]
        keys = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
        vals = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
        kv = harness.PagedKV(geom, B, 128, cuda_device, shuffle=True, seed=B)
        for layer in range(geom.layers):
            for b, c in enumerate(ctxs):
                kvb = torch.cat([keys[layer][b], vals[layer][b]], -1).to(cuda_device)
                for t0 in range(0, c, 16):
                    n = min(16, c - t0)
                    kv.kv_caches[layer][int(kv.block_table[b, t0 // 16]), :, :n, :] = kvb[:, t0:t0 + n, :]
        cur = torch.randint(0, geom.vocab, (B,), generator=gen)
        pos = torch.tensor(ctxs, dtype=torch.int64)
        hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                         seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                         slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                                         final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd,
                                         eps=geom.eps, lm_head=True)
        D.check_status(geom, cuda_device)
        rh, rl, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        assert (logits.cpu().float() - rl).abs().max() <= LOGIT_TOL, f"batch {B}"
        assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4, f"batch {B}"
