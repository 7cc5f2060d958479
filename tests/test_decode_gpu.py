"""GPU parity tests of the decode megakernel (called through torch.ops -> C ABI) against the CPU
oracles: the HuggingFace-eager golden run (committed fixture) and the rounding-point restatement.

Tolerances.  The target is max-abs 2e-2 on bf16 logits and token-exact greedy ids.  Two independent
implementations that round to bf16 at the same places still differ in fp32 summation order, and in
this random-init model a single one-ulp bf16 flip early in the stack grows to a few 1e-2 at the
logits (tests/test_oracle_decode.py measures that floor between two CPU implementations).  The bounds
asserted here sit within 1.5 x of what the kernel measures on a B200: SmolLM2-135M, 64 steps: median
0.018, max 0.023, 86 % of the steps within 2e-2; SmolLM2-360M, 256 steps at context 512-767: median
0.027, max 0.039 (HuggingFace against the CPU restatement: 0.039-0.046).  Greedy ids must be exact
wherever the oracle's top-2 margin exceeds twice the bound.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import decode_restatement as R
from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "decode_135m_b1.npz"
LOGIT_TOL = 2e-2       # north-star tolerance (bf16 logits, max-abs)
LOGIT_HARD = 3.5e-2    # SmolLM2-135M: bound on any step (measured max 0.023)
MIN_FRACTION_WITHIN_TOL = 0.6   # SmolLM2-135M: share of steps within LOGIT_TOL (measured 0.86)
# SmolLM2-360M, 512-token context: two CPU implementations (HuggingFace eager and the restatement) differ by
# 0.039-0.046 in the logits whichever way the softmax probabilities are rounded (tests/test_oracle_decode.py);
# the bound for the kernel is 1.5 x that measured floor.
LOGIT_360M = 7e-2


@pytest.fixture(autouse=True)
def _cuda_core_kernels_up_to_8_requests(cuda_device):
    """This module tests the CUDA-core kernels (1..8 requests per launch); by default batches of 4 or more go to the
    tensor-core kernel, which tests/test_decode_batched_gpu.py and tests/test_decode_real_configs_gpu.py cover."""
    from prime_kernels_b200 import decode as D

    D.set_tensor_core_min_batch(D.MAX_BATCH + 1)
    yield
    D.set_tensor_core_min_batch(0)


def _step(D, geom, wd, kv, csd, cur, pos, lm_head=True, layer_outputs=None):
    dev = kv.device
    out = D.decode_step(geom, input_ids=cur.to(dev), positions=pos.to(dev),
                        seq_lens=(pos + 1).to(torch.int32).to(dev), block_table=kv.block_table,
                        slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                        final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=geom.eps,
                        layer_outputs=layer_outputs, lm_head=lm_head)
    return out


@pytest.mark.parametrize("name,dims,B,ctx,shuffle", [
    ("gqa3-b1", (192, 512, 3, 3, 1, 1024), 1, 5, False),
    ("gqa3-b2-shuffled", (192, 512, 3, 3, 1, 1024), 2, 37, True),
    ("mha-b1", (128, 256, 2, 2, 2, 512), 1, 17, False),
    ("gqa3-b4", (192, 512, 3, 3, 1, 1024), 4, 100, False),
    ("gqa3-b3-ctx1", (192, 512, 2, 6, 2, 2048), 3, 1, False),
    ("gqa3-b1-ctx1000", (192, 512, 2, 3, 1, 1024), 1, 1000, True),
    ("gqa3-b6-padded", (192, 512, 2, 3, 1, 1024), 6, 50, True),
    ("mha-b8", (128, 256, 2, 2, 2, 512), 8, 30, False),
    ("gqa3-b16-two-launches", (192, 512, 2, 3, 1, 1024), 16, 40, True),       # batch 16
    ("gqa3-b19-ragged-groups", (192, 512, 2, 3, 1, 1024), 19, 33, False),     # 8 + 8 + 3 requests
])
def test_small_geometries_against_restatement(cuda_device, name, dims, B, ctx, shuffle):
    from prime_kernels_b200 import decode as D

    geom = D.Geometry(name, *dims)
    w = harness.make_weights(geom, 0, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    cs = harness.make_cos_sin_cache(geom, 1100)
    csd = cs.to(cuda_device)
    gen = torch.Generator().manual_seed(7)
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    keys = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, B, 1040, cuda_device, shuffle=shuffle)
    kv.load_prefix([torch.stack(k) for k in keys], [torch.stack(v) for v in vals])
    for s in range(3):
        pos = torch.full((B,), ctx + s, dtype=torch.int64)
        lo = torch.zeros(geom.layers, B, geom.hidden, dtype=torch.bfloat16, device=cuda_device)
        hid, logits, nxt = _step(D, geom, wd, kv, csd, cur, pos, layer_outputs=lo)
        D.check_status(geom, cuda_device)
        rh, rl, rlo = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        assert (lo.cpu().float() - rlo.float()).abs().max() <= 2 ** -4
        assert (logits.cpu().float() - rl).abs().max() <= LOGIT_TOL
        margin = rl.topk(2, -1).values
        sure = (margin[:, 0] - margin[:, 1]) > 2 * LOGIT_TOL
        assert (nxt.cpu()[sure] == rl.argmax(-1)[sure]).all()
        # the K/V this step appended equals the oracle's (one bf16 ulp)
        for b in range(B):
            got = kv.gather(0, b, ctx + s + 1)[:, -1, :].cpu().float()
            want = torch.cat([keys[0][b][:, -1, :], vals[0][b][:, -1, :]], -1).float()
            assert (got - want).abs().max() <= 2 ** -5
        cur = rl.argmax(-1)


def test_padded_row_skips_the_cache_write(cuda_device):
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("pad", 192, 512, 2, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 1), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 64, cuda_device)
    kv = harness.PagedKV(geom, 2, 64, cuda_device)
    for c in kv.kv_caches:
        c.fill_(0.5)
    before = [c.clone() for c in kv.kv_caches]
    pos = torch.tensor([3, 3])
    slots = kv.slots(pos)
    slots[1] = -1
    D.decode_step(geom, input_ids=torch.tensor([1, 2], device=cuda_device), positions=pos.to(cuda_device),
                  seq_lens=torch.tensor([4, 4], dtype=torch.int32, device=cuda_device), block_table=kv.block_table,
                  slot_mapping=slots, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                  kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=geom.eps)
    D.check_status(geom, cuda_device)
    blk1 = int(kv.block_table[1, 0])
    blk0 = int(kv.block_table[0, 0])
    for c, b in zip(kv.kv_caches, before):
        assert torch.equal(c[blk1], b[blk1])               # request 1 (slot -1): untouched
        assert not torch.equal(c[blk0, :, 3], b[blk0, :, 3])  # request 0: position 3 written
        assert torch.equal(c[blk0, :, :3], b[blk0, :, :3])


@pytest.mark.skipif(not GOLDEN.exists(), reason="golden fixture missing")
def test_smollm2_135m_against_hf_golden(cuda_device):
    """SmolLM2-135M, 32-token seeded prompt, 64 greedy steps, KV capacity 2048, against the committed HuggingFace-eager run."""
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel as MK

    geom = D.SMOLLM2_135M
    z = np.load(GOLDEN)
    wd = harness.weights_to(harness.make_weights(geom, 0), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 2048, cuda_device)
    pk = torch.from_numpy(z["prefill_k"]).view(torch.bfloat16)[:, None]     # [L, 1, KVH, 31, 64]
    pv = torch.from_numpy(z["prefill_v"]).view(torch.bfloat16)[:, None]
    ids = torch.from_numpy(z["ids"])
    sample_idx = torch.from_numpy(z["sample_idx"]).to(cuda_device)
    want_logits = torch.from_numpy(z["sample_logits"])
    want_hidden = torch.from_numpy(z["hidden"]).view(torch.bfloat16).float()

    # teacher-forced: every step fed the oracle's previous id
    kv = harness.PagedKV(geom, 1, 2048, cuda_device)
    kv.load_prefix(list(pk), list(pv))
    cur = torch.from_numpy(z["prompt"])[:, -1]
    dl, dh, agree = [], [], []
    for s in range(64):
        pos = torch.tensor([31 + s])
        hid, logits, nxt = _step(D, geom, wd, kv, csd, cur, pos)
        dl.append((logits[0, sample_idx].float().cpu() - want_logits[s]).abs().max().item())
        dh.append((hid[0].float().cpu() - want_hidden[s]).abs().max().item())
        agree.append(int(nxt[0]) == int(ids[s]))
        cur = ids[s:s + 1]
    D.check_status(geom, cuda_device)
    dl = np.array(dl)
    print(f"135M teacher-forced: logits max-abs median {np.median(dl):.4f} max {dl.max():.4f} "
          f"within {LOGIT_TOL}: {(dl <= LOGIT_TOL).mean():.2f}; hidden max {max(dh):.4f}; ids equal {sum(agree)}/64")
    assert dl.max() <= LOGIT_HARD
    assert (dl <= LOGIT_TOL).mean() >= MIN_FRACTION_WITHIN_TOL
    assert all(agree)                                    # golden top-2 margin >= 0.19 on every step

    # free-running greedy through the drop-in 135M surface + host-side argmax of the final hidden
    kv2 = harness.PagedKV(geom, 1, 2048, cuda_device)
    kv2.load_prefix(list(pk), list(pv))
    sess = D.DecodeSession(geom, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                           kv_caches=kv2.kv_caches, cos_sin_cache=csd, block_table=kv2.block_table)
    sess.start(torch.from_numpy(z["prompt"])[:, -1], torch.tensor([31]))
    got = sess.generate(64)
    assert got[:, 0].cpu().tolist() == ids.tolist()

    # drop-in op: hidden only (reference contract), compared with the lm_head variant's hidden
    kv3 = harness.PagedKV(geom, 1, 2048, cuda_device)
    kv3.load_prefix(list(pk), list(pv))
    pos = torch.tensor([31])
    hid = MK.decode_step(input_ids=torch.from_numpy(z["prompt"])[:, -1].to(cuda_device), positions=pos.to(cuda_device),
                         seq_lens=torch.tensor([32], dtype=torch.int32, device=cuda_device),
                         block_table=kv3.block_table, slot_mapping=kv3.slots(pos), embed=wd["embed"],
                         layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv3.kv_caches,
                         cos_sin_cache=csd, eps=MK.EPS)
    assert hid.shape == (1, MK.HIDDEN)
    assert (hid[0].float().cpu() - want_hidden[0]).abs().max() <= 2 ** -3


def test_mxfp8_weight_packing_is_bit_exact(cuda_device):
    """Packed MXFP8 rows against the CPU oracle's weight quantiser (bytes and scale bytes)."""
    from oracle import mxfp8
    from prime_kernels_b200 import decode as D

    g = torch.Generator().manual_seed(3)
    for rows, k in [(7, 960), (64, 2560), (33, 32), (5, 8192)]:
        w = (torch.randn(rows, k, generator=g) * 0.02).to(torch.bfloat16)
        w[0, :32] = 0                                            # zero group -> scale byte 0
        packed = D.pack_matrix_mxfp8(w.to(cuda_device)).cpu().numpy()
        vals, scales = mxfp8.quantise_weight(w.view(torch.int16).numpy().view(np.uint16))
        assert packed.shape[1] == D.packed_row_bytes(k) and packed.shape[1] % 16 == 0
        assert np.array_equal(packed[:, :k], vals)
        assert np.array_equal(packed[:, k:k + k // 32], scales)
        assert (packed[:, k + k // 32:] == 0).all()
        deq = D.unpack_matrix_mxfp8(torch.from_numpy(packed), k).float()
        assert ((deq - w.float()).abs() <= w.float().abs().view(rows, -1, 32).amax(-1, keepdim=True).expand(-1, -1, 32)
                .reshape(rows, k) * 2 ** -3 + 1e-30).all()


def test_mxfp8_weight_packing_floor_mode_is_bit_exact(cuda_device):
    """The second scale rule (floor: the block-scale rule of the reference's flash_moe kernels, values may saturate)
    against the CPU oracle, and a decode step on weights packed that way against the restatement on their exact
    de-quantisation: the kernels do not care which rule produced the bytes."""
    from oracle import mxfp8
    from prime_kernels_b200 import decode as D

    g = torch.Generator().manual_seed(4)
    saturated = 0
    for rows, k in [(7, 960), (64, 2560), (33, 32)]:
        w = (torch.randn(rows, k, generator=g) * 0.02).to(torch.bfloat16)
        w[0, :32] = 0
        packed = D.pack_matrix_mxfp8(w.to(cuda_device), scale_mode="floor").cpu().numpy()
        vals, scales = mxfp8.quantise_weight(w.view(torch.int16).numpy().view(np.uint16), scale_mode="floor")
        assert np.array_equal(packed[:, :k], vals)
        assert np.array_equal(packed[:, k:k + k // 32], scales)
        saturated += int(((vals & 0x7f) == 0x7e).sum())
        other = D.pack_matrix_mxfp8(w.to(cuda_device)).cpu().numpy()
        assert (packed[:, k:k + k // 32].astype(int) <= other[:, k:k + k // 32].astype(int)).all()     # floor never above round-up
    assert saturated > 0            # groups whose largest value lies in (448, 512) x scale saturate, by design
    geom = D.Geometry("mx-floor", 192, 512, 2, 3, 1, 1024, weight_format=1)
    wts = harness.make_weights(geom, 2, norm_weights="random")
    wq = D.pack_weights_mxfp8(harness.weights_to(wts, cuda_device), scale_mode="floor")
    wo = {"embed": D.unpack_matrix_mxfp8(wq["embed"], geom.hidden).cpu(), "embed_lookup": wts["embed"],
          "final_norm": wts["final_norm"], "layers": []}
    for (n1, _, _, n2, _, _), (_, qkv_p, o_p, _, gu_p, down_p) in zip(wts["layers"], wq["layers"]):
        wo["layers"].append((n1, D.unpack_matrix_mxfp8(qkv_p, geom.hidden).cpu(), D.unpack_matrix_mxfp8(o_p, geom.q_heads * 64).cpu(),
                             n2, D.unpack_matrix_mxfp8(gu_p, geom.hidden).cpu(), D.unpack_matrix_mxfp8(down_p, geom.intermediate).cpu()))
    cs = harness.make_cos_sin_cache(geom, 128)
    ctx = 33
    keys = [[torch.randn(1, ctx, 64, generator=g).to(torch.bfloat16)] for _ in range(geom.layers)]
    vals_ = [[torch.randn(1, ctx, 64, generator=g).to(torch.bfloat16)] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, 1, 64, cuda_device)
    kv.load_prefix([torch.stack(k) for k in keys], [torch.stack(v) for v in vals_])
    cur, pos = torch.tensor([77]), torch.tensor([ctx], dtype=torch.int64)
    hid, logits, _ = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                   seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                   slot_mapping=kv.slots(pos), embed=wq["embed"], embed_lookup=wq["embed_lookup"],
                                   layers=wq["layers"], final_norm=wq["final_norm"], kv_caches=kv.kv_caches,
                                   cos_sin_cache=cs.to(cuda_device), eps=geom.eps, lm_head=True)
    D.check_status(geom, cuda_device)
    rh, rl, _ = R.decode_step(geom, wo, cur, pos, keys, vals_, cs)
    assert (logits.cpu().float() - rl).abs().max() <= LOGIT_TOL
    assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4


@pytest.mark.parametrize("B", [1, 4])
def test_mxfp8_weights_decode_against_restatement(cuda_device, B):
    """MXFP8 weights (E4M3 + E8M0 per 32 along K), bf16 activations and KV: the oracle runs the same step on
    the exactly de-quantised weights."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("mx", 192, 512, 3, 3, 1, 1024, weight_format=1)
    w = harness.make_weights(geom, 0, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    wq = D.pack_weights_mxfp8(wd)
    # oracle weights = exact de-quantisation of the packed bytes
    wo = {"embed": D.unpack_matrix_mxfp8(wq["embed"], geom.hidden).cpu(), "embed_lookup": w["embed"],
          "final_norm": w["final_norm"], "layers": []}
    for (n1, qkv, o, n2, gu, down), (_, qkv_p, o_p, _, gu_p, down_p) in zip(w["layers"], wq["layers"]):
        wo["layers"].append((n1, D.unpack_matrix_mxfp8(qkv_p, geom.hidden).cpu(), D.unpack_matrix_mxfp8(o_p, geom.q_heads * 64).cpu(),
                             n2, D.unpack_matrix_mxfp8(gu_p, geom.hidden).cpu(), D.unpack_matrix_mxfp8(down_p, geom.intermediate).cpu()))
    cs = harness.make_cos_sin_cache(geom, 256)
    gen = torch.Generator().manual_seed(11)
    ctx = 70
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    keys = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, B, 128, cuda_device)
    kv.load_prefix([torch.stack(k) for k in keys], [torch.stack(v) for v in vals])
    for s in range(2):
        pos = torch.full((B,), ctx + s, dtype=torch.int64)
        hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                         seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                         slot_mapping=kv.slots(pos), embed=wq["embed"], embed_lookup=wq["embed_lookup"],
                                         layers=wq["layers"], final_norm=wq["final_norm"], kv_caches=kv.kv_caches,
                                         cos_sin_cache=cs.to(cuda_device), eps=geom.eps, lm_head=True)
        D.check_status(geom, cuda_device)
        rh, rl, _ = R.decode_step(geom, wo, cur, pos, keys, vals, cs)
        assert (logits.cpu().float() - rl).abs().max() <= LOGIT_TOL
        assert (hid.cpu().float() - rh.float()).abs().max() <= 2 ** -4
        cur = rl.argmax(-1)


@pytest.mark.parametrize("case", ["long-context", "fp32-cos-int32-ids", "block8-straddle", "ragged-batch"])
def test_edge_cases_against_restatement(cuda_device, case):
    """Maximum context (two-level merge, 64 chunks), fp32 rotary table with int32 ids, a KV block size that
    makes a 16-position run straddle cache blocks, and a batch whose requests have different lengths."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("edge-" + case, 192, 512, 2, 3, 1, 1024)
    w = harness.make_weights(geom, 2, norm_weights="random")
    wd = harness.weights_to(w, cuda_device)
    gen = torch.Generator().manual_seed(21)
    block_size, cap = 16, 256
    cs_dtype, id_dtype = torch.bfloat16, torch.int64
    if case == "long-context":
        ctxs, cap = [8100], 8192
    elif case == "fp32-cos-int32-ids":
        ctxs, cs_dtype, id_dtype = [40], torch.float32, torch.int32
    elif case == "block8-straddle":
        ctxs, block_size = [150], 8
    else:
        ctxs = [1, 117, 230]
    B = len(ctxs)
    cs = harness.make_cos_sin_cache(geom, cap, dtype=cs_dtype)
    keys = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, c, 64, generator=gen).to(torch.bfloat16) for c in ctxs] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, B, cap, cuda_device, block_size=block_size, shuffle=True)
    for layer in range(geom.layers):                        # ragged prefix: load request by request
        for b, c in enumerate(ctxs):
            kvb = torch.cat([keys[layer][b], vals[layer][b]], -1).to(cuda_device)
            for t0 in range(0, c, block_size):
                n = min(block_size, c - t0)
                kv.kv_caches[layer][int(kv.block_table[b, t0 // block_size]), :, :n, :] = kvb[:, t0:t0 + n, :]
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    for s in range(2):
        pos = torch.tensor([c + s for c in ctxs], dtype=torch.int64)
        hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(id_dtype).to(cuda_device), positions=pos.to(cuda_device),
                                         seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                         slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                                         final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                                         cos_sin_cache=cs.to(cuda_device), eps=geom.eps, lm_head=True)
        D.check_status(geom, cuda_device)
        rh, rl, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        assert (logits.cpu().float() - rl).abs().max() <= LOGIT_TOL
        margin = rl.topk(2, -1).values
        sure = (margin[:, 0] - margin[:, 1]) > 2 * LOGIT_TOL
        assert (nxt.cpu()[sure] == rl.argmax(-1)[sure]).all()
        cur = rl.argmax(-1)


def test_device_driven_generation_matches_stepwise(cuda_device):
    """`advance=True` (ids, positions, seq_lens and slot_mapping rewritten by the kernel) gives the same
    greedy sequence as feeding every step from the host."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("gen", 192, 512, 3, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 5, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 128, cuda_device)
    B, steps = 2, 20
    first = torch.tensor([11, 500])

    def fresh():
        return harness.PagedKV(geom, B, 128, cuda_device, shuffle=True, seed=3)

    kv_a = fresh()
    sess = D.DecodeSession(geom, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                           kv_caches=kv_a.kv_caches, cos_sin_cache=csd, block_table=kv_a.block_table)
    sess.start(first, torch.zeros(B, dtype=torch.int64))
    ids_a = sess.generate(steps).cpu()
    kv_b = fresh()
    cur, ids_b = first.clone(), []
    for s in range(steps):
        pos = torch.full((B,), s, dtype=torch.int64)
        _, _, nxt = _step(D, geom, wd, kv_b, csd, cur, pos)
        cur = nxt.cpu().clone()
        ids_b.append(cur)
    assert torch.equal(ids_a, torch.stack(ids_b))
    for ca, cb in zip(kv_a.kv_caches, kv_b.kv_caches):
        assert torch.equal(ca, cb)


def test_router_drives_the_real_kernel(cuda_device):
    """The caller-side router (decode_backend) on a vLLM-shaped model object: a pure-decode step goes through
    the fused kernel and gives the same hidden state as calling decode_step directly; a mixed step is repaired
    row by row."""
    from types import SimpleNamespace

    from prime_kernels_b200 import decode as D, decode_backend as db, harness

    class FlashAttentionMetadata:
        def __init__(self, **kw):
            self.__dict__.update(kw)

    geom = D.Geometry("router", 192, 512, 2, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 3), cuda_device)
    B, ctx = 3, 21
    kv = harness.PagedKV(geom, B, 64, cuda_device)
    g = torch.Generator().manual_seed(5)
    for cache in kv.kv_caches:
        cache.copy_((torch.randn(cache.shape, generator=g) * 0.5).to(torch.bfloat16))
    snapshot = [c.clone() for c in kv.kv_caches]
    csd = harness.make_cos_sin_cache(geom, 64, cuda_device)
    layers = []
    for i, (n1, qkv, o, n2, gu, dn) in enumerate(wd["layers"]):
        layers.append(SimpleNamespace(
            input_layernorm=SimpleNamespace(weight=n1), post_attention_layernorm=SimpleNamespace(weight=n2),
            self_attn=SimpleNamespace(qkv_proj=SimpleNamespace(weight=qkv), o_proj=SimpleNamespace(weight=o),
                                      attn=SimpleNamespace(kv_cache=kv.kv_caches[i], layer_name=f"l{i}"),
                                      rotary_emb=SimpleNamespace(cos_sin_cache=csd)),
            mlp=SimpleNamespace(gate_up_proj=SimpleNamespace(weight=gu), down_proj=SimpleNamespace(weight=dn))))
    config = SimpleNamespace(hidden_size=192, intermediate_size=512, num_hidden_layers=2, num_attention_heads=3,
                             num_key_value_heads=1, rms_norm_eps=geom.eps, vocab_size=1024, rope_theta=geom.rope_theta)
    model = SimpleNamespace(config=config, layers=layers, aux_hidden_state_layers=(),
                            embed_tokens=SimpleNamespace(weight=wd["embed"]),
                            norm=SimpleNamespace(weight=wd["final_norm"], variance_epsilon=geom.eps))
    ids = torch.tensor([7, 400, 33], device=cuda_device)
    pos = torch.full((B,), ctx, dtype=torch.int64, device=cuda_device)
    meta = FlashAttentionMetadata(max_query_len=1, num_actual_tokens=B,
                                  seq_lens=torch.full((B,), ctx + 1, dtype=torch.int32, device=cuda_device),
                                  block_table=kv.block_table, slot_mapping=kv.slots(pos),
                                  query_start_loc=torch.arange(B + 1, dtype=torch.int32, device=cuda_device))
    db.stats.clear()
    routed = db.route(model, ids, pos, meta).clone()
    assert db.stats["backend_decode"] == 1
    for c, s in zip(kv.kv_caches, snapshot):
        c.copy_(s)
    direct = D.decode_step(db.model_geometry(model), input_ids=ids, positions=pos, seq_lens=meta.seq_lens,
                           block_table=kv.block_table, slot_mapping=meta.slot_mapping, embed=wd["embed"],
                           layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                           cos_sin_cache=csd, eps=geom.eps).clone()
    assert torch.equal(routed, direct)
    # mixed step: request 0 is a 2-token prefill, requests 1 and 2 decode -> rows 2 and 3 are recomputed
    for c, s in zip(kv.kv_caches, snapshot):
        c.copy_(s)
    mixed = FlashAttentionMetadata(max_query_len=2, num_actual_tokens=4, seq_lens=meta.seq_lens, block_table=kv.block_table,
                                   slot_mapping=torch.cat([kv.slots(pos)[:1], kv.slots(pos)]),
                                   query_start_loc=torch.tensor([0, 2, 3, 4], dtype=torch.int32, device=cuda_device))
    ids4 = torch.tensor([1, 7, 400, 33], device=cuda_device)
    pos4 = torch.full((4,), ctx, dtype=torch.int64, device=cuda_device)
    stock = torch.zeros(4, 192, dtype=torch.bfloat16, device=cuda_device)
    fixed = db.repair_mixed_decode(model, D.decode_step, db.model_geometry(model), ids4, pos4, stock, mixed)
    assert torch.equal(fixed[2:], direct[1:]) and fixed[:2].abs().sum() == 0
    D.check_status(db.model_geometry(model), cuda_device)


def test_smollm2_360m_headline_against_hf_golden(cuda_device):
    """The headline configuration (SmolLM2-360M, 512-token seeded prompt, 256 greedy steps).  The prompt goes through the
    kernel token by token (which builds the KV cache), then every decode step is fed the oracle's previous id
    and its logits are compared with the HuggingFace-eager golden run."""
    from prime_kernels_b200 import decode as D

    geom = D.SMOLLM2_360M
    z = np.load(GOLDEN.parent / "decode_360m_b1.npz")
    prompt = torch.from_numpy(z["prompt"])
    ids = torch.from_numpy(z["ids"])
    sample_idx = torch.from_numpy(z["sample_idx"]).to(cuda_device)
    want = torch.from_numpy(z["sample_logits"])
    top_v, top_i = torch.from_numpy(z["top_values"]), torch.from_numpy(z["top_indices"]).to(cuda_device)
    wd = harness.weights_to(harness.make_weights(geom, 0), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 1024, cuda_device)
    kv = harness.PagedKV(geom, 1, 1024, cuda_device)
    for t in range(511):                                   # prefill: positions 0..510
        _step(D, geom, wd, kv, csd, prompt[:, t], torch.tensor([t]))
    cur = prompt[:, -1]
    dl, dt, wrong = [], [], []
    for s in range(256):
        _, logits, nxt = _step(D, geom, wd, kv, csd, cur, torch.tensor([511 + s]))
        dl.append((logits[0, sample_idx].float().cpu() - want[s]).abs().max().item())
        dt.append((logits[0, top_i[s]].float().cpu() - top_v[s]).abs().max().item())
        if int(nxt[0]) != int(ids[s]):
            wrong.append((s, float(top_v[s, 0] - top_v[s, 1])))
        cur = ids[s:s + 1]
    D.check_status(geom, cuda_device)
    dl, dt = np.array(dl), np.array(dt)
    print(f"360M teacher-forced: sampled logits max-abs median {np.median(dl):.4f} max {dl.max():.4f}, top-8 max {dt.max():.4f}, "
          f"within {LOGIT_TOL}: {(dl <= LOGIT_TOL).mean():.2f}; ids differing {wrong}")
    # At this depth and context HuggingFace eager and the CPU restatement already disagree by 0.035-0.046
    # whichever way the softmax probabilities are rounded (tests/test_oracle_decode.py), so the per-step 2e-2
    # target cannot be held; the kernel has to stay on that floor.
    assert max(dl.max(), dt.max()) <= 6e-2            # measured 0.039
    assert np.median(dl) <= 4.1e-2                    # measured 0.027
    # greedy ids are exact wherever the oracle's top-2 margin exceeds twice the observed logit error
    # (the golden run contains one exact top-2 tie, which no independent implementation can be held to)
    assert all(margin <= 2 * max(dl.max(), dt.max()) for _, margin in wrong)
    assert len(wrong) <= 1


def test_smollm2_360m_from_hf_prefill_cache(cuda_device):
    """Same configuration, but the 511-token KV cache is HuggingFace's own prefill cache (computed here on the
    host CPU), so every difference measured is the decode step's own: the kernel's logits against a fresh
    HuggingFace-eager run and against the CPU restatement (same rounding points as the kernel) on the same
    cache, teacher-forced with HuggingFace's ids."""
    from oracle import decode_hf
    from prime_kernels_b200 import decode as D

    geom = D.SMOLLM2_360M
    steps = 6
    w = harness.make_weights(geom, 0)
    prompt = torch.randint(0, geom.vocab, (1, 512), generator=torch.Generator().manual_seed(1234))
    ref = decode_hf.run(geom, w, prompt, steps)
    wd = harness.weights_to(w, cuda_device)
    cs = harness.make_cos_sin_cache(geom, 1024)
    csd = cs.to(cuda_device)
    kv = harness.PagedKV(geom, 1, 1024, cuda_device)
    kv.load_prefix(ref["prefill_k"], ref["prefill_v"])
    keys = [[ref["prefill_k"][l][0].clone()] for l in range(geom.layers)]
    vals = [[ref["prefill_v"][l][0].clone()] for l in range(geom.layers)]
    cur = prompt[:, -1]
    d_hf, d_rs, d_rs_hf = [], [], []
    for s in range(steps):
        pos = torch.tensor([511 + s])
        _, logits, nxt = _step(D, geom, wd, kv, csd, cur, pos)
        got = logits[0].float().cpu()
        d_hf.append((got - ref["logits"][s][0]).abs().max().item())
        if s < 2:                                        # the restatement takes seconds per step at this size
            _, rl, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
            d_rs.append((got - rl[0]).abs().max().item())
            d_rs_hf.append((rl[0] - ref["logits"][s][0]).abs().max().item())
        top = ref["logits"][s][0].topk(2).values
        if top[0] - top[1] > 2 * LOGIT_360M:
            assert int(nxt[0]) == int(ref["ids"][s][0])
        cur = ref["ids"][s]
    D.check_status(geom, cuda_device)
    print(f"360M from HF prefill cache: kernel vs HF {['%.4f' % d for d in d_hf]}; kernel vs restatement "
          f"{['%.4f' % d for d in d_rs]}; restatement vs HF {['%.4f' % d for d in d_rs_hf]}")
    # the kernel is as close to HuggingFace as the CPU restatement of the same rounding points is
    assert max(d_hf) <= LOGIT_360M
    assert max(d_rs) <= LOGIT_360M


def test_against_the_reference_projects_own_135m_kernel(cuda_device):
    """The reference's own SmolLM2-135M megakernel (compiled for this GPU from the reference checkout, its
    sm_89-only device check shimmed: oracle/ref_megakernel_wrapper.cu) and this library on the same device
    inputs: final hidden states and the K/V rows both kernels append, for batch 1..4 at ragged contexts."""
    from oracle import ref_megakernel as REF
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel as MK

    if not REF.available():
        pytest.skip("reference megakernel not built (oracle/build_ref.sh)")
    geom = D.SMOLLM2_135M
    wd = harness.weights_to(harness.make_weights(geom, 0, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 256, cuda_device)
    worst = 0.0
    for B, ctxs in [(1, [31]), (2, [17, 100]), (4, [5, 64, 129, 200])]:
        g = torch.Generator().manual_seed(7 + B)
        kvs = []
        for _ in range(2):                      # identical caches for the two kernels
            kv = harness.PagedKV(geom, B, 256, cuda_device, shuffle=True, seed=3)
            kvs.append(kv)
        for l in range(geom.layers):
            fill = (torch.randn(kvs[0].kv_caches[l].shape, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
            kvs[0].kv_caches[l].copy_(fill)
            kvs[1].kv_caches[l].copy_(fill)
        ids = torch.randint(0, geom.vocab, (B,), generator=g).to(cuda_device)
        pos = torch.tensor(ctxs, dtype=torch.int64, device=cuda_device)
        seq = (pos + 1).to(torch.int32)
        outs = []
        for kv, step in zip(kvs, (REF.decode_step, MK.decode_step)):
            outs.append(step(input_ids=ids, positions=pos, seq_lens=seq, block_table=kv.block_table,
                             slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                             final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=1e-5).float().clone())
        torch.cuda.synchronize()
        diff = (outs[0] - outs[1]).abs().max().item()
        scale = outs[0].abs().max().item()
        worst = max(worst, diff / scale)
        # appended K/V rows (position ctx of every request, every layer)
        kdiff, kdiff0 = 0.0, 0.0
        for l in (0, geom.layers // 2, geom.layers - 1):
            for b in range(B):
                a = kvs[0].gather(l, b, ctxs[b] + 1)[:, -1].float()
                c = kvs[1].gather(l, b, ctxs[b] + 1)[:, -1].float()
                d = (a - c).abs().max().item()
                kdiff = max(kdiff, d)
                if l == 0:
                    kdiff0 = max(kdiff0, d / max(a.abs().max().item(), 1.0))
        print(f"reference kernel vs this library, B={B}: hidden max-abs {diff:.4f} (scale {scale:.2f}), appended K/V max-abs layer 0 (relative) {kdiff0:.4f}, any layer {kdiff:.4f}")
        assert diff <= 2 ** -4 * max(scale, 1.0)
        # layer 0 sees identical inputs: the rows agree to a bf16 rounding or two (the 135M reference rounds RoPE
        # once, this library three times like HF eager); deeper layers carry the usual one-ulp-flip drift
        assert kdiff0 <= 2 ** -6 and kdiff <= 0.125
    D.check_status(geom, cuda_device)


def test_against_the_reference_projects_own_360m_kernel(cuda_device):
    """The reference's packaged SmolLM2-360M kernel (decode_megakernel_360m, the strict-parity line; compiled for
    this GPU like the 135M one) against this library at the headline geometry: batch 1 at context 520 and batch 2
    at ragged contexts."""
    from oracle import ref_megakernel as REF
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel_360m as MK360

    if not REF.available_360m():
        pytest.skip("reference 360M megakernel not built (oracle/build_ref.sh)")
    geom = D.SMOLLM2_360M
    wd = harness.weights_to(harness.make_weights(geom, 0, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 640, cuda_device)
    for B, ctxs in [(1, [520]), (2, [77, 300])]:
        g = torch.Generator().manual_seed(11 + B)
        kvs = [harness.PagedKV(geom, B, 640, cuda_device, shuffle=True, seed=5) for _ in range(2)]
        for l in range(geom.layers):
            fill = (torch.randn(kvs[0].kv_caches[l].shape, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
            kvs[0].kv_caches[l].copy_(fill)
            kvs[1].kv_caches[l].copy_(fill)
        ids = torch.randint(0, geom.vocab, (B,), generator=g).to(cuda_device)
        pos = torch.tensor(ctxs, dtype=torch.int64, device=cuda_device)
        seq = (pos + 1).to(torch.int32)
        outs, streams = [], []
        for kv, step in zip(kvs, (REF.decode_step_360m, MK360.decode_step)):
            lo = torch.zeros((geom.layers, B, geom.hidden), dtype=torch.bfloat16, device=cuda_device)
            outs.append(step(input_ids=ids, positions=pos, seq_lens=seq, block_table=kv.block_table,
                             slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"],
                             final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=1e-5,
                             layer_outputs=lo).float().clone())
            streams.append(lo.float())
        torch.cuda.synchronize()
        # residual stream after every layer: the first layer sees identical inputs and must agree to a rounding
        per_layer = (streams[0] - streams[1]).abs().amax(dim=(1, 2))
        rel0 = per_layer[0].item() / max(streams[0][0].abs().max().item(), 1.0)
        print(f"  residual stream max-abs per layer: first {per_layer[0].item():.4f} (relative {rel0:.4f}), "
              f"middle {per_layer[geom.layers // 2].item():.4f}, last {per_layer[-1].item():.4f}")
        assert rel0 <= 2 ** -6
        diff = (outs[0] - outs[1]).abs().max().item()
        scale = outs[0].abs().max().item()
        kdiff, kdiff0 = 0.0, 0.0
        for l in (0, geom.layers - 1):
            for b in range(B):
                a = kvs[0].gather(l, b, ctxs[b] + 1)[:, -1].float()
                c = kvs[1].gather(l, b, ctxs[b] + 1)[:, -1].float()
                d = (a - c).abs().max().item()
                kdiff = max(kdiff, d)
                if l == 0:
                    kdiff0 = max(kdiff0, d / max(a.abs().max().item(), 1.0))
        print(f"reference 360M kernel vs this library, B={B}: hidden max-abs {diff:.4f} (scale {scale:.2f}), appended K/V max-abs layer 0 (relative) {kdiff0:.4f}, any layer {kdiff:.4f}")
        assert diff <= 2 ** -4 * max(scale, 1.0)
        # layer 0 sees identical inputs: the rows agree to a bf16 rounding or two (the 135M reference rounds RoPE
        # once, this library three times like HF eager); deeper layers carry the usual one-ulp-flip drift
        assert kdiff0 <= 2 ** -6 and kdiff <= 0.125
    D.check_status(geom, cuda_device)


def test_against_the_reference_projects_fast_360m_kernel(cuda_device):
    """The reference's fast SmolLM2-360M line (decode_megakernel_360m_lossless, run on the plain bf16 weights) against
    this library at batch 1, context 520: final hidden states, the residual stream after the first layer and the K/V
    rows both kernels append."""
    from oracle import ref_megakernel as REF
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel_360m as MK360

    if not REF.available_360m_fast():
        pytest.skip("reference fast 360M megakernel not built (oracle/build_ref.sh)")
    geom = D.SMOLLM2_360M
    wd = harness.weights_to(harness.make_weights(geom, 0, norm_weights="random"), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 640, cuda_device)
    B, ctxs = 1, [520]
    g = torch.Generator().manual_seed(21)
    kvs = [harness.PagedKV(geom, B, 640, cuda_device, shuffle=True, seed=5) for _ in range(2)]
    for l in range(geom.layers):
        fill = (torch.randn(kvs[0].kv_caches[l].shape, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
        kvs[0].kv_caches[l].copy_(fill)
        kvs[1].kv_caches[l].copy_(fill)
    ids = torch.randint(0, geom.vocab, (B,), generator=g).to(cuda_device)
    pos = torch.tensor(ctxs, dtype=torch.int64, device=cuda_device)
    seq = (pos + 1).to(torch.int32)
    outs, streams = [], []
    for kv, step in zip(kvs, (REF.decode_step_360m_fast, MK360.decode_step)):
        lo = torch.zeros((geom.layers, B, geom.hidden), dtype=torch.bfloat16, device=cuda_device)
        outs.append(step(input_ids=ids, positions=pos, seq_lens=seq, block_table=kv.block_table,
                         slot_mapping=kv.slots(pos), embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                         kv_caches=kv.kv_caches, cos_sin_cache=csd, eps=1e-5, layer_outputs=lo).float().clone())
        streams.append(lo.float())
    torch.cuda.synchronize()
    per_layer = (streams[0] - streams[1]).abs().amax(dim=(1, 2))
    rel0 = per_layer[0].item() / max(streams[0][0].abs().max().item(), 1.0)
    diff = (outs[0] - outs[1]).abs().max().item()
    scale = outs[0].abs().max().item()
    a = kvs[0].gather(0, 0, ctxs[0] + 1)[:, -1].float()
    c = kvs[1].gather(0, 0, ctxs[0] + 1)[:, -1].float()
    kdiff0 = (a - c).abs().max().item() / max(a.abs().max().item(), 1.0)
    print(f"reference fast 360M kernel vs this library: hidden max-abs {diff:.4f} (scale {scale:.2f}), residual stream after "
          f"layer 0 (relative) {rel0:.4f}, last {per_layer[-1].item():.4f}, appended K/V layer 0 (relative) {kdiff0:.4f}")
    assert rel0 <= 2 ** -6
    assert diff <= 2 ** -4 * max(scale, 1.0)
    assert kdiff0 <= 2 ** -6
    D.check_status(geom, cuda_device)


def test_same_box_timing_against_the_reference_kernels(cuda_device):
    """Step time of the reference project's own kernels (24-CTA sm_89 designs, compiled for this GPU) and of this
    library on the same box and the same inputs: SmolLM2-135M batch 1 at context 64 and SmolLM2-360M batch 1 at
    context 520 (CUDA events around 40 back-to-back steps at a fixed position)."""
    from oracle import ref_megakernel as REF
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel as MK
    from prime_kernels_b200 import decode_megakernel_360m as MK360

    if not (REF.available() and REF.available_360m()):
        pytest.skip("reference megakernels not built (oracle/build_ref.sh)")
    cases = [(D.SMOLLM2_135M, 64, REF.decode_step, MK.decode_step, "decode_megakernel"),
             (D.SMOLLM2_360M, 520, REF.decode_step_360m, MK360.decode_step, "decode_megakernel_360m (strict parity)")]
    if REF.available_360m_fast():
        cases.append((D.SMOLLM2_360M, 520, REF.decode_step_360m_fast, MK360.decode_step,
                      "decode_megakernel_360m_lossless (fast line, no encoded gate-up table)"))
    for geom, ctx, ref_step, my_step, label in cases:
        wd = harness.weights_to(harness.make_weights(geom, 0), cuda_device)
        csd = harness.make_cos_sin_cache(geom, 640, cuda_device)
        kv = harness.PagedKV(geom, 1, 640, cuda_device)
        for cache in kv.kv_caches:
            cache.normal_()
        ids = torch.tensor([17], device=cuda_device)
        pos = torch.tensor([ctx], dtype=torch.int64, device=cuda_device)
        seq = (pos + 1).to(torch.int32)
        kw = dict(input_ids=ids, positions=pos, seq_lens=seq, block_table=kv.block_table, slot_mapping=kv.slots(pos),
                  embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                  cos_sin_cache=csd, eps=1e-5)
        times = []
        for step in (ref_step, my_step):
            for _ in range(5):
                step(**kw)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(40):
                step(**kw)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 40 * 1e3)
        print(f"{geom.name} B=1 ctx {ctx}: reference {label} {times[0]:.0f} us/step, this library {times[1]:.0f} us/step "
              f"({times[0] / times[1]:.1f}x)")
        assert times[1] < times[0]
    D.check_status(D.SMOLLM2_360M, cuda_device)


@pytest.mark.parametrize("graph", [True, False])
def test_host_driven_step_matches_device_driven_generation(cuda_device, graph):
    """decode.HostStep (inputs from pinned host buffers, one packed copy, optionally a captured CUDA graph) produces
    the same greedy ids as the device-driven session on the same prefix."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("host", 192, 512, 3, 3, 1, 1024)
    wd = harness.weights_to(harness.make_weights(geom, 2), cuda_device)
    csd = harness.make_cos_sin_cache(geom, 128, cuda_device)
    B, ctx, steps = 2, 19, 6
    kvs = [harness.PagedKV(geom, B, 128, cuda_device, shuffle=True, seed=1) for _ in range(2)]
    g = torch.Generator().manual_seed(4)
    for l in range(geom.layers):
        fill = (torch.randn(kvs[0].kv_caches[l].shape, generator=g) * 0.5).to(torch.bfloat16).to(cuda_device)
        kvs[0].kv_caches[l].copy_(fill)
        kvs[1].kv_caches[l].copy_(fill)
    first = torch.tensor([5, 900])
    sess = D.DecodeSession(geom, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                           kv_caches=kvs[0].kv_caches, cos_sin_cache=csd, block_table=kvs[0].block_table)
    sess.start(first, torch.full((B,), ctx, dtype=torch.int64))
    want = sess.generate(steps).cpu()
    step = D.HostStep(geom, B, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                      kv_caches=kvs[1].kv_caches, cos_sin_cache=csd, block_table=kvs[1].block_table, graph=graph)
    bt = kvs[1].block_table.cpu()
    cur, got = first.clone(), []
    for t in range(steps):
        pos = ctx + t
        nxt = step(cur, torch.full((B,), pos, dtype=torch.int64), torch.full((B,), pos + 1, dtype=torch.int32),
                   bt[:, pos // 16].to(torch.int64) * 16 + pos % 16)
        got.append(nxt.clone())
        cur = nxt.clone()
    assert torch.equal(torch.stack(got), want)
    D.check_status(geom, cuda_device)
    # the numpy entry (inputs written straight into the pinned staging buffer) on a fresh copy of the cache
    kv3 = harness.PagedKV(geom, B, 128, cuda_device, shuffle=True, seed=1)
    g3 = torch.Generator().manual_seed(4)
    for l in range(geom.layers):
        kv3.kv_caches[l].copy_((torch.randn(kv3.kv_caches[l].shape, generator=g3) * 0.5).to(torch.bfloat16).to(cuda_device))
    step3 = D.HostStep(geom, B, embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                       kv_caches=kv3.kv_caches, cos_sin_cache=csd, block_table=kv3.block_table, graph=graph)
    bt3 = kv3.block_table.cpu().numpy().astype("int64")
    cur3, got3 = first.numpy().copy(), []
    for t in range(steps):
        pos = ctx + t
        nxt = step3.step_numpy(cur3, pos, pos + 1, bt3[:, pos // 16] * 16 + pos % 16)
        got3.append(torch.from_numpy(nxt.copy()))
        cur3[:] = nxt
    assert torch.equal(torch.stack(got3), want)
    D.check_status(geom, cuda_device)


def test_wide_geometry_falls_back_to_smaller_launch_groups(cuda_device):
    """A geometry whose 8-request activation staging does not fit shared memory (SmolLM2-1.7B's widths, two layers):
    the step runs as launches of 4 requests and still matches the restatement (SmolLM2-1.7B widths, batch 8)."""
    from prime_kernels_b200 import decode as D

    geom = D.Geometry("wide", 2048, 8192, 2, 32, 32, 2048, rope_theta=130000.0)
    w = harness.make_weights(geom, 0)
    wd = harness.weights_to(w, cuda_device)
    cs = harness.make_cos_sin_cache(geom, 128)
    B, ctx = 8, 20
    gen = torch.Generator().manual_seed(3)
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    keys = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    vals = [[torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(B)] for _ in range(geom.layers)]
    kv = harness.PagedKV(geom, B, 64, cuda_device)
    kv.load_prefix([torch.stack(k) for k in keys], [torch.stack(v) for v in vals])
    pos = torch.full((B,), ctx, dtype=torch.int64)
    hid, logits, nxt = _step(D, geom, wd, kv, cs.to(cuda_device), cur, pos)
    D.check_status(geom, cuda_device)
    assert D._runtime(geom, torch.device(cuda_device)).group < D.MAX_BATCH
    rh, rl, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
    # 2048- and 8192-long dot products: the summation-order noise is larger than on the small geometries
    wide_tol = 5e-2
    assert (logits.cpu().float() - rl).abs().max() <= wide_tol
    margin = rl.topk(2, -1).values
    sure = (margin[:, 0] - margin[:, 1]) > 2 * wide_tol
    assert (nxt.cpu()[sure] == rl.argmax(-1)[sure]).all()

