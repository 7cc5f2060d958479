"""GPU parity at the real model sizes the benchmark configurations name: one teacher-forced decode step of
SmolLM2-360M with MXFP8 weights at context 4096 (batch 1, 4, 16) and of the 24-layer SmolLM2-1.7B at context
1024 (batch 1, 8, 16), against the CPU restatement of the rounding points on the same seeded inputs.  Batches
above 8 run on the tensor-core kernel, the others on the CUDA-core kernels; all go through torch.ops -> C ABI.
Contexts are ragged inside a batch and the physical cache blocks are shuffled."""
import functools

import pytest
import torch

from oracle import decode_restatement as R
from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu

# Logit bound.  With random norm weights and N(0,1) K/V these inputs amplify a one-ulp bf16 flip in an early
# layer to ~0.1-0.2 at the logits: the restatement's own two HuggingFace-compatible variants (softmax
# probabilities kept in fp32 or rounded to bf16 before P.V) differ by 0.12 (360M, context 4096) and 0.17 (1.7B,
# context 1024) on them.  That difference is measured on the same inputs and the kernel has to sit as close to the
# restatement as its two variants sit to each other; what pins the arithmetic itself is the first layer (same
# inputs on both sides: attention over the whole context, both GEMV pairs) to a rounding or two, and the
# appended K/V row.
LOGIT_BASE = 2e-2
FLOOR_FACTOR = 1.25


@functools.lru_cache(maxsize=1)
def _weights(name, seed):
    from prime_kernels_b200 import decode as D

    return harness.make_weights(D.GEOMETRIES[name], seed, norm_weights="random")


def _fill_cache(kv, layer, b, k, v):
    """Write request b's prefix ([kv_heads, T, 64] each) into its (shuffled) blocks with one indexed copy."""
    bs = kv.block_size
    T = k.shape[1]
    nblk = (T + bs - 1) // bs
    rows = torch.zeros(k.shape[0], nblk * bs, 128, dtype=torch.bfloat16)
    rows[:, :T, :64] = k
    rows[:, :T, 64:] = v
    blocks = rows.view(k.shape[0], nblk, bs, 128).permute(1, 0, 2, 3).contiguous().to(kv.device)
    kv.kv_caches[layer][kv.block_table[b, :nblk].long()] = blocks


def _one_step(cuda_device, geom, wd, wo, B, ctx, embed_lookup=None):
    from prime_kernels_b200 import decode as D

    gen = torch.Generator().manual_seed(100 + B)
    ctxs = [ctx - 37 * b for b in range(B)]
    cap = (ctx + 16 + 15) // 16 * 16
    cs = harness.make_cos_sin_cache(geom, cap)
    base_k = [torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(geom.layers)]
    base_v = [torch.randn(geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(geom.layers)]
    keys = [[base_k[l][:, :c].clone() for c in ctxs] for l in range(geom.layers)]
    vals = [[base_v[l][:, :c].clone() for c in ctxs] for l in range(geom.layers)]
    kv = harness.PagedKV(geom, B, cap, cuda_device, shuffle=True, seed=B)
    for l in range(geom.layers):
        for b, c in enumerate(ctxs):
            _fill_cache(kv, l, b, keys[l][b], vals[l][b])
    cur = torch.randint(0, geom.vocab, (B,), generator=gen)
    pos = torch.tensor(ctxs, dtype=torch.int64)
    lo = torch.zeros(geom.layers, B, geom.hidden, dtype=torch.bfloat16, device=cuda_device)
    hid, logits, nxt = D.decode_step(geom, input_ids=cur.to(cuda_device), positions=pos.to(cuda_device),
                                     seq_lens=(pos + 1).to(torch.int32).to(cuda_device), block_table=kv.block_table,
                                     slot_mapping=kv.slots(pos), embed=wd["embed"], embed_lookup=embed_lookup,
                                     layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                                     cos_sin_cache=cs.to(cuda_device), eps=geom.eps, layer_outputs=lo, lm_head=True)
    D.check_status(geom, cuda_device)
    keys2 = [[k.clone() for k in layer] for layer in keys]
    vals2 = [[v.clone() for v in layer] for layer in vals]
    rh, rl, rlo = R.decode_step(geom, wo, cur, pos, keys, vals, cs)
    _, rl_b, _ = R.decode_step(geom, wo, cur, pos, keys2, vals2, cs, probs="bf16")
    floor = (rl - rl_b).abs().max().item()
    tol = LOGIT_BASE + FLOOR_FACTOR * floor
    d_logit = (logits.cpu().float() - rl).abs()
    d_first = (lo[0].cpu().float() - rlo[0].float()).abs().max().item()
    d_last = (lo[-1].cpu().float() - rlo[-1].float()).abs().max().item()
    scale_last = rlo[-1].float().abs().max().item()
    margin = rl.topk(2, -1).values
    sure = (margin[:, 0] - margin[:, 1]) > 2 * tol
    print(f"{geom.name} B={B} ctx {ctx}: logits max {d_logit.max().item():.4f} (restatement variants differ by {floor:.4f}) median-of-rows "
          f"{d_logit.amax(-1).median().item():.4f}; residual stream layer 0 {d_first:.4f}, last {d_last:.4f} "
          f"(scale {scale_last:.1f}); ids equal {(nxt.cpu() == rl.argmax(-1)).sum().item()}/{B}")
    assert d_logit.max().item() <= tol
    assert d_first <= 2 ** -6 * max(1.0, rlo[0].float().abs().max().item())      # identical inputs: a rounding or two
    assert d_last <= 2 ** -4 * max(1.0, scale_last)
    assert (nxt.cpu()[sure] == rl.argmax(-1)[sure]).all()
    assert (nxt.cpu() == logits.float().argmax(-1).cpu()).all()
    for b in range(B):          # the K/V row appended at layer 0 (identical inputs) equals the oracle's within a bf16 ulp
        got = kv.gather(0, b, ctxs[b] + 1)[:, -1, :].cpu().float()
        want = torch.cat([keys[0][b][:, -1, :], vals[0][b][:, -1, :]], -1).float()
        assert (got - want).abs().max() <= 2 ** -5


@pytest.mark.parametrize("B", [1, 4, 16])
def test_smollm2_360m_mxfp8_context_4096(cuda_device, B):
    from prime_kernels_b200 import decode as D

    geom = D.GEOMETRIES["smollm2-360m"].with_format(1)
    w = _weights("smollm2-360m", 0)
    wq = D.pack_weights_mxfp8(harness.weights_to(w, cuda_device))
    wo = {"embed": D.unpack_matrix_mxfp8(wq["embed"], geom.hidden).cpu(), "embed_lookup": w["embed"],
          "final_norm": w["final_norm"], "layers": []}
    for (n1, _, _, n2, _, _), (_, qkv_p, o_p, _, gu_p, down_p) in zip(w["layers"], wq["layers"]):
        wo["layers"].append((n1, D.unpack_matrix_mxfp8(qkv_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(o_p, geom.q_heads * 64).cpu(), n2,
                             D.unpack_matrix_mxfp8(gu_p, geom.hidden).cpu(),
                             D.unpack_matrix_mxfp8(down_p, geom.intermediate).cpu()))
    _one_step(cuda_device, geom, wq, wo, B, 4096, embed_lookup=wq["embed_lookup"])


@pytest.mark.parametrize("B", [1, 8, 16])
def test_smollm2_1p7b_context_1024(cuda_device, B):
    from prime_kernels_b200 import decode as D

    geom = D.GEOMETRIES["smollm2-1.7b"]
    w = _weights("smollm2-1.7b", 0)
    wd = harness.weights_to(w, cuda_device)
    _one_step(cuda_device, geom, wd, w, B, 1024)
