"""TEST INFRASTRUCTURE: CPU restatement of one decode step with the kernel's rounding points written
out (fp32 arithmetic, explicit bf16 roundings), checked against the HuggingFace eager oracle in
tests/test_oracle_decode.py.

Rounding points follow the reference's HF-parity kernel line
(prime_kernels/decode_megakernel_360m_lossless/csrc/block360.cu:121-166 RMSNorm, :239-255 RoPE;
block360_kernel.inc:166-167 bf16 score then exact 1/8 scale, :403-408 bf16 attention output,
:422-436 O + residual, :487-559 SwiGLU, :566-582 down + residual) which mirror
transformers/models/llama/modeling_llama.py.

Softmax probabilities: HuggingFace eager normalises in fp32 and rounds the probabilities to bf16 before
the P.V product (the reference's strict line does the same,
prime_kernels/decode_megakernel_360m/csrc/block360_kernel.inc:252,311-312,346-347); ``probs="bf16"``
restates that.  ``probs="fp32"`` keeps them in fp32 like the reference's fast line
(prime_kernels/decode_megakernel_360m_lossless/csrc/block360_kernel.inc:166-234) and the CUDA kernel's
split-KV path, which only know un-normalised weights until the chunk partials are merged.
"""
from __future__ import annotations

import torch

HEAD_DIM = 64


def bf(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 to the nearest bf16, keep fp32 storage."""
    return x.to(torch.bfloat16).to(torch.float32)


def rms_norm(x, w, eps):
    s = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return bf(bf(x * s) * w.float())


def rope(x, cos, sin):
    """x [..., 64] fp32 (bf16 values); cos/sin [32] fp32 (bf16 values unless an fp32 cache is used)."""
    c = torch.cat([cos, cos], -1)
    s = torch.cat([sin, sin], -1)
    rot = torch.cat([-x[..., 32:], x[..., :32]], -1)
    return bf(bf(x * c) + bf(rot * s))


@torch.no_grad()
def decode_step(geometry, weights, token_ids, positions, keys, values, cos_sin_cache, probs="fp32"):
    """One decode step on the CPU.

    ``keys[l]`` / ``values[l]``: per-layer lists of per-request tensors ``[kv_heads, T_b, 64]`` (bf16) holding
    the context *before* this token; they are extended in place with the new token's K/V.
    Returns ``(hidden [B,H] bf16 final-normed, logits [B,V] fp32 of bf16 values, layer_outputs [L,B,H])``.
    """
    g = geometry
    B = len(token_ids)
    G = g.q_heads // g.kv_heads
    # input lookup: bf16 embedding rows (kept separately when the tied lm_head matrix is quantised)
    x = weights.get("embed_lookup", weights["embed"])[token_ids].float()      # [B, H]
    cs = cos_sin_cache.float()
    layer_outs = []
    for l, (n1, qkv_w, o_w, n2, gu_w, down_w) in enumerate(weights["layers"]):
        h = rms_norm(x, n1, g.eps)
        qkv = bf(h @ qkv_w.float().T)                             # [B, nqkv]
        qd, kd = g.q_heads * HEAD_DIM, g.kv_heads * HEAD_DIM
        attn = torch.zeros(B, qd)
        for b in range(B):
            pos = int(positions[b])
            cos, sin = cs[pos, :32], cs[pos, 32:]
            q = rope(qkv[b, :qd].view(g.q_heads, HEAD_DIM), cos, sin)
            k = rope(qkv[b, qd:qd + kd].view(g.kv_heads, HEAD_DIM), cos, sin)
            v = qkv[b, qd + kd:].view(g.kv_heads, HEAD_DIM)
            keys[l][b] = torch.cat([keys[l][b].float(), k[:, None, :]], 1).to(torch.bfloat16)
            values[l][b] = torch.cat([values[l][b].float(), v[:, None, :]], 1).to(torch.bfloat16)
            K = keys[l][b].float().repeat_interleave(G, 0)        # [QH, T, 64]
            V = values[l][b].float().repeat_interleave(G, 0)
            sc = bf(torch.einsum("hd,htd->ht", q, K)) * 0.125
            p = torch.softmax(sc, -1)
            if probs == "bf16":
                p = bf(p)
            attn[b] = bf(torch.einsum("ht,htd->hd", p, V)).reshape(-1)
        h1 = bf(x + bf(attn @ o_w.float().T))
        hn = rms_norm(h1, n2, g.eps)
        gu = bf(hn @ gu_w.float().T)
        gate, up = gu[:, :g.intermediate], gu[:, g.intermediate:]
        act = bf(bf(gate / (1.0 + torch.exp(-gate))) * up)
        x = bf(h1 + bf(act @ down_w.float().T))
        layer_outs.append(x.to(torch.bfloat16))
    hidden = rms_norm(x, weights["final_norm"], g.eps)
    logits = bf(hidden @ weights["embed"].float().T)
    return hidden.to(torch.bfloat16), logits, torch.stack(layer_outs)
