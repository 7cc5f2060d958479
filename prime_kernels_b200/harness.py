"""Synthetic-model harness for the decode path: seeded random weights in the fused layout the kernel
reads, the rotary cos/sin cache, and a paged KV cache with its vLLM-style metadata.

Used by the tests, the benchmark and the smoke check.  Everything here is plain PyTorch plumbing
(allocation, layout conversion); no model arithmetic happens here.
"""
from __future__ import annotations

import torch

from .geometry import HEAD_DIM, Geometry


def make_weights(geometry: Geometry, seed: int = 0, device="cpu", norm_weights: str = "ones", std: float = 0.02):
    """Random-init weights: Linear/Embedding ~ normal(0, std) in bf16, tied lm_head.

    Draw order (one CPU generator seeded with ``seed``): embed, then per layer q, k, v, o, gate, up,
    down, then (if ``norm_weights == "random"``) all norm weights ~ normal(1, 0.1).
    Returns a dict with ``embed [V,H]``, ``layers`` (list of 6-tuples norm1, qkv, o, norm2, gate_up,
    down) and ``final_norm [H]``, all bf16 on ``device``.
    """
    g = torch.Generator().manual_seed(seed)
    H, I, D = geometry.hidden, geometry.intermediate, HEAD_DIM

    def rnd(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)

    embed = rnd(geometry.vocab, H)
    raw = []
    for _ in range(geometry.layers):
        q = rnd(geometry.q_heads * D, H)
        k = rnd(geometry.kv_heads * D, H)
        v = rnd(geometry.kv_heads * D, H)
        o = rnd(H, geometry.q_heads * D)
        gate = rnd(I, H)
        up = rnd(I, H)
        down = rnd(H, I)
        raw.append((torch.cat([q, k, v], 0).contiguous(), o, torch.cat([gate, up], 0).contiguous(), down))

    def norm():
        if norm_weights == "ones":
            return torch.ones(H, dtype=torch.bfloat16)
        return (1.0 + 0.1 * torch.randn(H, generator=g, dtype=torch.float32)).to(torch.bfloat16)

    layers = []
    for qkv, o, gate_up, down in raw:
        layers.append((norm().to(device), qkv.to(device), o.to(device), norm().to(device), gate_up.to(device),
                       down.to(device)))
    return {"embed": embed.to(device), "layers": layers, "final_norm": norm().to(device)}


def weights_to(weights, device):
    return {"embed": weights["embed"].to(device),
            "layers": [tuple(t.to(device) for t in layer) for layer in weights["layers"]],
            "final_norm": weights["final_norm"].to(device)}


def make_cos_sin_cache(geometry: Geometry, max_pos: int, device="cpu", dtype=torch.bfloat16):
    """``[max_pos, 64]``: cos of the 32 rotary frequencies in columns 0..31, sin in 32..63, computed in
    fp32 as HuggingFace's default rotary embedding does and then cast to ``dtype``."""
    inv_freq = 1.0 / (geometry.rope_theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.int64).float() / HEAD_DIM))
    freqs = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.cat([freqs.cos(), freqs.sin()], dim=1).to(dtype).to(device)


class PagedKV:
    """Paged bf16 KV cache ``[blocks, kv_heads, block_size, 128]`` per layer (K in 0..63, V in 64..127)
    with a block table per request.  ``shuffle`` permutes the physical blocks."""

    def __init__(self, geometry: Geometry, batch: int, capacity: int, device, block_size: int = 16,
                 shuffle: bool = False, seed: int = 0):
        self.geometry, self.batch, self.block_size = geometry, batch, block_size
        self.blocks_per_seq = (capacity + block_size - 1) // block_size
        nblocks = batch * self.blocks_per_seq
        self.kv_caches = [torch.zeros((nblocks, geometry.kv_heads, block_size, 2 * HEAD_DIM), dtype=torch.bfloat16,
                                      device=device) for _ in range(geometry.layers)]
        order = torch.arange(nblocks)
        if shuffle:
            order = order[torch.randperm(nblocks, generator=torch.Generator().manual_seed(seed))]
        self.block_table = order.view(batch, self.blocks_per_seq).to(torch.int32).to(device)
        self.device = device

    def slots(self, positions: torch.Tensor) -> torch.Tensor:
        """Flat cache slot of ``positions [B]`` (int64) for each request."""
        pos = positions.to(self.device, torch.int64)
        rows = torch.arange(self.batch, device=self.device)
        blk = self.block_table[rows, (pos // self.block_size)].to(torch.int64)
        return blk * self.block_size + pos % self.block_size

    def load_prefix(self, keys, values):
        """Write a prefix into the cache: ``keys[l]`` / ``values[l]`` are ``[B, kv_heads, T, 64]``."""
        bs = self.block_size
        for layer, (k, v) in enumerate(zip(keys, values)):
            B, KVH, T, _ = k.shape
            kv = torch.cat([k, v], dim=-1).to(self.device, torch.bfloat16)   # [B, KVH, T, 128]
            for b in range(B):
                for t0 in range(0, T, bs):
                    n = min(bs, T - t0)
                    blk = int(self.block_table[b, t0 // bs])
                    self.kv_caches[layer][blk, :, :n, :] = kv[b, :, t0:t0 + n, :]

    def gather(self, layer: int, b: int, length: int):
        """Read back ``[kv_heads, length, 128]`` of request ``b`` (for parity checks)."""
        bs = self.block_size
        parts = []
        for t0 in range(0, length, bs):
            n = min(bs, length - t0)
            blk = int(self.block_table[b, t0 // bs])
            parts.append(self.kv_caches[layer][blk, :, :n, :])
        return torch.cat(parts, dim=1)
