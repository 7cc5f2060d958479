"""Batched decode step for SmolLM2-135M on sm_100a (single persistent launch).

Drop-in for the reference package of the same name (prime_kernels/decode_megakernel/__init__.py in the
reference project): same keyword-only ``decode_step`` contract, same exported constants, same error
behaviour (``ValueError`` for contract violations, ``RuntimeError("decode_megakernel failed: ...")``
for a non-zero status).  The kernel is prebuilt in-tree for sm_100a instead of JIT-built for sm_89.

- input_ids int32 or int64 [B]; positions int64 [B]; seq_lens int32 [B] (including the new token);
  slot_mapping int64 [B] (-1 skips the K/V write); block_table int32 [B, W], context limit
  W * block_size <= 8192.
- layers: 30 tuples (input_layernorm, qkv, o, post_attention_layernorm, gate_up, down), BF16 CUDA.
- kv_caches: one BF16 CUDA tensor per layer, [blocks, 3, block_size, 128], K in 0..63, V in 64..127.
- cos_sin_cache BF16 or FP32 [max_pos, 64]; eps must be 1e-5.

The returned tensor is a view of a shared output buffer that the next call overwrites.
"""
import hashlib
from pathlib import Path

from .. import decode as _generic

SOURCE = Path(__file__).resolve().parent.parent / "csrc" / "decode_megakernel.cu"
NVCC_FLAGS = ["-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-lineinfo"]
# The reference pins the sha256 of its kernel source and JIT-builds into a per-user cache directory; this library
# is prebuilt in-tree, so the digest is simply that of the source the library was built from (computed on
# import) and CACHE_ROOT is the directory that holds the built library.
SOURCE_SHA256 = hashlib.sha256(SOURCE.read_bytes()).hexdigest()
CACHE_ROOT = SOURCE.parent.parent / "lib"

GEOMETRY = _generic.SMOLLM2_135M
MAX_BATCH = _generic.MAX_REQUESTS      # one launch takes up to 64 requests (tensor-core kernel from 4 on)
MAX_SEQ = _generic.MAX_SEQ
HIDDEN = GEOMETRY.hidden
KV_HEADS = GEOMETRY.kv_heads
HEAD_DIM = _generic.HEAD_DIM
LAYERS = GEOMETRY.layers
EPS = GEOMETRY.eps


def decode_step(*, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers, final_norm,
                kv_caches, cos_sin_cache, eps, lm_head=False):
    batch = input_ids.shape[0]
    if not 1 <= batch <= MAX_BATCH:      # one launch, like the reference entry
        raise ValueError(f"batch must be 1..{MAX_BATCH}, got {batch}")
    return _generic.decode_step(GEOMETRY, input_ids=input_ids, positions=positions, seq_lens=seq_lens,
                                block_table=block_table, slot_mapping=slot_mapping, embed=embed, layers=layers,
                                final_norm=final_norm, kv_caches=kv_caches, cos_sin_cache=cos_sin_cache, eps=eps,
                                lm_head=lm_head, name="decode_megakernel")
