"""SmolLM2-360M fused decode step on sm_100a (single persistent launch).

Drop-in for the reference package of the same name (prime_kernels/decode_megakernel_360m/__init__.py in
the reference project): same keyword-only contract including ``layer_outputs``, ``debug`` and
``debug_layer_index``, same constants, same validation.  ``debug`` is accepted and left untouched (the
stage dump is not produced).

The returned tensor is a view into a shared per-device output buffer and is overwritten by the next
call on that device.  Consume or copy it before then.
"""
import hashlib
from pathlib import Path

import torch

from .. import decode as _generic

SOURCE = Path(__file__).resolve().parent.parent / "csrc" / "decode_megakernel.cu"
NVCC_FLAGS = ["-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-lineinfo"]
# The reference pins the sha256 of its kernel source and JIT-builds into a per-user cache directory; this library
# is prebuilt in-tree, so the digest is simply that of the source the library was built from (computed on
# import) and CACHE_ROOT is the directory that holds the built library.
SOURCE_SHA256 = hashlib.sha256(SOURCE.read_bytes()).hexdigest()
INCLUDE_SHA256 = hashlib.sha256((SOURCE.parent / "decode_fast.cuh").read_bytes()).hexdigest()
CACHE_ROOT = SOURCE.parent.parent / "lib"

GEOMETRY = _generic.SMOLLM2_360M
MAX_BATCH = _generic.MAX_REQUESTS      # one launch takes up to 64 requests (tensor-core kernel from 4 on)
MAX_SEQ = _generic.MAX_SEQ
HIDDEN = GEOMETRY.hidden
INTERMEDIATE = GEOMETRY.intermediate
LAYERS = GEOMETRY.layers
KV_HEADS = GEOMETRY.kv_heads
HEAD_DIM = _generic.HEAD_DIM
BLOCK_SIZE = 16
EPS = GEOMETRY.eps


def _check_tensor(tensor, name, *, dtype=None, device=None, shape=None):
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if dtype is not None and tensor.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}")
    if device is not None and tensor.device != device:
        raise ValueError(f"{name} must be on {device}")
    if shape is not None and tuple(tensor.shape) != shape:
        raise ValueError(f"{name} must have shape {shape}")


def decode_step(*, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers, final_norm,
                kv_caches, cos_sin_cache, eps, layer_outputs=None, debug=None, debug_layer_index=-1,
                lm_head=False):
    """Run one 360M decode step; inputs follow vLLM FLASH_ATTN metadata."""
    batch = input_ids.shape[0]
    if not 1 <= batch <= MAX_BATCH:
        raise ValueError(f"batch must be 1..{MAX_BATCH}, got {batch}")
    if eps != EPS:
        raise ValueError(f"the kernel is built for rms eps {EPS}, got {eps}")
    if len(layers) != LAYERS or len(kv_caches) != LAYERS:
        raise ValueError(f"expected {LAYERS} layers and KV caches")
    if debug_layer_index < -1 or debug_layer_index >= LAYERS:
        raise ValueError("debug_layer_index must be -1 or a layer index 0..31")
    device = input_ids.device
    _check_tensor(input_ids, "input_ids", device=device)
    if input_ids.dtype not in (torch.int32, torch.int64) or input_ids.ndim != 1:
        raise ValueError("input_ids must be a 1-D int32 or int64 tensor")
    _check_tensor(positions, "positions", dtype=torch.int64, device=device, shape=(batch,))
    _check_tensor(seq_lens, "seq_lens", dtype=torch.int32, device=device, shape=(batch,))
    _check_tensor(slot_mapping, "slot_mapping", dtype=torch.int64, device=device, shape=(batch,))
    if block_table.dtype != torch.int32 or block_table.device != device or block_table.ndim != 2 \
            or block_table.shape[0] < batch:
        raise ValueError("block_table must be int32 [B, width] on the input device")
    if block_table.stride(1) != 1:
        raise ValueError("block_table must have contiguous rows")
    if not 1 <= block_table.shape[1] * BLOCK_SIZE <= MAX_SEQ:
        raise ValueError(f"block_table context capacity must be 1..{MAX_SEQ}")
    _check_tensor(embed, "embed", dtype=torch.bfloat16, device=device)
    _check_tensor(final_norm, "final_norm", dtype=torch.bfloat16, device=device, shape=(HIDDEN,))
    if embed.ndim != 2 or embed.shape[1] != HIDDEN:
        raise ValueError("embed must be BF16 [vocab, 960]")
    expected = ((HIDDEN,), (HIDDEN + 2 * KV_HEADS * HEAD_DIM, HIDDEN), (HIDDEN, HIDDEN), (HIDDEN,),
                (2 * INTERMEDIATE, HIDDEN), (HIDDEN, INTERMEDIATE))
    for i, layer in enumerate(layers):
        if len(layer) != 6:
            raise ValueError(f"layer {i} must contain six weight tensors")
        for nm, tensor, shape in zip(("norm1", "qkv", "o", "norm2", "gate_up", "down"), layer, expected):
            _check_tensor(tensor, f"layer {i} {nm}", dtype=torch.bfloat16, device=device, shape=shape)
            if not tensor.is_contiguous():
                raise ValueError(f"layer {i} {nm} must be contiguous")
    kv0 = kv_caches[0]
    _check_tensor(kv0, "kv_caches[0]", dtype=torch.bfloat16, device=device)
    if kv0.ndim != 4 or kv0.shape[1] != KV_HEADS or kv0.shape[3] != 2 * HEAD_DIM or kv0.stride(3) != 1:
        raise ValueError("KV caches must use vLLM FLASH_ATTN [blocks, 5, 16, 128] K/V-packed layout")
    if kv0.shape[2] != BLOCK_SIZE:
        raise ValueError("the kernel requires KV block_size=16")
    for i, kv in enumerate(kv_caches):
        _check_tensor(kv, f"kv_caches[{i}]", dtype=torch.bfloat16, device=device, shape=tuple(kv0.shape))
        if kv.stride() != kv0.stride():
            raise ValueError("all KV caches must share strides")
    _check_tensor(cos_sin_cache, "cos_sin_cache", device=device)
    if cos_sin_cache.dtype not in (torch.bfloat16, torch.float32) or cos_sin_cache.ndim != 2 \
            or cos_sin_cache.shape[1] != HEAD_DIM:
        raise ValueError("cos_sin_cache must be BF16 or FP32 [max_position, 64]")
    if layer_outputs is not None:
        _check_tensor(layer_outputs, "layer_outputs", dtype=torch.bfloat16, device=device,
                      shape=(LAYERS, batch, HIDDEN))
        if not layer_outputs.is_contiguous():
            raise ValueError("layer_outputs must be contiguous")
    if debug is not None:
        _check_tensor(debug, "debug", dtype=torch.uint8, device=device)
        if not debug.is_contiguous():
            raise ValueError("debug must be contiguous raw byte storage")
        if debug.data_ptr() % 16:
            raise ValueError("debug buffer must be 16-byte aligned")
    return _generic.decode_step(GEOMETRY, input_ids=input_ids, positions=positions, seq_lens=seq_lens,
                                block_table=block_table, slot_mapping=slot_mapping, embed=embed, layers=layers,
                                final_norm=final_norm, kv_caches=kv_caches, cos_sin_cache=cos_sin_cache, eps=eps,
                                layer_outputs=layer_outputs, lm_head=lm_head, name="decode_megakernel_360m")
