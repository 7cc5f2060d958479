"""TEST INFRASTRUCTURE (imported only by tests and the comparison scripts they document).

ctypes front end for the reference project's own SmolLM2-135M decode megakernel, compiled for sm_100a from the
reference checkout by oracle/build_ref.sh (oracle/ref_megakernel_wrapper.cu).  ``decode_step`` takes the same
keywords as the reference's Python entry (prime_kernels/decode_megakernel/__init__.py:134-205 in the reference
project) and makes the same ``mk_decode`` call; scratch and output buffers are private to this module.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
LIB = HERE / "_ref" / "libref_megakernel135.so"
MAX_BATCH, MAX_SEQ, HIDDEN, LAYERS = 4, 8192, 576, 30

_lib = None
_state: dict = {}


def available() -> bool:
    return LIB.exists()


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(LIB))
        vp, ci, ll, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t
        lib.mk_workspace_bytes.argtypes = [ci, ci]
        lib.mk_workspace_bytes.restype = sz
        lib.mk_decode.argtypes = [vp, ci, vp, ci, vp, vp, vp, ci, vp, vp, vp, vp, vp,
                                  ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, sz, ci]
        lib.mk_decode.restype = ci
        lib.mk_status_string.argtypes = [ci]
        lib.mk_status_string.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def decode_step(*, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers, final_norm, kv_caches,
                cos_sin_cache, eps=1e-5):
    """One decode step of the reference kernel; returns the final-normed hidden ``[B, 576]`` (a fresh tensor)."""
    lib = library()
    device = input_ids.device
    batch = input_ids.shape[0]
    assert 1 <= batch <= MAX_BATCH and len(layers) == LAYERS and len(kv_caches) == LAYERS and eps == 1e-5
    st = _state.setdefault(device, {})
    if "scratch" not in st:
        st["scratch"] = torch.zeros(lib.mk_workspace_bytes(MAX_BATCH, MAX_SEQ), dtype=torch.uint8, device=device)
        st["out"] = torch.empty((MAX_BATCH, HIDDEN), dtype=torch.bfloat16, device=device)
    # keep the tables alive until the launch has been issued on the current stream
    st["layers_t"] = torch.tensor([[t.data_ptr() for t in layer] for layer in layers], dtype=torch.int64).to(device)
    st["kv_t"] = torch.tensor([kv.data_ptr() for kv in kv_caches], dtype=torch.int64).to(device)
    kv0 = kv_caches[0]
    block_size = kv0.shape[2]
    rc = lib.mk_decode(torch.cuda.current_stream(device).cuda_stream, batch, input_ids.data_ptr(),
                       int(input_ids.dtype == torch.int64), positions.data_ptr(), seq_lens.data_ptr(),
                       block_table.data_ptr(), block_table.stride(0), slot_mapping.data_ptr(), st["layers_t"].data_ptr(),
                       embed.data_ptr(), final_norm.data_ptr(), st["kv_t"].data_ptr(), 0, kv0.shape[3] // 2,
                       kv0.stride(0), kv0.stride(2), kv0.stride(1), block_size, cos_sin_cache.data_ptr(),
                       int(cos_sin_cache.dtype == torch.float32), st["out"].data_ptr(), st["scratch"].data_ptr(),
                       st["scratch"].numel(), block_table.shape[1] * block_size)
    if rc != 0:
        raise RuntimeError(f"reference decode_megakernel failed: {lib.mk_status_string(rc).decode()}")
    return st["out"][:batch].clone()


# ---------------------------------------------------------------- SmolLM2-360M (decode_megakernel_360m)
LIB360 = HERE / "_ref" / "libref_megakernel360.so"
_lib360 = None
_state360: dict = {}


def available_360m() -> bool:
    return LIB360.exists()


def library_360m() -> ctypes.CDLL:
    global _lib360
    if _lib360 is None:
        lib = ctypes.CDLL(str(LIB360))
        vp, ci, ll, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t
        lib.decode360_workspace_bytes.argtypes = []
        lib.decode360_workspace_bytes.restype = sz
        lib.decode360.argtypes = [vp, ci, vp, vp, vp, vp, vp, vp, ci, vp, vp, vp,
                                  ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, vp, sz,
                                  vp, sz, ci, ci]
        lib.decode360.restype = ci
        lib.decode360_status_string.argtypes = [ci]
        lib.decode360_status_string.restype = ctypes.c_char_p
        _lib360 = lib
    return _lib360


def decode_step_360m(*, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers, final_norm, kv_caches,
                     cos_sin_cache, eps=1e-5, layer_outputs=None):
    """One decode step of the reference's packaged 360M kernel (batch 1 or 2, KV block size 16); the call is the one
    prime_kernels/decode_megakernel_360m/__init__.py:186-207 of the reference project makes.  Returns ``[B, 960]``;
    ``layer_outputs`` (optional, bf16 ``[32, B, 960]``) receives the residual stream after every layer."""
    lib = library_360m()
    device = input_ids.device
    batch = input_ids.shape[0]
    assert 1 <= batch <= 2 and len(layers) == 32 and len(kv_caches) == 32 and eps == 1e-5
    kv0 = kv_caches[0]
    assert kv0.shape[1] == 5 and kv0.shape[2] == 16 and kv0.shape[3] == 128
    st = _state360.setdefault(device, {})
    if "scratch" not in st:
        st["scratch"] = torch.zeros(lib.decode360_workspace_bytes(), dtype=torch.uint8, device=device)
        st["out"] = torch.empty((2, 960), dtype=torch.bfloat16, device=device)
    st["ids"] = input_ids.to(torch.int32)
    st["layers_t"] = torch.tensor([[t.data_ptr() for t in layer] for layer in layers], dtype=torch.int64).to(device)
    st["kv_t"] = torch.tensor([kv.data_ptr() for kv in kv_caches], dtype=torch.int64).to(device)
    rc = lib.decode360(torch.cuda.current_stream(device).cuda_stream, batch, st["ids"].data_ptr(), embed.data_ptr(),
                       final_norm.data_ptr(), positions.data_ptr(), seq_lens.data_ptr(), block_table.data_ptr(),
                       block_table.stride(0), slot_mapping.data_ptr(), st["layers_t"].data_ptr(), st["kv_t"].data_ptr(),
                       0, 64, kv0.stride(0), kv0.stride(2), kv0.stride(1), 16, cos_sin_cache.data_ptr(),
                       int(cos_sin_cache.dtype == torch.float32), st["out"].data_ptr(),
                       layer_outputs.data_ptr() if layer_outputs is not None else None, st["scratch"].data_ptr(),
                       st["scratch"].numel(), None, 0, block_table.shape[1] * 16, -1)
    if rc != 0:
        raise RuntimeError(f"reference decode_megakernel_360m failed: {lib.decode360_status_string(rc).decode()}")
    return st["out"][:batch].clone()


# ---------------------------------------------------------------- SmolLM2-360M, fast line (decode_megakernel_360m_lossless)
LIB360F = HERE / "_ref" / "libref_megakernel360f.so"
_lib360f = None
_state360f: dict = {}


def available_360m_fast() -> bool:
    return LIB360F.exists()


def library_360m_fast() -> ctypes.CDLL:
    global _lib360f
    if _lib360f is None:
        lib = ctypes.CDLL(str(LIB360F))
        vp, ci, ll, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t
        lib.decode360_workspace_bytes.argtypes = []
        lib.decode360_workspace_bytes.restype = sz
        lib.decode360_lossless.argtypes = [vp, ci, vp, vp, vp, vp, vp, vp, ci, vp, vp, vp,
                                           ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, vp, sz,
                                           vp, sz, ci, ci, vp]
        lib.decode360_lossless.restype = ci
        lib.decode360_status_string.argtypes = [ci]
        lib.decode360_status_string.restype = ctypes.c_char_p
        _lib360f = lib
    return _lib360f


def decode_step_360m_fast(*, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers, final_norm,
                          kv_caches, cos_sin_cache, eps=1e-5, layer_outputs=None):
    """One decode step of the reference's fast 360M line (batch 1 or 2, KV block size 16) with no encoded gate-up
    table, i.e. on the plain bf16 weights; the call is the one
    prime_kernels/decode_megakernel_360m_lossless/__init__.py of the reference project makes when the lossless
    encoding is not enabled (entry prime_kernels/decode_megakernel_360m_lossless/csrc/block360_kernel.inc:641-716).
    Returns ``[B, 960]``."""
    lib = library_360m_fast()
    device = input_ids.device
    batch = input_ids.shape[0]
    assert 1 <= batch <= 2 and len(layers) == 32 and len(kv_caches) == 32 and eps == 1e-5
    kv0 = kv_caches[0]
    assert kv0.shape[1] == 5 and kv0.shape[2] == 16 and kv0.shape[3] == 128
    st = _state360f.setdefault(device, {})
    if "scratch" not in st:
        st["scratch"] = torch.zeros(lib.decode360_workspace_bytes(), dtype=torch.uint8, device=device)
        st["out"] = torch.empty((2, 960), dtype=torch.bfloat16, device=device)
    st["ids"] = input_ids.to(torch.int32)
    st["layers_t"] = torch.tensor([[t.data_ptr() for t in layer] for layer in layers], dtype=torch.int64).to(device)
    st["kv_t"] = torch.tensor([kv.data_ptr() for kv in kv_caches], dtype=torch.int64).to(device)
    rc = lib.decode360_lossless(torch.cuda.current_stream(device).cuda_stream, batch, st["ids"].data_ptr(),
                                embed.data_ptr(), final_norm.data_ptr(), positions.data_ptr(), seq_lens.data_ptr(),
                                block_table.data_ptr(), block_table.stride(0), slot_mapping.data_ptr(),
                                st["layers_t"].data_ptr(), st["kv_t"].data_ptr(), 0, 64, kv0.stride(0), kv0.stride(2),
                                kv0.stride(1), 16, cos_sin_cache.data_ptr(), int(cos_sin_cache.dtype == torch.float32),
                                st["out"].data_ptr(), layer_outputs.data_ptr() if layer_outputs is not None else None,
                                st["scratch"].data_ptr(), st["scratch"].numel(), None, 0, block_table.shape[1] * 16, -1,
                                None)
    if rc != 0:
        raise RuntimeError(f"reference decode_megakernel_360m_lossless failed: {lib.decode360_status_string(rc).decode()}")
    return st["out"][:batch].clone()
