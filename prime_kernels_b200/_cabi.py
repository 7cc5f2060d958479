"""Loader for the in-tree shared libraries.

``library()`` returns the ctypes handle of the C ABI (declared in include/prime_kernels_b200.h);
``load_ops()`` loads the torch binding so that ``torch.ops.prime_rmsnorm`` / ``torch.ops.prime_decode``
exist.  Both raise ``RuntimeError`` when the libraries have not been built: there is no fallback.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIBRARY = _PKG / "lib" / "libprime_kernels_b200.so"
BINDING = _PKG / "lib" / "libprime_kernels_b200_torch.so"

_lib = None
_ops_loaded = False

vp, ci, ll, sz, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t, ctypes.c_float
ip = ctypes.POINTER(ctypes.c_int)


class PkDecodeModel(ctypes.Structure):
    _fields_ = [("hidden", ci), ("intermediate", ci), ("layers", ci), ("q_heads", ci), ("kv_heads", ci),
                ("vocab", ci), ("weight_format", ci), ("eps", cf)]


class PkDecodeArgs(ctypes.Structure):
    _fields_ = [("stream", vp), ("batch", ci), ("input_ids", vp), ("ids_i64", ci), ("positions", vp),
                ("seq_lens", vp), ("block_table", vp), ("bt_stride", ci), ("slot_mapping", vp), ("layers", vp),
                ("embed", vp), ("embed_lookup", vp), ("final_norm", vp), ("kv_layers", vp), ("k_off", ll),
                ("v_off", ll), ("block_stride", ll), ("token_stride", ll), ("head_stride", ll), ("block_size", ci),
                ("cos_sin", vp), ("cs_fp32", ci), ("out_hidden", vp), ("logits", vp), ("next_ids", vp),
                ("layer_outputs", vp), ("workspace", vp), ("workspace_bytes", sz), ("max_seq_len", ci),
                ("lm_head", ci), ("advance", ci)]


# name -> (restype, argtypes): every symbol include/prime_kernels_b200.h declares
SYMBOLS = {
    "pk_fused_rmsnorm_residual_forward": (ci, [vp, vp, vp, vp, vp, vp, cf, ci, ci, vp]),
    "pk_fused_rmsnorm_residual_forward_ex": (ci, [vp, vp, vp, vp, vp, vp, vp, cf, ci, ci, ci, vp]),
    "pk_rmsnorm_scale_bytes": (ll, [ci, ci]),
    "pk_rmsnorm_dispatch": (ci, [vp, vp, vp, vp, ci, ci]),
    "pk_rmsnorm_wait_timeouts": (ll, []),
    "pk_apply_rotary": (ci, [vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, vp]),
    "pk_rmsnorm_forward": (ci, [vp, vp, vp, vp, vp, ll, ci, cf, vp]),
    "pk_swiglu_forward": (ci, [vp, vp, vp, ll, ci, ll, ll, vp]),
    "pk_apply_rotary_backward": (ci, [vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, vp]),
    "pk_swiglu_backward": (ci, [vp, vp, vp, vp, vp, ll, ci, ll, ll, vp]),
    "pk_rmsnorm_backward_parts": (ci, [ll]),
    "pk_rmsnorm_backward": (ci, [vp, vp, vp, vp, vp, vp, vp, ll, ci, ctypes.c_float, vp]),
    "pk_mxfp8_packed_row_bytes": (ll, [ci]),
    "pk_pack_weights_mxfp8": (ci, [vp, vp, ll, ci, vp]),
    "pk_pack_weights_mxfp8_ex": (ci, [vp, vp, ll, ci, ci, vp]),
    "pk_decode_workspace_bytes": (sz, [ctypes.POINTER(PkDecodeModel), ci]),
    "pk_decode_step": (ci, [ctypes.POINTER(PkDecodeModel), ctypes.POINTER(PkDecodeArgs)]),
    "pk_decode_step_tc": (ci, [ctypes.POINTER(PkDecodeModel), ctypes.POINTER(PkDecodeArgs)]),
    "pk_decode_step_cc": (ci, [ctypes.POINTER(PkDecodeModel), ctypes.POINTER(PkDecodeArgs)]),
    "pk_decode_set_tc_min_batch": (None, [ci]),
    "pk_decode_step_static": (ci, [ctypes.POINTER(PkDecodeModel), ctypes.POINTER(PkDecodeArgs)]),
    "pk_decode_static_scratch_bytes": (sz, []),
    "pk_decode_static_status": (ci, [vp]),
    "pk_decode_workspace_init": (ci, [vp, sz, vp]),
    "pk_decode_workspace_forget": (None, [vp]),
    "pk_decode_status": (ci, [vp, vp]),
    "pk_decode_query": (ci, [ip] * 7),
    "pk_decode_set_profile": (None, [vp, sz]),
    "pk_status_string": (ctypes.c_char_p, [ci]),
    "pk_decode_set_fast_path": (ci, [ci]),
    "pk_decode_set_spin_limit": (None, [ctypes.c_uint]),
    "pk_decode_wait_probe": (ci, [vp, sz, ctypes.c_uint, vp]),
    "mk_query": (ci, [ip] * 7),
    "mk_workspace_bytes": (sz, [ci, ci]),
    "mk_decode": (ci, [vp, ci, vp, ci, vp, vp, vp, ci, vp, vp, vp, vp, vp, ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, sz, ci]),
    "mk_status_string": (ctypes.c_char_p, [ci]),
    "decode360_workspace_bytes": (sz, []),
    "decode360_debug_bytes": (sz, []),
    "decode360": (ci, [vp, ci, vp, vp, vp, vp, vp, vp, ci, vp, vp, vp, ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, vp, sz,
                       vp, sz, ci, ci]),
    "decode360_status_string": (ctypes.c_char_p, [ci]),
}


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIBRARY.exists():
            raise RuntimeError(f"{LIBRARY} is missing: build it with `python -m prime_kernels_b200._build` "
                               "(there is no CPU fallback)")
        lib = ctypes.CDLL(str(LIBRARY))
        for name, (restype, argtypes) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def load_ops() -> None:
    global _ops_loaded
    if _ops_loaded:
        return
    import torch

    if not BINDING.exists():
        raise RuntimeError(f"{BINDING} is missing: build it with `python -m prime_kernels_b200._build` "
                           "(there is no CPU fallback)")
    library()  # the binding links against the kernel library; load it first so the loader finds it
    torch.ops.load_library(str(BINDING))
    _ops_loaded = True
